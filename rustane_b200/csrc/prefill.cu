// Host side of the batched prompt pass: workspace, TMA tensor maps, and the per-layer
// sequence of tensor-core GEMMs (prefill.cuh).  Restates the naive forward of the reference
// (full_model.rs:336-437 and layer.rs:1287-1431) for the prompt positions only, with the
// residual stream in fp32 and 16-bit GEMM inputs; K and V go straight into the pages the
// decode kernels read.  Used by cd_prefill for bf16 / fp16 models on one GPU; every other
// case keeps feeding the prompt one token at a time.
#include "prefill.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "kernels.cuh"
#include "model.h"

namespace cd {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct SampleGraphKey {
    int ns = 0, mode = 0, top_k = 0;
    float t = 0.f, softcap = 0.f;
    int split = 0;
    int len0 = -1;  // the prompt length the graphs were captured for: the number of shared prompt tokens is a launch argument
    bool operator==(const SampleGraphKey& o) const {
        return ns == o.ns && mode == o.mode && top_k == o.top_k && t == o.t && softcap == o.softcap && split == o.split && len0 == o.len0;
    }
};

struct PrefillCtx {
    EncodeTiledFn encode = nullptr;
    SampleGraphKey s_key;
    std::map<int, cudaGraphExec_t> s_graphs;  // captured multi-sample steps by number of occupied attention slices
    uint64_t s_graph_nodes = 0;
    std::vector<CUtensorMap> w_qkv, w_o, w_13, w_2, k_pages;  // per layer, built once
    CUtensorMap w_head;
    std::vector<CUtensorMap> sk_qkv, sk_o, sk_13, sk_2;  // the same matrices in 128-row boxes (multi-sample decode)
    CUtensorMap sk_head;
    // FP8 linears: one layer's four matrices widened to 16 bits before its GEMMs (the maps of every layer view these)
    void *f8_qkv = nullptr, *f8_o = nullptr, *f8_13 = nullptr, *f8_2 = nullptr;
    // multi-sample decode workspace (one arena, sized for s_cap samples)
    int s_cap = 0;
    char* s_arena = nullptr;
    float *sx = nullptr, *sq = nullptr, *sattn = nullptr, *slogits = nullptr, *spart_acc = nullptr, *spart_ml = nullptr;
    float* sksum = nullptr;  // [8 K slices][16][dim] partial sums of the linears that are cut along K
    float *sblock_vals = nullptr, *stopk_vals = nullptr, *smaxes = nullptr, *ssums = nullptr;
    uint32_t *sblock_idxs = nullptr, *stopk_idxs = nullptr, *sout_token = nullptr, *sring = nullptr;
    unsigned int *scounters = nullptr, *shead_counters = nullptr;
    void *sxn = nullptr, *sgate = nullptr;  // [2][s_cap][...] hi, lo
    DevState* sst = nullptr;
    // workspace (grow-only)
    size_t rows = 0, key_ld = 0;
    float* x = nullptr;       // [rows][dim] residual stream
    void* xn = nullptr;       // [2][rows][max(dim, q_dim)] normalised input / attention output (hi, lo)
    void* q = nullptr;        // [2][rows][q_dim]
    void* gate = nullptr;     // [2][rows][hidden]
    float* s = nullptr;       // [heads][rows][key_ld]
    void* p = nullptr;        // [2][heads][rows][key_ld]
    void* vt = nullptr;       // [kv_heads * hd][key_ld]
};

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool encode_2d(PrefillCtx* c, CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows,
               uint64_t row_bytes, uint32_t box_rows) {
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)PF_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return c->encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the K half of one layer's pages as {d, token in page, kv head, k|v, page}; a box is 128 keys of one head
bool encode_k_pages(PrefillCtx* c, CUtensorMap* map, CUtensorMapDataType dt, const void* base, int hd, int page_tokens, int kv_heads,
                    int num_pages) {
    const cuuint64_t dims[5] = {(cuuint64_t)hd, (cuuint64_t)page_tokens, (cuuint64_t)kv_heads, 2, (cuuint64_t)num_pages};
    const cuuint64_t e = 2;
    const cuuint64_t strides[4] = {hd * e, (cuuint64_t)page_tokens * hd * e, (cuuint64_t)kv_heads * page_tokens * hd * e,
                                   (cuuint64_t)2 * kv_heads * page_tokens * hd * e};
    const cuuint32_t box[5] = {(cuuint32_t)PF_BK, (cuuint32_t)page_tokens, 1, 1, (cuuint32_t)(128 / page_tokens)};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return c->encode(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// instruction descriptor of tcgen05.mma kind::f16: fp32 accumulate, both operands K-major, M = 128
inline uint32_t make_idesc(int bn, bool bf16) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(PF_BM >> 4) << 24);
}

template <int BN, bool SPLIT, class Epi>
cudaError_t pf_launch_t(cd_model* m, const CUtensorMap& a, const CUtensorMap& a_lo, const CUtensorMap& b, const PfGemm& p, bool bf16, int zdim,
                        const Epi& epi) {
    auto kern = pf_gemm_kernel<BN, SPLIT, Epi>;
    static bool attr_set = false;  // per instantiation
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PfTile<BN, SPLIT>::SMEM);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const dim3 grid((p.N + BN - 1) / BN, (p.M + PF_BM - 1) / PF_BM, zdim);
    kern<<<grid, PF_THREADS, PfTile<BN, SPLIT>::SMEM, m->stream>>>(a, a_lo, b, p, make_idesc(BN, bf16), epi);
    m->launches++;
    return cudaGetLastError();
}

// a: the activation's hi and lo maps (lo unused when split is off)
template <int BN, class Epi>
cudaError_t pf_launch(cd_model* m, bool split, const CUtensorMap (&a)[2], const CUtensorMap& b, const PfGemm& p, bool bf16, int zdim, const Epi& epi) {
    return split ? pf_launch_t<BN, true>(m, a[0], a[1], b, p, bf16, zdim, epi) : pf_launch_t<BN, false>(m, a[0], a[0], b, p, bf16, zdim, epi);
}

// the few-rows GEMM: w in 128-row boxes, x = the [NB][K] activation block (hi rows, then lo rows)
template <int NB, class Epi>
cudaError_t sk_launch_t(cd_model* m, const CUtensorMap& w, const CUtensorMap& x, int N, int K, int ns, bool bf16,
                        const Epi& epi, int kslices) {
    auto kern = pf_skinny_kernel<NB, Epi>;
    static bool attr_set = false;  // per instantiation
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SkTile<NB>::SMEM);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((N + 127) / 128, kslices);
    lc.blockDim = dim3(PF_THREADS);
    lc.dynamicSmemBytes = SkTile<NB>::SMEM;
    lc.stream = m->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel fetches weights before it waits for its predecessor
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = m->pdl ? 1 : 0;
    m->launches++;
    return cudaLaunchKernelEx(&lc, kern, w, x, N, K, ns, make_idesc(NB, bf16), &m->st->error, epi);
}
template <class Epi>
cudaError_t sk_launch(cd_model* m, bool split, const CUtensorMap& w, const CUtensorMap& x, int N, int K, int ns, bool bf16,
                      const Epi& epi, int kslices = 1) {
    return split ? sk_launch_t<32>(m, w, x, N, K, ns, bf16, epi, kslices) : sk_launch_t<16>(m, w, x, N, K, ns, bf16, epi, kslices);
}

// weights, LM head and K pages: maps built once per model
int ensure_weight_maps(cd_model* m, PrefillCtx* c, CUtensorMapDataType dt, CUtensorMapDataType kdt) {
    if (!c->w_qkv.empty()) return CD_OK;
    const cd_config& cf = m->cfg;
    const int D = cf.dim, Q = cf.q_dim, KV = cf.kv_dim, H = cf.hidden;
    c->w_qkv.resize(cf.nlayers); c->w_o.resize(cf.nlayers); c->w_13.resize(cf.nlayers); c->w_2.resize(cf.nlayers); c->k_pages.resize(cf.nlayers);
    c->sk_qkv.resize(cf.nlayers); c->sk_o.resize(cf.nlayers); c->sk_13.resize(cf.nlayers); c->sk_2.resize(cf.nlayers);
    bool ok = encode_2d(c, &c->w_head, dt, m->lm_head, D, m->v_loc, (uint64_t)D * 2, 256) &&
              encode_2d(c, &c->sk_head, dt, m->lm_head, D, m->v_loc, (uint64_t)D * 2, 128);
    if (m->opt.weight_dtype == CD_DTYPE_FP8_E4M3) {
        const size_t n_qkv = (size_t)(Q + 2 * KV) * D, n_o = (size_t)D * Q, n_13 = (size_t)2 * H * D, n_2 = (size_t)D * H;
        if (cudaMalloc(&c->f8_qkv, n_qkv * 2) != cudaSuccess || cudaMalloc(&c->f8_o, n_o * 2) != cudaSuccess ||
            cudaMalloc(&c->f8_13, n_13 * 2) != cudaSuccess || cudaMalloc(&c->f8_2, n_2 * 2) != cudaSuccess) {
            c->w_qkv.clear();
            return fail(m, CD_ERR_CUDA, "prompt-pass buffers for the widened FP8 matrices");
        }
        for (int l = 0; l < cf.nlayers && ok; ++l) {
            ok = ok && encode_2d(c, &c->w_qkv[l], dt, c->f8_qkv, D, Q + 2 * KV, (uint64_t)D * 2, 256);
            ok = ok && encode_2d(c, &c->w_o[l], dt, c->f8_o, Q, D, (uint64_t)Q * 2, 256);
            ok = ok && encode_2d(c, &c->w_13[l], dt, c->f8_13, D, 2 * H, (uint64_t)D * 2, 256);
            ok = ok && encode_2d(c, &c->w_2[l], dt, c->f8_2, H, D, (uint64_t)H * 2, 256);
            ok = ok && encode_k_pages(c, &c->k_pages[l], kdt, m->layers[l].kv, cf.hd, m->page_tokens, cf.kv_heads, m->num_pages);
        }
        if (!ok) { c->w_qkv.clear(); return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for a weight matrix"); }
        return CD_OK;
    }
    for (int l = 0; l < cf.nlayers && ok; ++l) {
        const cd_layer_dev& L = m->layers[l];
        ok = ok && encode_2d(c, &c->sk_qkv[l], dt, L.wqkv, D, Q + 2 * KV, (uint64_t)D * 2, 128);
        ok = ok && encode_2d(c, &c->sk_o[l], dt, L.wo, Q, D, (uint64_t)Q * 2, 128);
        ok = ok && encode_2d(c, &c->sk_13[l], dt, L.w13, D, 2 * H, (uint64_t)D * 2, 128);
        ok = ok && encode_2d(c, &c->sk_2[l], dt, L.w2, H, D, (uint64_t)H * 2, 128);
        ok = ok && encode_2d(c, &c->w_qkv[l], dt, L.wqkv, D, Q + 2 * KV, (uint64_t)D * 2, 256);
        ok = ok && encode_2d(c, &c->w_o[l], dt, L.wo, Q, D, (uint64_t)Q * 2, 256);
        ok = ok && encode_2d(c, &c->w_13[l], dt, L.w13, D, 2 * H, (uint64_t)D * 2, 256);
        ok = ok && encode_2d(c, &c->w_2[l], dt, L.w2, H, D, (uint64_t)H * 2, 256);
        ok = ok && encode_k_pages(c, &c->k_pages[l], kdt, L.kv, cf.hd, m->page_tokens, cf.kv_heads, m->num_pages);
    }
    if (!ok) { c->w_qkv.clear(); return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for a weight matrix"); }
    return CD_OK;
}

// the context of a model the tensor-core passes can serve, or CD_ERR_UNSUPPORTED
int get_ctx(cd_model* m, PrefillCtx** out, bool fp8_ok, bool tp_ok = false) {
    const cd_config& cf = m->cfg;
    const int dt = m->opt.weight_dtype;
    if (dt != CD_DTYPE_BF16 && dt != CD_DTYPE_F16 && !(fp8_ok && dt == CD_DTYPE_FP8_E4M3)) return CD_ERR_UNSUPPORTED;
    // tensor parallel: the prompt pass only (the ranks' partial products meet in the link region's buffers)
    if (m->tp_world > 1 && (!tp_ok || m->tp_pf_rows == 0 || dt == CD_DTYPE_FP8_E4M3)) return CD_ERR_UNSUPPORTED;
    if (cf.dim % 32 || cf.q_dim % 32 || cf.hidden % 16 || (cf.hd != 64 && cf.hd != 128)) return CD_ERR_UNSUPPORTED;
    if (m->page_tokens > 128 || 128 % m->page_tokens) return CD_ERR_UNSUPPORTED;
    PrefillCtx* c = (PrefillCtx*)m->prefill_ctx;
    if (!c) {
        c = new PrefillCtx();
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            delete c;
            return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        }
        c->encode = (EncodeTiledFn)fn;
        m->prefill_ctx = c;
    }
    *out = c;
    return CD_OK;
}

// T16: the 16-bit type of the weights and of the linears' activation operands; KT: the type of the KV
// cache, which the attention GEMMs' other operands (q, the probabilities, V transposed) share.
template <typename T16, typename KT>
int run(cd_model* m, PrefillCtx* c, size_t n, bool split) {
    const cd_config& cf = m->cfg;
    const bool bf16 = std::is_same<T16, __nv_bfloat16>::value, kbf16 = std::is_same<KT, __nv_bfloat16>::value;
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapDataType kdt = kbf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int D = cf.dim, Q = cf.q_dim, KV = cf.kv_dim, H = cf.hidden, hd = cf.hd;
    const int pos0 = (int)m->len, M = (int)n, nkeys = pos0 + M;
    auto cuda_fail = [&](const char* what, cudaError_t e) { return fail(m, CD_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); };

    int rc = ensure_weight_maps(m, c, dt, kdt);
    if (rc) return rc;
    // ---- workspace
    const size_t rows = round_up(n, PF_BM), key_ld = round_up((size_t)nkeys, 128);
    if (rows > c->rows || key_ld > c->key_ld) {
        for (void* ptr : {(void*)c->x, c->xn, c->q, c->gate, (void*)c->s, c->p, c->vt}) if (ptr) cudaFree(ptr);
        c->x = nullptr; c->xn = c->q = c->gate = c->p = c->vt = nullptr; c->s = nullptr;
        const size_t r = std::max(rows, c->rows), k = std::max(key_ld, c->key_ld);
        c->rows = c->key_ld = 0;
        struct { void** ptr; size_t bytes; } want[] = {
            {(void**)&c->x, r * D * 4}, {&c->xn, 2 * r * (size_t)std::max(D, Q) * 2}, {&c->q, 2 * r * (size_t)Q * 2}, {&c->gate, 2 * r * (size_t)H * 2},
            {(void**)&c->s, (size_t)cf.heads * r * k * 4}, {&c->p, 2 * (size_t)cf.heads * r * k * 2}, {&c->vt, (size_t)cf.kv_heads * hd * k * 2}};
        for (auto& w : want) {
            cudaError_t e = cudaMalloc(w.ptr, w.bytes);
            if (e == cudaSuccess) e = cudaMemsetAsync(*w.ptr, 0, w.bytes, m->stream);
            if (e != cudaSuccess) return cuda_fail("prefill workspace", e);
        }
        c->rows = r; c->key_ld = k;
    }
    const size_t R = c->rows, KL = c->key_ld, plane = R * KL;
    // hi matrices first, lo matrices (split mode) in the second half of each buffer
    T16* xn = (T16*)c->xn; KT* qb = (KT*)c->q; T16* gate = (T16*)c->gate; KT* pm = (KT*)c->p; KT* vt = (KT*)c->vt;
    T16* xn_lo = split ? xn + R * (size_t)std::max(D, Q) : nullptr;
    KT* q_lo = split ? qb + R * (size_t)Q : nullptr;
    T16* gate_lo = split ? gate + R * (size_t)H : nullptr;
    KT* p_lo = split ? pm + (size_t)cf.heads * plane : nullptr;
    CUtensorMap a_xn[2], a_attn[2], a_gate[2], a_q[2], a_p[2], b_vt;
    bool ok = encode_2d(c, &b_vt, kdt, c->vt, KL, (uint64_t)cf.kv_heads * hd, (uint64_t)KL * 2, (uint32_t)hd);
    for (int h = 0; h < (split ? 2 : 1) && ok; ++h) {
        ok = encode_2d(c, &a_xn[h], dt, h ? xn_lo : xn, D, R, (uint64_t)D * 2, PF_BM) && encode_2d(c, &a_attn[h], dt, h ? xn_lo : xn, Q, R, (uint64_t)Q * 2, PF_BM) &&
             encode_2d(c, &a_gate[h], dt, h ? gate_lo : gate, H, R, (uint64_t)H * 2, PF_BM) && encode_2d(c, &a_q[h], kdt, h ? q_lo : qb, Q, R, (uint64_t)Q * 2, PF_BM) &&
             encode_2d(c, &a_p[h], kdt, h ? p_lo : pm, KL, (uint64_t)cf.heads * R, (uint64_t)KL * 2, PF_BM);
    }
    if (!ok) return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for an activation buffer");

    cudaError_t e;
#define PF_TRY(what, x) do { e = (x); if (e != cudaSuccess) return cuda_fail(what, e); } while (0)
    pf_embed_kernel<T16><<<M, 256, 0, m->stream>>>((const T16*)m->embed, m->prompt_dev, c->x, D);
    m->launches++;
    // tensor parallel: Wo and W2 are split along their input, so their products are partial sums that the ranks exchange
    // through two alternating buffers of the link region (prefill.cuh, tp_pf_reduce_kernel)
    const bool tpar = m->tp_world > 1;
    const size_t pf_flags = TpRegion::pf_flags_off(m->tp_world, D, m->tp_nb), pf_bufs = TpRegion::pf_buf_off(m->tp_world, D, m->tp_nb);
    if (tpar && rows > m->tp_pf_rows) return fail(m, CD_ERR_CAPACITY, "prompt chunk longer than the tensor-parallel partial-sum buffers");
    auto tp_buf = [&]() { return reinterpret_cast<float*>(m->link_region + pf_bufs + (size_t)((m->tp_pf_seq + 1) & 1u) * m->tp_pf_rows * D * 4); };
    auto tp_allreduce = [&]() {
        m->tp_pf_seq += 1;
        const int buf = (int)(m->tp_pf_seq & 1u);
        tp_pf_publish_kernel<<<1, 32, 0, m->stream>>>(m->tp, pf_flags, buf, m->tp_pf_seq);
        tp_pf_reduce_kernel<<<m->sm_count * 4, 256, 0, m->stream>>>(m->tp, pf_flags, pf_bufs, buf, m->tp_pf_seq, c->x, M, m->tp_pf_rows, m->alpha,
                                                                   &m->st->error);
        m->launches += 2;
        return cudaGetLastError();
    };
    PfGemm g = {};
    g.b_zdiv = 1; g.page_tokens = m->page_tokens; g.pos0 = pos0; g.err = &m->st->error;
    const float scale = 1.0f / std::sqrt((float)hd);
    const bool fp8 = m->opt.weight_dtype == CD_DTYPE_FP8_E4M3;
    auto quantised = [&](PfGemm& p, const void* rows, int K) {  // the GEMM's output columns take the FP8 row scales
        if (!fp8) return;
        p.qrows = (const unsigned char*)rows; p.qstride = Wfmt<Fp8Row>::row_stride(K); p.qscale_off = Wfmt<Fp8Row>::scale_off(K);
    };
    for (int l = 0; l < cf.nlayers; ++l) {
        const cd_layer_dev& L = m->layers[l];
        if (fp8) {  // this layer's e4m3 values as 16-bit matrices (exact); the previous layer's GEMMs are done with the buffers (stream order)
            const int wb = m->sm_count * 8;
            pf_widen_fp8_kernel<T16><<<wb, 256, 0, m->stream>>>((const unsigned char*)L.wqkv, Wfmt<Fp8Row>::row_stride(D), (T16*)c->f8_qkv, Q + 2 * KV, D);
            pf_widen_fp8_kernel<T16><<<wb, 256, 0, m->stream>>>((const unsigned char*)L.wo, Wfmt<Fp8Row>::row_stride(Q), (T16*)c->f8_o, D, Q);
            pf_widen_fp8_kernel<T16><<<wb, 256, 0, m->stream>>>((const unsigned char*)L.w13, Wfmt<Fp8Row>::row_stride(D), (T16*)c->f8_13, 2 * H, D);
            pf_widen_fp8_kernel<T16><<<wb, 256, 0, m->stream>>>((const unsigned char*)L.w2, Wfmt<Fp8Row>::row_stride(H), (T16*)c->f8_2, D, H);
            m->launches += 4;
        }
        pf_rmsnorm_kernel<T16><<<M, 256, 0, m->stream>>>(c->x, L.gamma1, xn, xn_lo, D);
        m->launches++;
        {   // q, k, v = xn Wqkv with RoPE; k and v into the pages
            PfGemm p = g; p.M = M; p.N = Q + 2 * KV; p.K = D;
            quantised(p, L.wqkv, D);
            PfEpiQKV<KT> epi{qb, q_lo, (KT*)L.kv, m->page_table, m->rope, Q, KV, hd, cf.kv_heads, m->page_tokens, pos0};
            PF_TRY("qkv gemm", (pf_launch<256>(m, split, a_xn, c->w_qkv[l], p, bf16, 1, epi)));
        }
        pf_transpose_v_kernel<KT><<<dim3((unsigned)(KL / 64), cf.kv_heads), 256, 0, m->stream>>>((const KT*)L.kv, m->page_table, vt, nkeys, (int)KL,
                                                                                                 cf.kv_heads, hd, m->page_tokens);
        m->launches++;
        {   // scores = q k^T per head over the cached keys (tiles above the diagonal skipped)
            PfGemm p = g; p.M = M; p.N = nkeys; p.K = hd; p.a_col_z = hd; p.b_zdiv = cf.gqa_ratio; p.b_paged = 1; p.causal = 1;
            PF_TRY("score gemm", (pf_launch<128>(m, split, a_q, c->k_pages[l], p, kbf16, cf.heads, PfEpiScores{c->s, plane, (int)KL})));
        }
        pf_softmax_kernel<KT><<<dim3(M, cf.heads), 256, 0, m->stream>>>(c->s, pm, p_lo, plane, (int)KL, pos0, scale);
        m->launches++;
        {   // attention output = P V per head (the K loop stops at the diagonal)
            PfGemm p = g; p.M = M; p.N = hd; p.K = nkeys; p.a_row_z = (int)R; p.b_row_z = hd; p.b_zdiv = cf.gqa_ratio; p.causal = 2;
            PfEpiAttnOut<T16> epi{xn, xn_lo, Q, hd};
            if (hd == 128) PF_TRY("pv gemm", (pf_launch<128>(m, split, a_p, b_vt, p, kbf16, cf.heads, epi)));
            else PF_TRY("pv gemm", (pf_launch<64>(m, split, a_p, b_vt, p, kbf16, cf.heads, epi)));
        }
        {   // x2 = x + alpha * (attn Wo)
            PfGemm p = g; p.M = M; p.N = D; p.K = Q;
            quantised(p, L.wo, Q);
            if (tpar) {
                PF_TRY("wo gemm", (pf_launch<256>(m, split, a_attn, c->w_o[l], p, bf16, 1, PfEpiPartial{tp_buf(), D})));
                PF_TRY("wo all-reduce", tp_allreduce());
            } else {
                PF_TRY("wo gemm", (pf_launch<256>(m, split, a_attn, c->w_o[l], p, bf16, 1, PfEpiResidual{c->x, D, m->alpha})));
            }
        }
        pf_rmsnorm_kernel<T16><<<M, 256, 0, m->stream>>>(c->x, L.gamma2, xn, xn_lo, D);
        m->launches++;
        {   // gate = act(x2n W1) * (x2n W3)
            PfGemm p = g; p.M = M; p.N = 2 * H; p.K = D;
            quantised(p, L.w13, D);
            PF_TRY("w13 gemm", (pf_launch<256>(m, split, a_xn, c->w_13[l], p, bf16, 1, PfEpiGate<T16>{gate, gate_lo, H, m->opt.activation})));
        }
        {   // x = x2 + alpha * (gate W2^T)
            PfGemm p = g; p.M = M; p.N = D; p.K = H;
            quantised(p, L.w2, H);
            if (tpar) {
                PF_TRY("w2 gemm", (pf_launch<256>(m, split, a_gate, c->w_2[l], p, bf16, 1, PfEpiPartial{tp_buf(), D})));
                PF_TRY("w2 all-reduce", tp_allreduce());
            } else {
                PF_TRY("w2 gemm", (pf_launch<256>(m, split, a_gate, c->w_2[l], p, bf16, 1, PfEpiResidual{c->x, D, m->alpha})));
            }
        }
    }
    // the last prompt position's hidden state, where the LM-head GEMV expects it
    PF_TRY("copy last row", cudaMemcpyAsync(m->x_a, c->x + (size_t)(M - 1) * D, (size_t)D * 4, cudaMemcpyDeviceToDevice, m->stream));
#undef PF_TRY
    return CD_OK;
}

// ---------------------------------------------------------------- several samples per step
// `--samples N` sharing a prompt (inference.rs:255-297 runs them one after the other): all N
// continuations advance together, one token each per step, so every weight byte is read once
// per step for all of them.  The linears are the prompt-pass GEMMs with one row per sample;
// attention, head reductions and samplers are the single-sample kernels, run per sample on that
// sample's state, so each sample's draws are those of its own sequential loop.
template <typename T16, typename KT>
int run_samples(cd_model* m, PrefillCtx* c, const uint32_t* first, int ns, size_t nsteps, int mode, int top_k, float t, float softcap,
                uint64_t* rng, uint32_t* out_ids, bool split) {
    const cd_config& cf = m->cfg;
    const bool bf16 = std::is_same<T16, __nv_bfloat16>::value;
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapDataType kdt = std::is_same<KT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int D = cf.dim, Q = cf.q_dim, KV = cf.kv_dim, H = cf.hidden, hd = cf.hd, V = m->v_loc, NB = m->nblocks;
    const int Vp = (V + 31) & ~31;  // row stride of the logits: the GEMM epilogue writes whole 32-column chunks
    const int pps = m->pages_per_seq, pt = m->page_tokens, len0 = (int)m->len, ring_ld = cf.seq + 1;
    auto cuda_fail = [&](const char* what, cudaError_t e) { return fail(m, CD_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); };
    int rc = ensure_weight_maps(m, c, dt, kdt);
    if (rc) return rc;
    cudaError_t e;
#define PF_TRY(what, x) do { e = (x); if (e != cudaSuccess) return cuda_fail(what, e); } while (0)
    if (ns > c->s_cap) {
        if (c->s_arena) cudaFree(c->s_arena);
        c->s_arena = nullptr; c->s_cap = 0;
        const size_t S = SK_ROWS, W = (size_t)std::max(D, Q);  // blocks of 16 rows: hi parts, then lo parts
        size_t off = 0;
        auto carve = [&](size_t bytes) { const size_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
        const size_t o_x = carve(S * D * 4), o_q = carve(S * Q * 4), o_attn = carve(S * Q * 4), o_logits = carve(S * Vp * 4);
        const size_t o_pacc = carve(S * cf.heads * m->nsplit * hd * 4), o_pml = carve(S * cf.heads * m->nsplit * 2 * 4);
        const size_t o_cnt = carve(S * cf.heads * 4), o_hcnt = carve(S * 4);
        const size_t o_bv = carve(S * NB * 4), o_bi = carve(S * NB * 4), o_tv = carve(S * NB * CD_MAX_GPU_TOPK * 4), o_ti = carve(S * NB * CD_MAX_GPU_TOPK * 4);
        const size_t o_mx = carve(S * NB * 4), o_sm = carve(S * NB * 4), o_tok = carve(S * 64), o_ring = carve(S * ring_ld * 4);
        const size_t o_xn = carve(2 * S * W * 2), o_gate = carve(2 * S * H * 2), o_st = carve(S * sizeof(DevState));
        const size_t o_ks = carve(8 * S * D * 4);
        PF_TRY("sample workspace", cudaMalloc((void**)&c->s_arena, off));
        PF_TRY("sample workspace", cudaMemsetAsync(c->s_arena, 0, off, m->stream));
        char* b = c->s_arena;
        c->sx = (float*)(b + o_x); c->sq = (float*)(b + o_q); c->sattn = (float*)(b + o_attn); c->slogits = (float*)(b + o_logits);
        c->spart_acc = (float*)(b + o_pacc); c->spart_ml = (float*)(b + o_pml); c->scounters = (unsigned int*)(b + o_cnt);
        c->shead_counters = (unsigned int*)(b + o_hcnt); c->sblock_vals = (float*)(b + o_bv); c->sblock_idxs = (uint32_t*)(b + o_bi);
        c->stopk_vals = (float*)(b + o_tv); c->stopk_idxs = (uint32_t*)(b + o_ti); c->smaxes = (float*)(b + o_mx); c->ssums = (float*)(b + o_sm);
        c->sout_token = (uint32_t*)(b + o_tok); c->sring = (uint32_t*)(b + o_ring); c->sxn = b + o_xn; c->sgate = b + o_gate;
        c->sst = (DevState*)(b + o_st);
        c->sksum = (float*)(b + o_ks);
        c->s_cap = (int)S;
    }
    const size_t S = (size_t)c->s_cap, W = (size_t)std::max(D, Q);
    T16* xn = (T16*)c->sxn; T16* gate = (T16*)c->sgate;
    // the lo block starts 16 rows into the buffer, in rows of whatever width the buffer currently holds
    T16* xn_lo = split ? xn + S * (size_t)D : nullptr;
    T16* attn_lo = split ? xn + S * (size_t)Q : nullptr;
    T16* gate_lo = split ? gate + S * (size_t)H : nullptr;
    // one map per activation buffer: rows 0-15 the hi parts, rows 16-31 the lo parts
    const uint32_t xrows = split ? 2 * SK_ROWS : SK_ROWS;
    CUtensorMap a_xn, a_attn, a_gate;
    const bool ok = encode_2d(c, &a_xn, dt, xn, D, xrows, (uint64_t)D * 2, xrows) && encode_2d(c, &a_attn, dt, xn, Q, xrows, (uint64_t)Q * 2, xrows) &&
                    encode_2d(c, &a_gate, dt, gate, H, xrows, (uint64_t)H * 2, xrows);
    if (!ok) return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for an activation buffer");

    // page tables: prompt pages that are full are shared, the page the prompt ends in is copied, later pages are the sample's own
    std::vector<int> table((size_t)ns * pps);
    for (int s = 0; s < ns; ++s)
        for (int j = 0; j < pps; ++j) table[(size_t)s * pps + j] = (s == 0 || (j + 1) * pt <= len0) ? j : s * pps + j;
    PF_TRY("page tables", cudaMemcpyAsync(m->page_table, table.data(), table.size() * 4, cudaMemcpyHostToDevice, m->stream));
    PF_TRY("page tables", cudaStreamSynchronize(m->stream));  // the host vector goes away
    if (len0 % pt) {
        const int jp = len0 / pt;
        const size_t page_bytes = (size_t)2 * cf.kv_heads * pt * hd * sizeof(KT);
        for (int l = 0; l < cf.nlayers; ++l)
            for (int s = 1; s < ns; ++s)
                PF_TRY("prompt page copy", cudaMemcpyAsync((char*)m->layers[l].kv + ((size_t)s * pps + jp) * page_bytes,
                                                           (char*)m->layers[l].kv + (size_t)jp * page_bytes, page_bytes, cudaMemcpyDeviceToDevice, m->stream));
    }
    for (int s = 0; s < ns; ++s) {
        begin_loop_kernel<<<1, 1, 0, m->stream>>>(c->sst + s, len0, first[s], rng ? rng[s] : 0ull);
        m->launches++;
    }
    PF_TRY("sample states", cudaGetLastError());
    PF_TRY("event", cudaEventRecord(m->ev0, m->stream));

    const float scale = 1.0f / std::sqrt((float)hd);
    const float inv_t = 1.0f / std::max(t, 1.17549435e-38f);  // decode.rs:174
    const int split_blocks = (int)std::min<size_t>(256, ((size_t)ns * Q + 255) / 256);
    // one step of all samples; everything that changes from step to step is read on the device, except the
    // number of attention slices that hold keys (`nsp`), which selects the captured graph
    auto enqueue_step = [&](int nsp) -> int {
        pf_embed_samples_kernel<T16><<<ns, 256, 0, m->stream>>>((const T16*)m->embed, c->sst, c->sx, D, m->full_cfg.vocab);
        m->launches++;
        // Wo and W2 have few output rows: they are cut along K into `ks` slices and the following
        // RMSNorm kernel adds the slices' partial sums (in slice order) into the residual stream
        const int ks = std::max(1, std::min(8, m->sm_count / ((D + 127) / 128)));
        const int nthreads = std::min(1024, std::max(256, D / 4 / 32 * 32));
        for (int l = 0; l < cf.nlayers; ++l) {
            const cd_layer_dev& L = m->layers[l];
            if (l == 0) pf_rmsnorm_kernel<T16><<<ns, 256, 0, m->stream>>>(c->sx, L.gamma1, xn, xn_lo, D);
            else pf_reduce_rmsnorm_kernel<T16><<<ns, nthreads, 0, m->stream>>>(c->sx, c->sksum, ks, m->alpha, L.gamma1, xn, xn_lo, D);
            {
                SkEpiQKV<KT> epi{c->sq, (KT*)L.kv, m->page_table, m->rope, c->sst, Q, KV, hd, cf.kv_heads, pt, pps};
                PF_TRY("qkv gemm", sk_launch(m, split, c->sk_qkv[l], a_xn, Q + 2 * KV, D, ns, bf16, epi));
            }
            // two samples per attention CTA share each K/V tile of the prompt pages (measured best of 1, 2, 4, 8)
            const dim3 agrid(cf.heads, nsp, (ns + 1) / 2);
            const int shared_tokens = len0 / pt * pt;
            if (hd == 128)
                attn_decode_group_kernel<KT, 128, 2><<<agrid, 128, 0, m->stream>>>(c->sq, (const KT*)L.kv, m->page_table, c->sst, c->spart_acc, c->spart_ml,
                                                                                    c->scounters, c->sattn, cf.kv_heads, cf.gqa_ratio, pt, nsp, scale, pps, ns,
                                                                                    shared_tokens);
            else
                attn_decode_group_kernel<KT, 64, 2><<<agrid, 128, 0, m->stream>>>(c->sq, (const KT*)L.kv, m->page_table, c->sst, c->spart_acc, c->spart_ml,
                                                                                   c->scounters, c->sattn, cf.kv_heads, cf.gqa_ratio, pt, nsp, scale, pps, ns,
                                                                                   shared_tokens);
            pf_split_kernel<T16><<<split_blocks, 256, 0, m->stream>>>(c->sattn, xn, attn_lo, (size_t)ns * Q);
            PF_TRY("wo gemm", sk_launch(m, split, c->sk_o[l], a_attn, D, Q, ns, bf16, SkEpiPartial{c->sksum, D}, ks));
            pf_reduce_rmsnorm_kernel<T16><<<ns, nthreads, 0, m->stream>>>(c->sx, c->sksum, ks, m->alpha, L.gamma2, xn, xn_lo, D);
            PF_TRY("w13 gemm", sk_launch(m, split, c->sk_13[l], a_xn, 2 * H, D, ns, bf16, SkEpiGate<T16>{gate, gate_lo, H, m->opt.activation}));
            PF_TRY("w2 gemm", sk_launch(m, split, c->sk_2[l], a_gate, D, H, ns, bf16, SkEpiPartial{c->sksum, D}, ks));
            m->launches += 4;
        }
        pf_reduce_rmsnorm_kernel<T16><<<ns, nthreads, 0, m->stream>>>(c->sx, c->sksum, ks, m->alpha, m->gamma_final, xn, xn_lo, D);
        m->launches++;
        PF_TRY("head gemm", sk_launch(m, split, c->sk_head, a_xn, V, D, ns, bf16, SkEpiStore{c->slogits, Vp}));
        // each sample's own reductions and draw, on its own state; one launch covers all samples
        if (mode == 0) {
            head_argmax_kernel<<<dim3(NB, ns), 256, 0, m->stream>>>(c->slogits, V, c->sblock_vals, c->sblock_idxs, c->shead_counters, c->sout_token, c->sst, c->sring, 1, 0,
                                                                   TpLink{}, (size_t)Vp, (size_t)NB, (size_t)16, (size_t)ring_ld);
            m->launches++;
        } else if (mode == 1) {
            const size_t cs = (size_t)NB * CD_MAX_GPU_TOPK;
            head_topk_kernel<<<dim3(NB, ns), 256, 0, m->stream>>>(c->slogits, V, top_k, c->stopk_vals, c->stopk_idxs, (size_t)Vp, cs);
            sample_topk_kernel<<<ns, 1024, 0, m->stream>>>(c->stopk_vals, c->stopk_idxs, NB * top_k, top_k, t, softcap, c->sst, c->sring, cs, (size_t)ring_ld);
            m->launches += 2;
        } else {
            head_stats_kernel<<<dim3(NB, ns), 256, 0, m->stream>>>(c->slogits, V, inv_t, softcap, c->smaxes, c->ssums, (size_t)Vp, (size_t)NB);
            sample_fullvocab_kernel<<<ns, 256, 0, m->stream>>>(c->slogits, cf.vocab, c->smaxes, c->ssums, NB, t, softcap, c->sst, c->sring, (size_t)Vp, (size_t)NB,
                                                           (size_t)ring_ld);
            m->launches += 2;
        }
        PF_TRY("step launch", cudaGetLastError());
        return CD_OK;
    };
    // graphs of a step are kept per `nsp` for as long as the request parameters stay the same
    const SampleGraphKey key{ns, mode, top_k, t, softcap, split ? 1 : 0, len0};
    if (!(key == c->s_key)) {
        for (auto& kv : c->s_graphs) cudaGraphExecDestroy(kv.second);
        c->s_graphs.clear();
        c->s_key = key;
    }
    for (size_t step = 0; step < nsteps; ++step) {
        const int attn_len = len0 + (int)step + 1;
        const int nsp = std::max(1, std::min(m->nsplit, (attn_len + pt - 1) / pt));  // slices that hold keys at this position
        if (!m->opt.use_graph) {
            if ((rc = enqueue_step(nsp))) return rc;
            continue;
        }
        auto it = c->s_graphs.find(nsp);
        if (it == c->s_graphs.end()) {
            cudaGraph_t graph = nullptr;
            const uint64_t before = m->launches;
            PF_TRY("graph capture", cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
            rc = enqueue_step(nsp);
            const cudaError_t e2 = cudaStreamEndCapture(m->stream, &graph);
            if (rc || e2 != cudaSuccess) {
                if (graph) cudaGraphDestroy(graph);
                return rc ? rc : cuda_fail("graph capture", e2);
            }
            cudaGraphExec_t exec = nullptr;
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return cuda_fail("graph instantiate", e);
            c->s_graph_nodes = m->launches - before;
            m->launches = before;
            it = c->s_graphs.emplace(nsp, exec).first;
        }
        PF_TRY("graph launch", cudaGraphLaunch(it->second, m->stream));
        m->launches += c->s_graph_nodes;
    }
    PF_TRY("event", cudaEventRecord(m->ev1, m->stream));
    std::vector<DevState> hst(ns);
    std::vector<uint32_t> hring((size_t)ns * ring_ld);
    PF_TRY("read back", cudaMemcpyAsync(hst.data(), c->sst, (size_t)ns * sizeof(DevState), cudaMemcpyDeviceToHost, m->stream));
    PF_TRY("read back", cudaMemcpyAsync(hring.data(), c->sring, hring.size() * 4, cudaMemcpyDeviceToHost, m->stream));
    PF_TRY("read back", cudaMemcpyAsync(m->h_state, m->st, sizeof(DevState), cudaMemcpyDeviceToHost, m->stream));
    PF_TRY("sync", cudaStreamSynchronize(m->stream));
    PF_TRY("event", cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
#undef PF_TRY
    for (int s = 0; s < ns; ++s) {
        memcpy(out_ids + (size_t)s * nsteps, hring.data() + (size_t)s * ring_ld, nsteps * 4);
        if (rng) rng[s] = hst[s].rng;
        if (hst[s].error) {
            cudaMemsetAsync(&c->sst[s].error, 0, sizeof(int32_t), m->stream);
            return device_wait_failed(m, hst[s].error, " during the multi-sample decode");
        }
    }
    if (m->h_state->error) return device_wait_failed(m, m->h_state->error, " during the multi-sample decode");
    return CD_OK;
}

}  // namespace

int decode_samples(cd_model* m, const uint32_t* first, int ns, size_t nsteps, int mode, int top_k, float t, float softcap, uint64_t* rng,
                   uint32_t* out_ids) {
    PrefillCtx* c = nullptr;
    int rc = get_ctx(m, &c, false);
    if (rc) return rc;
    const char* pm = getenv("CD_PREFILL");
    const bool split = !(pm && !strcmp(pm, "fast"));
    if (m->opt.weight_dtype == CD_DTYPE_F16) return run_samples<__half, __half>(m, c, first, ns, nsteps, mode, top_k, t, softcap, rng, out_ids, split);
    return m->kv_dtype == CD_DTYPE_F16 ? run_samples<__nv_bfloat16, __half>(m, c, first, ns, nsteps, mode, top_k, t, softcap, rng, out_ids, split)
                                       : run_samples<__nv_bfloat16, __nv_bfloat16>(m, c, first, ns, nsteps, mode, top_k, t, softcap, rng, out_ids, split);
}

int prefill_batched(cd_model* m, size_t n) {
    PrefillCtx* c = nullptr;
    int rc = get_ctx(m, &c, true, true);
    if (rc) return rc;
    const int dt = m->opt.weight_dtype;
    // CD_PREFILL=fast: one 16-bit rounding of every GEMM input (about 1 % of the logit range at 5B);
    // default: hi + lo pairs, which keeps the prompt pass within the decode path's distance of the oracle
    const char* mode = getenv("CD_PREFILL");
    const bool split = !(mode && !strcmp(mode, "fast"));
    if (dt == CD_DTYPE_F16) return run<__half, __half>(m, c, n, split);
    // bf16 and FP8 linears: bf16 activations and head; the cache is fp16 or bf16
    return m->kv_dtype == CD_DTYPE_F16 ? run<__nv_bfloat16, __half>(m, c, n, split) : run<__nv_bfloat16, __nv_bfloat16>(m, c, n, split);
}

void prefill_release(cd_model* m) {
    PrefillCtx* c = (PrefillCtx*)m->prefill_ctx;
    if (!c) return;
    for (auto& kv : c->s_graphs) cudaGraphExecDestroy(kv.second);
    for (void* ptr : {(void*)c->x, c->xn, c->q, c->gate, (void*)c->s, c->p, c->vt, (void*)c->s_arena, c->f8_qkv, c->f8_o, c->f8_13, c->f8_2}) if (ptr) cudaFree(ptr);
    delete c;
    m->prefill_ctx = nullptr;
}

}  // namespace cd
