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
#include <string>
#include <vector>

#include "model.h"

namespace cd {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct PrefillCtx {
    EncodeTiledFn encode = nullptr;
    std::vector<CUtensorMap> w_qkv, w_o, w_13, w_2, k_pages;  // per layer, built once
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

template <typename T16>
int run(cd_model* m, PrefillCtx* c, size_t n, bool split) {
    const cd_config& cf = m->cfg;
    const bool bf16 = std::is_same<T16, __nv_bfloat16>::value;
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const int D = cf.dim, Q = cf.q_dim, KV = cf.kv_dim, H = cf.hidden, hd = cf.hd;
    const int pos0 = (int)m->len, M = (int)n, nkeys = pos0 + M;
    auto cuda_fail = [&](const char* what, cudaError_t e) { return fail(m, CD_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); };

    // ---- weights and pages: maps built once
    if (c->w_qkv.empty()) {
        c->w_qkv.resize(cf.nlayers); c->w_o.resize(cf.nlayers); c->w_13.resize(cf.nlayers); c->w_2.resize(cf.nlayers); c->k_pages.resize(cf.nlayers);
        bool ok = true;
        for (int l = 0; l < cf.nlayers && ok; ++l) {
            const cd_layer_dev& L = m->layers[l];
            ok = ok && encode_2d(c, &c->w_qkv[l], dt, L.wqkv, D, Q + 2 * KV, (uint64_t)D * 2, 256);
            ok = ok && encode_2d(c, &c->w_o[l], dt, L.wo, Q, D, (uint64_t)Q * 2, 256);
            ok = ok && encode_2d(c, &c->w_13[l], dt, L.w13, D, 2 * H, (uint64_t)D * 2, 256);
            ok = ok && encode_2d(c, &c->w_2[l], dt, L.w2, H, D, (uint64_t)H * 2, 256);
            ok = ok && encode_k_pages(c, &c->k_pages[l], dt, L.kv, hd, m->page_tokens, cf.kv_heads, m->num_pages);
        }
        if (!ok) { c->w_qkv.clear(); return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for a weight matrix"); }
    }
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
    T16* xn = (T16*)c->xn; T16* qb = (T16*)c->q; T16* gate = (T16*)c->gate; T16* pm = (T16*)c->p; T16* vt = (T16*)c->vt;
    T16* xn_lo = split ? xn + R * (size_t)std::max(D, Q) : nullptr;
    T16* q_lo = split ? qb + R * (size_t)Q : nullptr;
    T16* gate_lo = split ? gate + R * (size_t)H : nullptr;
    T16* p_lo = split ? pm + (size_t)cf.heads * plane : nullptr;
    CUtensorMap a_xn[2], a_attn[2], a_gate[2], a_q[2], a_p[2], b_vt;
    bool ok = encode_2d(c, &b_vt, dt, c->vt, KL, (uint64_t)cf.kv_heads * hd, (uint64_t)KL * 2, (uint32_t)hd);
    for (int h = 0; h < (split ? 2 : 1) && ok; ++h) {
        ok = encode_2d(c, &a_xn[h], dt, h ? xn_lo : xn, D, R, (uint64_t)D * 2, PF_BM) && encode_2d(c, &a_attn[h], dt, h ? xn_lo : xn, Q, R, (uint64_t)Q * 2, PF_BM) &&
             encode_2d(c, &a_gate[h], dt, h ? gate_lo : gate, H, R, (uint64_t)H * 2, PF_BM) && encode_2d(c, &a_q[h], dt, h ? q_lo : qb, Q, R, (uint64_t)Q * 2, PF_BM) &&
             encode_2d(c, &a_p[h], dt, h ? p_lo : pm, KL, (uint64_t)cf.heads * R, (uint64_t)KL * 2, PF_BM);
    }
    if (!ok) return fail(m, CD_ERR_CUDA, "cuTensorMapEncodeTiled failed for an activation buffer");

    cudaError_t e;
#define PF_TRY(what, x) do { e = (x); if (e != cudaSuccess) return cuda_fail(what, e); } while (0)
    pf_embed_kernel<T16><<<M, 256, 0, m->stream>>>((const T16*)m->embed, m->prompt_dev, c->x, D);
    m->launches++;
    PfGemm g = {};
    g.b_zdiv = 1; g.page_tokens = m->page_tokens; g.pos0 = pos0; g.err = &m->st->error;
    const float scale = 1.0f / std::sqrt((float)hd);
    for (int l = 0; l < cf.nlayers; ++l) {
        const cd_layer_dev& L = m->layers[l];
        pf_rmsnorm_kernel<T16><<<M, 256, 0, m->stream>>>(c->x, L.gamma1, xn, xn_lo, D);
        m->launches++;
        {   // q, k, v = xn Wqkv with RoPE; k and v into the pages
            PfGemm p = g; p.M = M; p.N = Q + 2 * KV; p.K = D;
            PfEpiQKV<T16> epi{qb, q_lo, (T16*)L.kv, m->page_table, m->rope, Q, KV, hd, cf.kv_heads, m->page_tokens, pos0};
            PF_TRY("qkv gemm", (pf_launch<256>(m, split, a_xn, c->w_qkv[l], p, bf16, 1, epi)));
        }
        pf_transpose_v_kernel<T16><<<dim3((unsigned)(KL / 64), cf.kv_heads), 256, 0, m->stream>>>((const T16*)L.kv, m->page_table, vt, nkeys, (int)KL,
                                                                                                 cf.kv_heads, hd, m->page_tokens);
        m->launches++;
        {   // scores = q k^T per head over the cached keys (tiles above the diagonal skipped)
            PfGemm p = g; p.M = M; p.N = nkeys; p.K = hd; p.a_col_z = hd; p.b_zdiv = cf.gqa_ratio; p.b_paged = 1; p.causal = 1;
            PF_TRY("score gemm", (pf_launch<128>(m, split, a_q, c->k_pages[l], p, bf16, cf.heads, PfEpiScores{c->s, plane, (int)KL})));
        }
        pf_softmax_kernel<T16><<<dim3(M, cf.heads), 256, 0, m->stream>>>(c->s, pm, p_lo, plane, (int)KL, pos0, scale);
        m->launches++;
        {   // attention output = P V per head (the K loop stops at the diagonal)
            PfGemm p = g; p.M = M; p.N = hd; p.K = nkeys; p.a_row_z = (int)R; p.b_row_z = hd; p.b_zdiv = cf.gqa_ratio; p.causal = 2;
            PfEpiAttnOut<T16> epi{xn, xn_lo, Q, hd};
            if (hd == 128) PF_TRY("pv gemm", (pf_launch<128>(m, split, a_p, b_vt, p, bf16, cf.heads, epi)));
            else PF_TRY("pv gemm", (pf_launch<64>(m, split, a_p, b_vt, p, bf16, cf.heads, epi)));
        }
        {   // x2 = x + alpha * (attn Wo)
            PfGemm p = g; p.M = M; p.N = D; p.K = Q;
            PF_TRY("wo gemm", (pf_launch<256>(m, split, a_attn, c->w_o[l], p, bf16, 1, PfEpiResidual{c->x, D, m->alpha})));
        }
        pf_rmsnorm_kernel<T16><<<M, 256, 0, m->stream>>>(c->x, L.gamma2, xn, xn_lo, D);
        m->launches++;
        {   // gate = act(x2n W1) * (x2n W3)
            PfGemm p = g; p.M = M; p.N = 2 * H; p.K = D;
            PF_TRY("w13 gemm", (pf_launch<256>(m, split, a_xn, c->w_13[l], p, bf16, 1, PfEpiGate<T16>{gate, gate_lo, H, m->opt.activation})));
        }
        {   // x = x2 + alpha * (gate W2^T)
            PfGemm p = g; p.M = M; p.N = D; p.K = H;
            PF_TRY("w2 gemm", (pf_launch<256>(m, split, a_gate, c->w_2[l], p, bf16, 1, PfEpiResidual{c->x, D, m->alpha})));
        }
    }
    // the last prompt position's hidden state, where the LM-head GEMV expects it
    PF_TRY("copy last row", cudaMemcpyAsync(m->x_a, c->x + (size_t)(M - 1) * D, (size_t)D * 4, cudaMemcpyDeviceToDevice, m->stream));
#undef PF_TRY
    return CD_OK;
}

}  // namespace

int prefill_batched(cd_model* m, size_t n) {
    const cd_config& cf = m->cfg;
    const int dt = m->opt.weight_dtype;
    if ((dt != CD_DTYPE_BF16 && dt != CD_DTYPE_F16) || m->tp_world > 1) return CD_ERR_UNSUPPORTED;
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
    // CD_PREFILL=fast: one 16-bit rounding of every GEMM input (about 1 % of the logit range at 5B);
    // default: hi + lo pairs, which keeps the prompt pass within the decode path's distance of the oracle
    const char* mode = getenv("CD_PREFILL");
    const bool split = !(mode && !strcmp(mode, "fast"));
    return dt == CD_DTYPE_BF16 ? run<__nv_bfloat16>(m, c, n, split) : run<__half>(m, c, n, split);
}

void prefill_release(cd_model* m) {
    PrefillCtx* c = (PrefillCtx*)m->prefill_ctx;
    if (!c) return;
    for (void* ptr : {(void*)c->x, c->xn, c->q, c->gate, (void*)c->s, c->p, c->vt}) if (ptr) cudaFree(ptr);
    delete c;
    m->prefill_ctx = nullptr;
}

}  // namespace cd
