// Construction of the MoE + MLA decoder (cd_moe_model_create_synthetic): device memory for its
// weights and scratch, synthetic tensors generated in place.  The step itself is enqueued by
// model.cu (enqueue_step_moe_t) from the kernels of moe.cuh.  No reference counterpart.
#include <algorithm>
#include <cstring>
#include <vector>

#include "kernels.cuh"
#include "moe.cuh"
#include "model.h"

using namespace cd;

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline size_t esize(int dtype) { return dtype == CD_DTYPE_F32 ? 4 : 2; }

// tensor ids of the synthetic generator: uid = 0x100000 + 1024 * layer + local
enum { L_WQ = 0, L_WDKV, L_WKR, L_WUK, L_WUV, L_WO, L_WR, L_WS1, L_WS3, L_WS2, L_EXPERT0 = 16 };
inline uint64_t moe_uid(int layer, int local) { return 0x100000ull + (uint64_t)layer * 1024ull + (uint64_t)local; }

template <typename WT>
cudaError_t synth(cd_model* m, void* dst, int in, int out, int transposed, int row_mul, int row_off, uint64_t seed, uint64_t uid, float std,
                  int full_in, int full_out, int in0, int out0) {
    synth_kernel<WT><<<m->sm_count * 8, 256, 0, m->stream>>>((WT*)dst, in, out, transposed, row_mul, row_off, synth_key(seed, uid), std / 65536.0f,
                                                            full_in, full_out, in0, out0);
    return cudaGetLastError();
}

__global__ void fill_ones_kernel(float* p, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = 1.0f;
}

template <typename WT>
int build(cd_model* m, uint64_t seed, float std, int untied) {
    const cd_config& c = m->cfg;
    cd_moe_state& S = *m->moe;
    const cd_moe_config& mc = S.mc;
    const int D = c.dim, Hd = c.hidden, H = c.heads, C = mc.kv_latent, R = mc.rope_dim, N = mc.nope_dim, V = mc.v_dim, QH = N + R;
    const int SH = mc.n_shared * Hd;  // the shared FFN's columns in the whole model
    cudaError_t e = cudaSuccess;
#define SY(...) do { if (e == cudaSuccess) e = synth<WT>(m, __VA_ARGS__); } while (0)
    // embedding and head: [vocab, dim] as stored
    SY(m->embed, D, c.vocab, 0, 1, 0, seed, 0, std, D, c.vocab, 0, 0);
    if (untied) SY(m->lm_head, D, c.vocab, 0, 1, 0, seed, 2, std, D, c.vocab, 0, 0);
    for (int l = 0; l < c.nlayers; ++l) {
        cd_moe_layer_dev& L = S.layers[l];
        const size_t rb = (size_t)D * sizeof(WT);
        // wq | wdkv | wkr: logical [dim, out] each, stacked as rows of one matrix
        SY(L.wqa, D, H * QH, 1, 1, 0, seed, moe_uid(l, L_WQ), std, D, H * QH, 0, 0);
        SY((char*)L.wqa + (size_t)H * QH * rb, D, C, 1, 1, 0, seed, moe_uid(l, L_WDKV), std, D, C, 0, 0);
        SY((char*)L.wqa + (size_t)(H * QH + C) * rb, D, R, 1, 1, 0, seed, moe_uid(l, L_WKR), std, D, R, 0, 0);
        // wuk logical [latent, heads * nope]: per head, row c holds the head's nope columns of latent row c
        for (int h = 0; h < H; ++h)
            SY((char*)L.wuk_t + (size_t)h * C * N * sizeof(WT), N, C, 0, 1, 0, seed, moe_uid(l, L_WUK), std, H * N, C, h * N, 0);
        SY(L.wuv_t, C, H * V, 1, 1, 0, seed, moe_uid(l, L_WUV), std, C, H * V, 0, 0);   // logical [latent, heads * v_dim]
        SY(L.wo, H * V, D, 1, 1, 0, seed, moe_uid(l, L_WO), std, H * V, D, 0, 0);      // logical [heads * v_dim, dim]
        SY(L.wr, D, mc.n_experts, 1, 1, 0, seed, moe_uid(l, L_WR), std, D, mc.n_experts, 0, 0);
        // the shared FFN: this rank's columns sc0 .. sc0 + shared_cols of logical w1 / w3 [dim, SH] and w2 [dim (out), SH (in)]
        if (S.shared_cols > 0) {
            SY(L.ws13, D, S.shared_cols, 1, 2, 0, seed, moe_uid(l, L_WS1), std, D, SH, 0, S.sc0);
            SY(L.ws13, D, S.shared_cols, 1, 2, 1, seed, moe_uid(l, L_WS3), std, D, SH, 0, S.sc0);
            SY(L.ws2, S.shared_cols, D, 0, 1, 0, seed, moe_uid(l, L_WS2), std, SH, D, S.sc0, 0);
        }
        for (int le = 0; le < S.n_local; ++le) {
            const int ex = S.e0 + le;
            char* w13 = (char*)L.w13 + (size_t)le * 2 * Hd * rb;
            SY(w13, D, Hd, 1, 2, 0, seed, moe_uid(l, L_EXPERT0 + 3 * ex + 0), std, D, Hd, 0, 0);
            SY(w13, D, Hd, 1, 2, 1, seed, moe_uid(l, L_EXPERT0 + 3 * ex + 1), std, D, Hd, 0, 0);
            SY((char*)L.w2 + (size_t)le * D * Hd * sizeof(WT), Hd, D, 0, 1, 0, seed, moe_uid(l, L_EXPERT0 + 3 * ex + 2), std, Hd, D, 0, 0);
        }
    }
#undef SY
    if (e != cudaSuccess) return fail(m, CD_ERR_CUDA, std::string("synthetic MoE tensors: ") + cudaGetErrorString(e));
    e = cudaStreamSynchronize(m->stream);
    if (e != cudaSuccess) return fail(m, CD_ERR_CUDA, std::string("synthetic MoE tensors: ") + cudaGetErrorString(e));
    return CD_OK;
}

}  // namespace

namespace cd {
void moe_release(cd_model* m) {
    if (!m->moe) return;
    if (m->moe->arena) cudaFree(m->moe->arena);
    if (m->moe->ws) cudaFree(m->moe->ws);
    delete m->moe;
    m->moe = nullptr;
}
}  // namespace cd

extern "C" int cd_moe_model_create_synthetic(const cd_config* cfg, const cd_moe_config* moe, const cd_options* opts, uint64_t seed, float std,
                                             int untied_head, cd_model** out) {
    if (!cfg || !moe || !out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    *out = nullptr;
    cd_model* m = nullptr;
    int rc = model_alloc(cfg, opts, untied_head != 0, &m, moe);
    if (rc) return rc;
    auto bail = [&](int code) { set_global_error(m->err); cd_model_destroy(m); return code; };
    const cd_config& c = m->cfg;
    cd_moe_state* S = new cd_moe_state();
    m->moe = S;
    S->mc = *moe;
    {
        int32_t e0 = 0, ne = 0, s0 = 0, sc = 0;
        if (cd_moe_shard_plan(&c, moe, m->tp_world, m->tp_rank, &e0, &ne, &s0, &sc)) {
            fail(m, CD_ERR_UNSUPPORTED, "expert placement: n_experts and the shared FFN's columns / 8 must be divisible by the world size");
            return bail(CD_ERR_UNSUPPORTED);
        }
        S->e0 = e0; S->n_local = ne; S->sc0 = s0; S->shared_cols = sc;
    }
    S->nsplit = std::max(1, std::min(64, (c.seq + MLA_MMA_TILE - 1) / MLA_MMA_TILE));
    S->layers.resize(c.nlayers);

    const size_t es = esize(m->opt.weight_dtype);
    const size_t D = c.dim, Hd = c.hidden, H = c.heads, C = moe->kv_latent, R = moe->rope_dim, N = moe->nope_dim, V = moe->v_dim, QH = N + R;
    size_t off = 0;
    auto carve = [&](size_t bytes) { const size_t o = off; off = align_up(off + bytes, 256); return o; };
    struct LO { size_t wqa, wuk, wuv, wo, wr, w13, w2, ws13, ws2, g1, g2, gkv; };
    std::vector<LO> lo(c.nlayers);
    for (auto& l : lo) {
        l.wqa = carve((H * QH + C + R) * D * es); l.wuk = carve(H * C * N * es); l.wuv = carve(H * V * C * es); l.wo = carve(D * H * V * es);
        l.wr = carve((size_t)moe->n_experts * D * es); l.w13 = carve((size_t)S->n_local * 2 * Hd * D * es); l.w2 = carve((size_t)S->n_local * D * Hd * es);
        l.ws13 = carve((size_t)2 * S->shared_cols * D * es); l.ws2 = carve(D * (size_t)S->shared_cols * es);
        l.g1 = carve(D * 4); l.g2 = carve(D * 4); l.gkv = carve(C * 4);
    }
    cudaError_t e = cudaMalloc(&S->arena, off);
    if (e != cudaSuccess) { fail(m, CD_ERR_CUDA, std::string("MoE weight arena: ") + cudaGetErrorString(e)); return bail(CD_ERR_CUDA); }
    m->weight_bytes += off;
    char* wb = (char*)S->arena;
    for (int l = 0; l < c.nlayers; ++l) {
        cd_moe_layer_dev& L = S->layers[l];
        L.wqa = wb + lo[l].wqa; L.wuk_t = wb + lo[l].wuk; L.wuv_t = wb + lo[l].wuv; L.wo = wb + lo[l].wo; L.wr = wb + lo[l].wr;
        L.w13 = wb + lo[l].w13; L.w2 = wb + lo[l].w2; L.ws13 = wb + lo[l].ws13; L.ws2 = wb + lo[l].ws2;
        L.gamma1 = (float*)(wb + lo[l].g1); L.gamma2 = (float*)(wb + lo[l].g2); L.gamma_kv = (float*)(wb + lo[l].gkv);
        fill_ones_kernel<<<8, 256, 0, m->stream>>>(L.gamma1, D);
        fill_ones_kernel<<<8, 256, 0, m->stream>>>(L.gamma2, D);
        fill_ones_kernel<<<8, 256, 0, m->stream>>>(L.gamma_kv, C);
    }
    // scratch of a step
    off = 0;
    const size_t units = (size_t)moe->top_k * Hd + S->shared_cols;
    const size_t o_qa = carve((H * QH + C + R) * 4), o_qabs = carve(H * (C + R) * 4), o_pacc = carve((size_t)S->nsplit * H * C * 4);
    const size_t o_pml = carve((size_t)S->nsplit * H * 2 * 4), o_xn = carve(D * 4), o_sel = carve((size_t)c.nlayers * moe->top_k * 4), o_selw = carve(moe->top_k * 4);
    const size_t o_gate = carve(units * 4);
    const size_t o_rl = carve((size_t)moe->n_experts * 4), o_rc = carve(4), o_lid = carve(SRC_MAX_LIST * 4), o_lw = carve(SRC_MAX_LIST * 4), o_nl = carve(4), o_qs = carve(32 * (C + R) * 2);
    e = cudaMalloc(&S->ws, off);
    if (e == cudaSuccess) e = cudaMemsetAsync(S->ws, 0, off, m->stream);
    if (e != cudaSuccess) { fail(m, CD_ERR_CUDA, std::string("MoE scratch: ") + cudaGetErrorString(e)); return bail(CD_ERR_CUDA); }
    char* ws = (char*)S->ws;
    S->qa = (float*)(ws + o_qa); S->qabs = (float*)(ws + o_qabs); S->part_acc = (float*)(ws + o_pacc); S->part_ml = (float*)(ws + o_pml);
    S->xn2 = (float*)(ws + o_xn); S->sel_ids = (int*)(ws + o_sel); S->sel_w = (float*)(ws + o_selw); S->gate = (float*)(ws + o_gate);
    S->router_logits = (float*)(ws + o_rl); S->router_counter = (unsigned int*)(ws + o_rc); S->loc_ids = (int*)(ws + o_lid);
    S->loc_w = (float*)(ws + o_lw); S->n_loc = (int*)(ws + o_nl); S->qsplit = ws + o_qs;
    {
        // the streamed GEMV takes the expert matrices when a thread's share of the widest row fits its registers
        // (at most eight 16-byte chunks of x per thread) and every piece of a gathered row is a whole number of 16 bytes
        const size_t epc = 16 / es;
        const size_t k2 = units / epc, k13 = D / epc;
        S->stream_ffn = (k2 + 255) / 256 <= 8 && (k13 + 255) / 256 <= 8 && (Hd * es) % 16 == 0 && ((size_t)S->shared_cols * es) % 16 == 0 && (D * es) % 16 == 0 &&
                        units % epc == 0;
    }

    switch (m->opt.weight_dtype) {
        case CD_DTYPE_F32: rc = build<float>(m, seed, std, untied_head); break;
        case CD_DTYPE_F16: rc = build<__half>(m, seed, std, untied_head); break;
        default: rc = build<__nv_bfloat16>(m, seed, std, untied_head); break;
    }
    if (rc == CD_OK) rc = model_finish(m);
    if (rc) return bail(rc);
    *out = m;
    return CD_OK;
}

extern "C" int cd_moe_last_experts(cd_model* m, int layer, int32_t* out_ids, size_t cap) {
    if (!m || !out_ids) return fail(m, CD_ERR_INVALID, "null argument");
    if (!m->moe) return fail(m, CD_ERR_INVALID, "not a MoE + MLA model");
    if (layer < 0 || layer >= m->cfg.nlayers) return fail(m, CD_ERR_INVALID, "layer index out of range");
    if (cap < (size_t)m->moe->mc.top_k) return fail(m, CD_ERR_CAPACITY, "out_ids too small for top_k expert ids");
    cudaError_t e = cudaMemcpyAsync(out_ids, m->moe->sel_ids + (size_t)layer * m->moe->mc.top_k, (size_t)m->moe->mc.top_k * 4, cudaMemcpyDeviceToHost, m->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (e != cudaSuccess) return fail(m, CD_ERR_CUDA, std::string("cd_moe_last_experts: ") + cudaGetErrorString(e));
    return CD_OK;
}
