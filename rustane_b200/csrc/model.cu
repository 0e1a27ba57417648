// cd_model: device memory, the per-token launch sequence and the C ABI that mirrors
// metal_decode::Model (crates/metal-decode/src/lib.rs:129-511).
#include "model.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <type_traits>

#include "mega.cuh"
#include "moe.cuh"

using namespace cd;

namespace {
thread_local std::string g_error;
}

namespace cd {
void set_global_error(const std::string& msg) { g_error = msg; }
int fail(cd_model* m, int code, const std::string& msg) {
    if (m) m->err = msg;
    g_error = msg;
    return code;
}
// A bounded device-side wait ran out (DevState::error holds where).  The word is cleared so the handle stays
// usable: the failed call's results are void, the cache length did not advance.
int device_wait_failed(cd_model* m, int dev_code, const char* where) {
    static const char* names[] = {"", "weight ring: stage never filled", "weight ring: stage never freed", "grid barrier", "tensor-parallel peer"};
    if (dev_code == DEV_ERR_BAD_TOKEN) {
        cudaMemsetAsync(&m->st->error, 0, sizeof(int32_t), m->stream);
        cudaStreamSynchronize(m->stream);
        return fail(m, CD_ERR_INVALID, std::string("the device selected a token id outside the vocabulary (logits without a finite maximum); row 0 was used") + where);
    }
    const char* what = dev_code >= 1 && dev_code <= 4 ? names[dev_code] : "tensor-core pipeline";
    cudaMemsetAsync(&m->st->error, 0, sizeof(int32_t), m->stream);
    cudaStreamSynchronize(m->stream);
    return fail(m, CD_ERR_DEVICE_WAIT, std::string("a bounded device-side wait ran out (") + what + ", code " + std::to_string(dev_code) + ")" + where);
}
}  // namespace cd

#define CK(m, call)                                                                              \
    do {                                                                                         \
        cudaError_t e_ = (call);                                                                 \
        if (e_ != cudaSuccess)                                                                   \
            return fail((m), CD_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));   \
    } while (0)

#define DISPATCH_WT(dtype, WT, ...)                                  \
    switch (dtype) {                                                 \
        case CD_DTYPE_F32: { typedef float WT; __VA_ARGS__; } break; \
        case CD_DTYPE_F16: { typedef __half WT; __VA_ARGS__; } break; \
        default: { typedef __nv_bfloat16 WT; __VA_ARGS__; } break;   \
    }
// storage of the embedding and the LM head (16-bit for the quantised kinds)
#define EMBED_DTYPE(m) (is_quant((m)->opt.weight_dtype) ? CD_DTYPE_BF16 : (m)->opt.weight_dtype)

namespace {

// kernel classes for per-class timing (cd_profile_decode_step)
enum { CLS_MISC = 0, CLS_QKV, CLS_ATTN, CLS_WO, CLS_W13, CLS_W2, CLS_HEAD, CLS_SAMPLE, CLS_COUNT };

// Counts a launch; in profiling mode also drops an event behind it so the time since
// the previous event can be charged to the launch's class.
inline void count_launch(cd_model* m) {
    m->launches++;
    if (m->profiling) {
        cudaEvent_t ev;
        cudaEventCreate(&ev);
        cudaEventRecord(ev, m->stream);
        m->prof_events.push_back(ev);
        m->prof_classes.push_back(m->cur_cls);
    }
}

inline size_t esize(int dtype) { return dtype == CD_DTYPE_F32 ? 4 : 2; }  // embedding, LM head, KV cache (never a quantised code)
inline bool is_quant(int dtype) { return dtype == CD_DTYPE_FP8_E4M3 || dtype == CD_DTYPE_INT4_G32; }
// bytes of one row of a linear with K inputs
inline size_t lin_row_bytes(int dtype, int K) {
    return dtype == CD_DTYPE_FP8_E4M3 ? Wfmt<Fp8Row>::row_stride(K) : dtype == CD_DTYPE_INT4_G32 ? Wfmt<Int4G32>::row_stride(K) : (size_t)K * esize(dtype);
}
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------ GEMV launch
template <typename WT, int NITER, int R, int UNIT, bool NORM, class Epi, class Src = SrcPlain>
cudaError_t gemv_go(cd_model* m, const WT* W, const float* x, const float* gamma, float* norm_out, int N, int K,
                    int NT, const Epi& epi, const Src& src = Src{}) {
    const int nunits_all = N / UNIT;
    {
        // one persistent CTA per SM, ring of up to eight 16-24 KB stages
        constexpr int G = Wfmt<WT>::QUANT ? 2 : 1;  // consumer groups: the quantised formats need twice the decode warps
        constexpr int RT = G == 2 ? (NITER == 1 ? 8 : 4) : NITER == 1 ? 4 : NITER == 2 ? 2 : 1;
        auto tk = gemv_tma_kernel<WT, NITER, RT, UNIT, NORM, Epi, G, Src>;
        const int grid = std::max(1, std::min(nunits_all, m->sm_count));
        const int rows_cap = (nunits_all / grid + 1) * UNIT;
        const size_t stage_bytes = (size_t)RT * Wfmt<WT>::row_stride(K);
        const size_t fixed = ((size_t)rows_cap * (GEMV_CONSUMERS / 32) + 32) * sizeof(float) + 2 * 8 * 8 + 128;
        const size_t budget = (size_t)m->ring_kb * 1024;
        const int nstages = fixed + 2 * stage_bytes <= budget ? (int)std::min<size_t>(8, (budget - fixed) / stage_bytes) : 0;
        if (nstages >= 2) {
            // never less than half an SM's shared memory: two of these CTAs (of consecutive kernels, under programmatic
            // dependent launch) on one SM measured 16 % slower per token and, rarely, gave run-to-run different logits
            const size_t smem = std::max((size_t)nstages * stage_bytes + fixed, (size_t)116 * 1024);
            static size_t smem_set = 0;  // per instantiation
            if (smem > smem_set) {
                cudaError_t e = cudaFuncSetAttribute(tk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return e;
                smem_set = smem;
            }
            cudaLaunchConfig_t lc = {};
            lc.gridDim = dim3(grid);
            lc.blockDim = dim3(G * GEMV_CONSUMERS + 32);
            lc.dynamicSmemBytes = smem;
            lc.stream = m->stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            lc.attrs = at;
            lc.numAttrs = m->pdl ? 1 : 0;
            NextStream next = m->next_stream;
            next.test_drop = (m->opt.test_flags & 8) ? 1 : 0;
            if (next.w && std::min(next.nunits, m->sm_count) != grid) next.w = nullptr;  // partitions would not line up
            m->next_stream.w = nullptr;
            TpLink tp = m->tp;
            tp.in_reduce = m->tp_in.in_reduce; tp.res = m->tp_in.res; tp.alpha = m->alpha; tp.x_out = m->tp_in.x_out; tp.ar_out = 0;
            m->tp_in.in_reduce = 0;
            cudaError_t e = cudaLaunchKernelEx(&lc, tk, W, x, gamma, norm_out, N, K, rows_cap, nstages, &m->st->error, next, tp, epi, src);
            count_launch(m);
            return e;
        }
    }
    return cudaErrorInvalidConfiguration;  // a stage of this shape does not fit the ring twice
}

// N and K of a gathered source (Src::DYNAMIC) are the upper bounds of its shape.  cudaErrorInvalidValue: no
// instantiation takes a K this wide (the caller may have another kernel for it).
template <typename WT, int UNIT, bool NORM, class Epi, class Src = SrcPlain>
cudaError_t launch_gemv(cd_model* m, const void* W, const float* x, const float* gamma, float* norm_out, int N, int K,
                        const Epi& epi, const Src& src = Src{}) {
    constexpr int EPC = Wfmt<WT>::EPC;
    const int nchunks = K / EPC;
    const int NT = std::min(256, (nchunks + 31) / 32 * 32);
    const int niter = (nchunks + NT - 1) / NT;
    const WT* w = reinterpret_cast<const WT*>(W);
    switch (niter) {
        case 1: return gemv_go<WT, 1, 8, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
        case 2: return gemv_go<WT, 2, 4, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
        case 3: return gemv_go<WT, 3, 2, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
        case 4: return gemv_go<WT, 4, 2, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
        default: break;
    }
    if constexpr (!Wfmt<WT>::QUANT) {  // the quantised formats hold 16 / 32 elements of x per chunk: four chunks per thread at most
        switch (niter) {
            case 5:
            case 6: return gemv_go<WT, 6, 2, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
            case 7:
            case 8: return gemv_go<WT, 8, 1, UNIT, NORM, Epi, Src>(m, w, x, gamma, norm_out, N, K, NT, epi, src);
            default: break;
        }
    }
    return cudaErrorInvalidValue;
}

template <typename KT, int HD>
cudaError_t launch_attn_hd(cd_model* m, const cd_layer_dev& L) {
    const cd_config& c = m->cfg;
    const float scale = 1.0f / std::sqrt((float)c.hd);  // ATTN_SCALE, lib.rs:1352
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(c.heads, m->nsplit);
    lc.blockDim = dim3(128);
    lc.stream = m->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = m->pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&lc, attn_decode_kernel<KT, HD>, (const float*)m->q, (const KT*)L.kv, (const int*)m->page_table,
                                       (const DevState*)m->st, m->part_acc, m->part_ml, m->counters, m->attn, c.kv_heads,
                                       c.gqa_ratio, m->page_tokens, m->nsplit, scale);
    count_launch(m);
    return e;
}

template <typename KT>
cudaError_t launch_attn(cd_model* m, const cd_layer_dev& L) {
    return m->cfg.hd == 128 ? launch_attn_hd<KT, 128>(m, L) : launch_attn_hd<KT, 64>(m, L);
}

__global__ void softcap_copy_kernel(const float* __restrict__ in, float* __restrict__ out, int n, float c) {
    const float inv = 1.0f / c;  // decode.rs:120-124: scale, tanh, scale
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) out[i] = c * tanhf(in[i] * inv);
}

// ------------------------------------------------------------------ persistent kernel launch
template <typename WT, typename KT, int ND, int NH, bool TPAR>
cudaError_t launch_mega_t(cd_model* m, int input_embed, int want_logits) {
    constexpr int RD = ND == 1 ? 4 : ND == 2 ? 2 : 1;
    constexpr int RH = NH == 1 ? 4 : NH == 2 ? 2 : 1;
    const cd_config& c = m->cfg;
    auto kern = decode_mega_kernel<WT, KT, ND, RD, NH, RH, TPAR>;
    const int grid = m->sm_count;
    const size_t es = sizeof(WT);
    const size_t stage_cap = (std::max((size_t)RD * c.dim * es, (size_t)RH * c.hidden * es) + 127) / 128 * 128;
    int max_rows = 0;
    for (int n : {c.q_dim + 2 * c.kv_dim, c.dim, 2 * c.hidden, want_logits ? m->v_loc : 0}) max_rows = std::max(max_rows, n / grid + 2);
    const int xs_dim = m->tp_world > 1 ? std::max(c.q_dim, c.dim) : c.q_dim;
    const size_t fixed = ((size_t)max_rows * (GEMV_CONSUMERS / 32) + 32 * MEGA_GROUPS + mega_attn_smem_floats(xs_dim)) * sizeof(float) + 32 +
                         (size_t)((m->pages_per_seq + 3) & ~3) * 4 + 2 * 16 * 8 + 128;
    const size_t budget = (size_t)m->ring_kb * 1024;
    if (fixed + 2 * stage_cap > budget) return cudaErrorInvalidConfiguration;
    const int nstages = (int)std::min<size_t>(16, (budget - fixed) / stage_cap) & ~1;  // even: slots alternate between the two consumer groups
    const size_t smem = (size_t)nstages * stage_cap + fixed;
    // attention tiles: the largest power-of-two run of cached positions that stays inside a page and fits a stage
    int tile = 64;
    while (tile > 1 && (tile > m->page_tokens || m->page_tokens % tile || (size_t)tile * c.hd * sizeof(KT) > stage_cap)) tile >>= 1;
    static size_t smem_set = 0;
    if (smem > smem_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        smem_set = smem;
    }
    MegaParams p;
    p.layers = (const MegaLayer*)m->mega_layers;
    p.embed = m->embed; p.lm_head = m->lm_head; p.gamma_final = m->gamma_final;
    p.x_a = m->x_a; p.x_b = m->x_b; p.q = m->q; p.gate = m->gate; p.logits = m->logits; p.norm_final = m->norm_final;
    p.part_acc = m->part_acc; p.part_ml = m->part_ml; p.grid_counter = m->grid_counter;
    p.st = m->st; p.page_table = m->page_table; p.rope = m->rope;
    p.dim = c.dim; p.hidden = c.hidden; p.heads = c.heads; p.kv_heads = c.kv_heads; p.hd = c.hd; p.nlayers = c.nlayers;
    p.vocab = m->v_loc; p.embed_rows = m->full_cfg.vocab; p.q_dim = c.q_dim; p.kv_dim = c.kv_dim; p.gqa = c.gqa_ratio; p.page_tokens = m->page_tokens;
    p.activation = m->opt.activation; p.alpha = m->alpha; p.attn_scale = 1.0f / std::sqrt((float)c.hd);
    p.trace = m->mega_trace;
    p.npages = m->pages_per_seq;
    p.tile_tokens = tile;
    p.wait_ns = m->wait_ns;
    p.tp = m->tp;  // world <= 1 on one GPU
    p.tp.wait_ns = m->wait_ns;
    p.xs_dim = xs_dim;
    p.nstages = nstages; p.stage_cap = (uint32_t)stage_cap; p.rows_cap = max_rows; p.input_embed = input_embed; p.want_logits = want_logits;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(MEGA_THREADS);
    lc.dynamicSmemBytes = smem;
    lc.stream = m->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident: they meet at grid barriers
    at[0].val.cooperative = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&lc, kern, p);
    count_launch(m);
    return e;
}

template <typename WT, typename KT, bool TPAR>
cudaError_t launch_mega_tp(cd_model* m, int input_embed, int want_logits) {
    switch (m->mega_nd * 10 + m->mega_nh) {
        case 11: return launch_mega_t<WT, KT, 1, 1, TPAR>(m, input_embed, want_logits);
        case 12: return launch_mega_t<WT, KT, 1, 2, TPAR>(m, input_embed, want_logits);
        case 24: return launch_mega_t<WT, KT, 2, 4, TPAR>(m, input_embed, want_logits);
        case 26: return launch_mega_t<WT, KT, 2, 6, TPAR>(m, input_embed, want_logits);
        default: return cudaErrorInvalidConfiguration;
    }
}
template <typename WT, typename KT>
cudaError_t launch_mega(cd_model* m, int input_embed, int want_logits) {
    if constexpr (!std::is_same<WT, float>::value) {  // the tensor-parallel form exists for the 16-bit storage types
        if (m->tp_world > 1) return launch_mega_tp<WT, KT, true>(m, input_embed, want_logits);
    }
    return launch_mega_tp<WT, KT, false>(m, input_embed, want_logits);
}

struct StepParams {
    int input;  // 0: x already in x_a; 1: embed st->token; 2: take the next prompt token, then embed
    int head;   // cd_head_mode
    int k = 0;
    float t = 0.f, softcap = 0.f, inv_t = 1.f;
};

// What follows the layers: nothing (hidden state wanted), or the final RMSNorm + LM head and the head reduction /
// sampler the step asks for.  `ars`: all-reduces the token issued (tensor / expert parallel), `last_ar`: index of the
// one whose sum is still in the inboxes.  WT: storage of the LM head; LT: row format of the next token's first GEMV.
template <typename WT, typename LT>
cudaError_t enqueue_head_t(cd_model* m, const StepParams& p, bool use_mega, unsigned int ars, int last_ar) {
    const cd_config& c = m->cfg;
    cudaError_t e;
#define TRY(x) do { e = (x); if (e != cudaSuccess) return e; } while (0)
    // a vocabulary-sharded head exchanges candidates between the ranks; the MoE model's head is replicated
    const bool xhead = m->tp_world > 1 && m->moe == nullptr;
    const TpLink htp = xhead ? m->tp : TpLink{};
    m->cur_cls = CLS_MISC;
    if (p.head == HEAD_NONE) {
        if (m->tp_world > 1) {  // nobody else reads the last all-reduce of this token: consume it
            TpLink tp = m->tp;
            tp.in_reduce = last_ar; tp.res = m->x_b; tp.x_out = m->x_a; tp.alpha = m->alpha;
            tp_consume_kernel<<<8, 256, 0, m->stream>>>(tp, &m->st->error);
            count_launch(m);
        }
        advance_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
        count_launch(m);
        return cudaGetLastError();
    }
    // encode_rmsnorm(gamma_final) + LM head (lib.rs:867-986), logits left in HBM
    m->cur_cls = CLS_HEAD;
    if (!use_mega) {
    m->next_stream = NextStream{(m->prefetch_kb > 0 && !m->moe) ? m->layers[0].wqkv : nullptr, Wfmt<LT>::row_stride(c.dim),
                                (c.q_dim + 2 * c.kv_dim) / 2, 2, (uint32_t)m->prefetch_kb * 1024u};
    if (m->tp_world > 1) { m->tp_in.in_reduce = last_ar; m->tp_in.res = m->x_b; m->tp_in.x_out = m->x_a; }
    TRY((launch_gemv<WT, 1, true>(m, m->lm_head, m->x_a, m->gamma_final, m->norm_final, m->v_loc, c.dim, EpiStore{m->logits})));
    }
    unsigned int* head_counter = m->counters + c.heads;
    m->cur_cls = CLS_SAMPLE;
    bool count_ars = m->tp_world > 1 && !xhead;  // the single-GPU head kernels do not count the token's all-reduces
    switch (p.head) {
        case HEAD_LOGITS:
            advance_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
            count_ars = false;
            break;
        case HEAD_ARGMAX:
        case LOOP_GREEDY:
            head_argmax_kernel<<<m->nblocks, 256, 0, m->stream>>>(m->logits, m->v_loc, m->block_vals, m->block_idxs, head_counter,
                                                                 m->out_token, m->st, m->out_ring, p.head == LOOP_GREEDY, m->v0, htp);
            if (xhead) {
                count_launch(m);
                tp_pick_kernel<<<1, 32, 0, m->stream>>>(m->tp, m->out_token, m->st, m->out_ring, p.head == LOOP_GREEDY, ars);
            }
            break;
        case HEAD_TOPK:
        case LOOP_TOPK:
            head_topk_kernel<<<m->nblocks, 256, 0, m->stream>>>(m->logits, m->v_loc, p.k, m->topk_vals, m->topk_idxs);
            count_launch(m);
            if (p.head == LOOP_TOPK && xhead) {
                // every rank's candidates to every rank, then the same merge and draw everywhere
                tp_push_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->topk_vals, m->topk_idxs, m->nblocks, m->tp_nb, p.k, m->v0);
                tp_wait_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->st, m->tp_topk_vals, m->tp_topk_idxs, m->tp_nb, m->tp_nb * 32);
                sample_topk_kernel<<<1, 1024, 0, m->stream>>>(m->tp_topk_vals, m->tp_topk_idxs, m->tp_world * m->tp_nb * 32, p.k, p.t, p.softcap,
                                                              m->st, m->out_ring);
                count_launch(m); count_launch(m); count_launch(m);
                tp_count_allreduces_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
            } else if (p.head == LOOP_TOPK)
                sample_topk_kernel<<<1, 1024, 0, m->stream>>>(m->topk_vals, m->topk_idxs, m->nblocks * p.k, p.k, p.t, p.softcap,
                                                              m->st, m->out_ring);
            else {
                if (xhead) {  // the per-token call: every rank's candidates to every rank, the host copies them out in block order
                    tp_push_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->topk_vals, m->topk_idxs, m->nblocks, m->tp_nb, p.k, m->v0);
                    tp_wait_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->st, m->tp_topk_vals, m->tp_topk_idxs, m->tp_nb, m->tp_nb * 32);
                    count_launch(m); count_launch(m);
                }
                advance_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
                count_ars = false;
            }
            break;
        case HEAD_STATS:
        case LOOP_FULLVOCAB:
            head_stats_kernel<<<m->nblocks, 256, 0, m->stream>>>(m->logits, m->v_loc, p.inv_t, p.softcap, m->maxes, m->sums);
            count_launch(m);
            if (p.head == LOOP_FULLVOCAB && xhead) {
                // every rank's per-block (max, sum) to every rank; all pick the same block, its owner draws the token
                tp_push_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->maxes, reinterpret_cast<const uint32_t*>(m->sums), m->nblocks, m->tp_nb, 1, 0);
                tp_wait_topk_kernel<<<1, 256, 0, m->stream>>>(m->tp, m->st, m->tp_topk_vals, m->tp_topk_idxs, m->tp_nb, m->tp_nb);
                count_launch(m); count_launch(m);
                tp_sample_fullvocab_kernel<<<1, 256, 0, m->stream>>>(m->logits, m->v0, m->full_cfg.vocab, m->tp_topk_vals, m->tp_topk_idxs, m->tp_nb,
                                                                    p.t, p.softcap, m->st, m->out_ring, m->tp, ars);
            } else if (p.head == LOOP_FULLVOCAB)
                sample_fullvocab_kernel<<<1, 256, 0, m->stream>>>(m->logits, c.vocab, m->maxes, m->sums, m->nblocks, p.t, p.softcap,
                                                                 m->st, m->out_ring);
            else {
                advance_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
                count_ars = false;
            }
            break;
        default: return cudaErrorInvalidValue;
    }
    count_launch(m);
    if (count_ars) {
        tp_count_allreduces_kernel<<<1, 1, 0, m->stream>>>(m->st, ars);
        count_launch(m);
    }
    return cudaGetLastError();
#undef TRY
}

// A launch in the token's chain of kernels: under programmatic dependent launch the kernel may become resident while
// its predecessor still runs (each of them waits, griddepcontrol.wait, before it touches anything the chain produced).
template <typename... KArgs, typename... Args>
cudaError_t launch_chain(cd_model* m, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = m->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at;
    lc.numAttrs = m->pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&lc, kern, std::forward<Args>(args)...);
    count_launch(m);
    return e;
}

// One token through the MoE + MLA decoder (moe.cuh).  WT: storage of all weights; KT: storage of the latent cache.
template <typename WT, typename KT>
cudaError_t enqueue_step_moe_t(cd_model* m, const StepParams& p) {
    const cd_config& c = m->cfg;
    cd_moe_state& S = *m->moe;
    const cd_moe_config& mc = S.mc;
    cudaError_t e;
#define TRY(x) do { e = (x); if (e != cudaSuccess) return e; } while (0)
    m->cur_cls = CLS_MISC;
    m->next_stream.w = nullptr;
    if (p.input == 2) {
        next_prompt_kernel<<<1, 1, 0, m->stream>>>(m->st, m->prompt_dev);
        count_launch(m);
    }
    if (p.input >= 1) {
        embed_kernel<WT><<<std::max(1, c.dim / 256), 256, 0, m->stream>>>((const WT*)m->embed, m->st, m->x_a, c.dim, m->full_cfg.vocab);
        count_launch(m);
        TRY(cudaGetLastError());
    }
    const MlaDims md{c.heads, mc.kv_latent, mc.rope_dim, mc.nope_dim, mc.v_dim, m->page_tokens};
    const MoeDims ed{c.dim, c.hidden, S.shared_cols};
    const MoePick pick{S.loc_ids, S.loc_w, S.n_loc};
    const int W = mc.kv_latent + mc.rope_dim, QA = c.q_dim + W, units = mc.top_k * c.hidden + S.shared_cols;
    const bool ep = m->tp_world > 1;
    const float scale = 1.0f / std::sqrt((float)c.hd);
    // the tensor-core attention takes a 16-bit cache of the 512-wide latent geometry; anything else the plain kernel
    const bool attn_mma = !std::is_same<KT, float>::value && mc.kv_latent == MLA_MMA_C && W % 16 == 0 && c.heads <= 16;
    const size_t attn_smem = attn_mma ? mla_mma_smem_bytes(W)
                                      : ((size_t)(c.heads + MLA_TILE) * (W + 1) + (size_t)c.heads * MLA_TILE + 3 * c.heads) * sizeof(float);
    static size_t attn_set = 0, w2_set = 0;  // per instantiation
    if (attn_smem > attn_set) {
        if constexpr (!std::is_same<KT, float>::value) TRY(cudaFuncSetAttribute(mla_attn_mma_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(attn_smem, mla_mma_smem_bytes(W))));
        TRY(cudaFuncSetAttribute(mla_attn_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem));
        attn_set = attn_smem;
    }
    if (!S.stream_ffn && (size_t)units * 4 > w2_set) {
        TRY(cudaFuncSetAttribute(moe_w2_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, units * 4));
        w2_set = (size_t)units * 4;
    }
    const uint32_t es = (uint32_t)sizeof(WT);
    for (int l = 0; l < c.nlayers; ++l) {
        const cd_moe_layer_dev& L = S.layers[l];
        int* sel = S.sel_ids + (size_t)l * mc.top_k;
        m->cur_cls = CLS_QKV;
        if (ep && l > 0) { m->tp_in.in_reduce = l; m->tp_in.res = m->x_b; m->tp_in.x_out = m->x_a; }  // x = x2 + alpha * sum(ranks' FFN partials)
        TRY((launch_gemv<WT, 1, true>(m, L.wqa, m->x_a, L.gamma1, nullptr, QA, c.dim, EpiStore{S.qa})));
        m->cur_cls = CLS_ATTN;
        TRY(launch_chain(m, mla_post_kernel<WT, KT>, dim3((c.heads * mc.kv_latent + 127) / 128 + 1), dim3(128), std::max(c.heads * mc.nope_dim, mc.kv_latent) * sizeof(float),
                         (const float*)S.qa, (const WT*)L.wuk_t, (const float*)L.gamma_kv, (const float2*)m->rope, (const int*)m->page_table, (const DevState*)m->st,
                         (KT*)m->layers[l].kv, S.qabs, attn_mma ? (KT*)S.qsplit : (KT*)nullptr, md));
        if constexpr (!std::is_same<KT, float>::value) {
            if (attn_mma)
                TRY(launch_chain(m, mla_attn_mma_kernel<KT>, dim3(S.nsplit), dim3(MLA_MMA_THREADS), attn_smem, (const KT*)S.qsplit, (const KT*)m->layers[l].kv,
                                 (const int*)m->page_table, (const DevState*)m->st, S.part_acc, S.part_ml, md, S.nsplit, scale, &m->st->error));
        }
        if (!attn_mma)
            TRY(launch_chain(m, mla_attn_kernel<KT>, dim3(S.nsplit), dim3(256), attn_smem, (const float*)S.qabs, (const KT*)m->layers[l].kv, (const int*)m->page_table,
                             (const DevState*)m->st, S.part_acc, S.part_ml, md, S.nsplit, scale));
        TRY(launch_chain(m, mla_out_kernel<WT>, dim3(c.heads, (mc.v_dim + 31) / 32), dim3(256), (mc.kv_latent + S.nsplit) * sizeof(float), (const float*)S.part_acc,
                         (const float*)S.part_ml, (const WT*)L.wuv_t, m->attn, (const DevState*)m->st, md, S.nsplit, attn_mma ? MLA_MMA_TILE : MLA_TILE));
        m->cur_cls = CLS_WO;
        TRY((launch_gemv<WT, 1, false>(m, L.wo, m->attn, nullptr, nullptr, c.dim, c.heads * mc.v_dim, EpiResidual{m->x_a, m->x_b, m->alpha})));
        m->cur_cls = CLS_W13;
        TRY(launch_chain(m, moe_router_kernel<WT>, dim3((mc.n_experts + 3) / 4), dim3(128), std::max(c.dim, mc.n_experts) * sizeof(float), (const float*)m->x_b,
                         (const float*)L.gamma2, (const WT*)L.wr, S.xn2, S.router_logits, S.router_counter, sel, S.sel_w, S.loc_ids, S.loc_w, S.n_loc, c.dim, mc.n_experts,
                         mc.top_k, S.e0, S.n_local));
        TpLink tp = m->tp;
        tp.ar_out = l + 1;
        if (S.stream_ffn) {
            // the chosen experts' rows gathered by the streamed GEMV's copy engine; K and N are upper bounds (all top_k local)
            const SrcExpertRows s13{S.loc_ids, S.n_loc, L.ws13, 2 * c.hidden, 2 * S.shared_cols};
            TRY((launch_gemv<WT, 2, false>(m, L.w13, S.xn2, nullptr, nullptr, 2 * units, c.dim, EpiGateMoe{S.gate, S.loc_w, S.n_loc, c.hidden}, s13)));
            m->cur_cls = CLS_W2;
            const SrcExpertCols s2{S.loc_ids, S.n_loc, L.ws2, c.hidden, S.shared_cols, c.dim, (uint32_t)c.hidden * es, (uint32_t)S.shared_cols * es};
            if (ep) TRY((launch_gemv<WT, 1, false>(m, L.w2, S.gate, nullptr, nullptr, c.dim, units, EpiPush{tp}, s2)));
            else TRY((launch_gemv<WT, 1, false>(m, L.w2, S.gate, nullptr, nullptr, c.dim, units, EpiResidual{m->x_b, m->x_a, m->alpha}, s2)));
        } else {
            TRY(launch_chain(m, moe_w13_kernel<WT>, dim3((units + 7) / 8), dim3(256), c.dim * sizeof(float), (const float*)S.xn2, (const WT*)L.w13, (const WT*)L.ws13, pick,
                             S.gate, ed));
            m->cur_cls = CLS_W2;
            TRY(launch_chain(m, moe_w2_kernel<WT>, dim3((c.dim + 7) / 8), dim3(256), units * sizeof(float), (const float*)S.gate, (const WT*)L.w2, (const WT*)L.ws2, pick,
                             (const float*)m->x_b, m->x_a, m->alpha, ed, ep ? tp : TpLink{}));
        }
        TRY(cudaGetLastError());
    }
    return enqueue_head_t<WT, WT>(m, p, false, ep ? (unsigned int)c.nlayers : 0u, c.nlayers);
#undef TRY
}

// One token through the whole model; everything is enqueued on m->stream.
// WT: storage of the embedding and the LM head; LT: row format of the linears; KT: storage of the KV cache.
template <typename WT, typename LT, typename KT>
cudaError_t enqueue_step_t(cd_model* m, const StepParams& p) {
    const cd_config& c = m->cfg;
    cudaError_t e;
#define TRY(x) do { e = (x); if (e != cudaSuccess) return e; } while (0)
    m->cur_cls = CLS_MISC;
    if (p.input == 2) {
        next_prompt_kernel<<<1, 1, 0, m->stream>>>(m->st, m->prompt_dev);
        count_launch(m);
    }
    const bool use_mega = std::is_same<WT, LT>::value && m->mega && m->mega_nd > 0 && !m->profiling;
    if (use_mega) {
        if constexpr (std::is_same<WT, LT>::value) TRY((launch_mega<WT, KT>(m, p.input >= 1 ? 1 : 0, p.head != HEAD_NONE ? 1 : 0)));
    } else if (p.input >= 1) {
        embed_kernel<WT><<<std::max(1, c.dim / 256), 256, 0, m->stream>>>((const WT*)m->embed, m->st, m->x_a, c.dim, m->full_cfg.vocab);
        count_launch(m);
        TRY(cudaGetLastError());
    }
    for (int l = 0; l < c.nlayers && !use_mega; ++l) {
        const cd_layer_dev& L = m->layers[l];
        EpiQKV<KT> eq{m->q, (KT*)L.kv, m->page_table, m->st, m->rope, c.q_dim, c.kv_dim, c.hd, c.kv_heads, m->page_tokens};
        const bool last = l + 1 == c.nlayers;
        auto hint = [&](const void* w, int K, int N, int unit, bool head = false) {
            const uint32_t rb = head ? (uint32_t)(K * sizeof(WT)) : Wfmt<LT>::row_stride(K);
            m->next_stream = NextStream{m->prefetch_kb > 0 ? w : nullptr, rb, N / unit, unit, (uint32_t)m->prefetch_kb * 1024u};
        };
        const bool tp_on = m->tp_world > 1;
        EpiPush push{m->tp};
        m->cur_cls = CLS_QKV;
        hint(L.wo, c.q_dim, c.dim, 1);
        if (tp_on && l > 0) { m->tp_in.in_reduce = 2 * l; m->tp_in.res = m->x_b; m->tp_in.x_out = m->x_a; }  // x = x2 + alpha * sum(W2 partials)
        TRY((launch_gemv<LT, 2, true>(m, L.wqkv, m->x_a, L.gamma1, nullptr, c.q_dim + 2 * c.kv_dim, c.dim, eq)));
        m->cur_cls = CLS_ATTN;
        TRY(launch_attn<KT>(m, L));
        m->cur_cls = CLS_WO;
        hint(L.w13, c.dim, 2 * c.hidden, 2);
        push.tp.ar_out = 2 * l + 1;
        if (tp_on) TRY((launch_gemv<LT, 1, false>(m, L.wo, m->attn, nullptr, nullptr, c.dim, c.q_dim, push)));
        else TRY((launch_gemv<LT, 1, false>(m, L.wo, m->attn, nullptr, nullptr, c.dim, c.q_dim, EpiResidual{m->x_a, m->x_b, m->alpha})));
        m->cur_cls = CLS_W13;
        hint(L.w2, c.hidden, c.dim, 1);
        if (tp_on) { m->tp_in.in_reduce = 2 * l + 1; m->tp_in.res = m->x_a; m->tp_in.x_out = m->x_b; }  // x2 = x + alpha * sum(Wo partials)
        TRY((launch_gemv<LT, 2, true>(m, L.w13, m->x_b, L.gamma2, nullptr, 2 * c.hidden, c.dim, EpiGate{m->gate, m->opt.activation})));
        m->cur_cls = CLS_W2;
        if (!last) hint(m->layers[l + 1].wqkv, c.dim, c.q_dim + 2 * c.kv_dim, 2);
        else if (p.head != HEAD_NONE) hint(m->lm_head, c.dim, m->v_loc, 1, true);
        else hint(m->layers[0].wqkv, c.dim, c.q_dim + 2 * c.kv_dim, 2);
        push.tp.ar_out = 2 * l + 2;
        if (tp_on) TRY((launch_gemv<LT, 1, false>(m, L.w2, m->gate, nullptr, nullptr, c.dim, c.hidden, push)));
        else TRY((launch_gemv<LT, 1, false>(m, L.w2, m->gate, nullptr, nullptr, c.dim, c.hidden, EpiResidual{m->x_b, m->x_a, m->alpha})));
    }
    return enqueue_head_t<WT, LT>(m, p, use_mega, m->tp_world > 1 ? 2u * (unsigned int)c.nlayers : 0u, 2 * c.nlayers);
#undef TRY
}

// final RMSNorm + LM head on the hidden state in x_a; logits stay in HBM, the state is not advanced
cudaError_t enqueue_head_only(cd_model* m) {
    m->cur_cls = CLS_HEAD;
    m->next_stream.w = nullptr;
    cudaError_t e = cudaSuccess;
    DISPATCH_WT(EMBED_DTYPE(m), WT,
                e = (launch_gemv<WT, 1, true>(m, m->lm_head, m->x_a, m->gamma_final, m->norm_final, m->v_loc, m->cfg.dim, EpiStore{m->logits})));
    return e;
}

cudaError_t enqueue_step(cd_model* m, const StepParams& p) {
    cudaError_t e = cudaSuccess;
    if (m->moe) {
        switch (m->opt.weight_dtype) {
            case CD_DTYPE_F32: return enqueue_step_moe_t<float, float>(m, p);
            case CD_DTYPE_F16: return enqueue_step_moe_t<__half, __half>(m, p);
            default: return m->kv_dtype == CD_DTYPE_F16 ? enqueue_step_moe_t<__nv_bfloat16, __half>(m, p) : enqueue_step_moe_t<__nv_bfloat16, __nv_bfloat16>(m, p);
        }
    }
    const bool kv16 = m->kv_dtype == CD_DTYPE_F16;  // otherwise the cache has the embedding's type (model_alloc admits nothing else)
    switch (m->opt.weight_dtype) {
        case CD_DTYPE_F32: e = enqueue_step_t<float, float, float>(m, p); break;
        case CD_DTYPE_F16: e = enqueue_step_t<__half, __half, __half>(m, p); break;
        case CD_DTYPE_FP8_E4M3:
            e = kv16 ? enqueue_step_t<__nv_bfloat16, Fp8Row, __half>(m, p) : enqueue_step_t<__nv_bfloat16, Fp8Row, __nv_bfloat16>(m, p);
            break;
        case CD_DTYPE_INT4_G32:
            e = kv16 ? enqueue_step_t<__nv_bfloat16, Int4G32, __half>(m, p) : enqueue_step_t<__nv_bfloat16, Int4G32, __nv_bfloat16>(m, p);
            break;
        default:
            e = kv16 ? enqueue_step_t<__nv_bfloat16, __nv_bfloat16, __half>(m, p) : enqueue_step_t<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(m, p);
            break;
    }
    return e;
}

// Run one step: directly, or by replaying the captured graph of the same shape.
int run_step(cd_model* m, const StepParams& p) {
    if (!m->opt.use_graph) {
        cudaError_t e = enqueue_step(m, p);
        if (e != cudaSuccess) return fail(m, CD_ERR_CUDA, std::string("step launch: ") + cudaGetErrorString(e));
        return CD_OK;
    }
    const cd_graph_key key{p.head, p.k, p.input, p.t, p.inv_t, p.softcap};
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        const uint64_t before = m->launches;
        cudaGraph_t graph = nullptr;
        CK(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t e = enqueue_step(m, p);
        cudaError_t e2 = cudaStreamEndCapture(m->stream, &graph);
        if (e != cudaSuccess || e2 != cudaSuccess) {
            if (graph) cudaGraphDestroy(graph);
            return fail(m, CD_ERR_CUDA, std::string("graph capture: ") + cudaGetErrorString(e != cudaSuccess ? e : e2));
        }
        cudaGraphExec_t exec = nullptr;
        CK(m, cudaGraphInstantiate(&exec, graph, 0));
        cudaGraphDestroy(graph);
        const cd_graph_entry entry{exec, m->launches - before};
        m->launches = before;
        it = m->graphs.emplace(key, entry).first;
    }
    CK(m, cudaGraphLaunch(it->second.exec, m->stream));
    m->launches += it->second.nodes;
    return CD_OK;
}

int check_room(cd_model* m, size_t need) {
    if (m->tp_world > 1 && !m->tp_connected)
        return fail(m, CD_ERR_INVALID, "tensor-parallel model is not connected to its peers (cd_tp_connect)");
    if (m->len + need > (size_t)m->cfg.seq)
        return fail(m, CD_ERR_SEQ_FULL, "metal decode only supports lengths within cfg.seq");
    return CD_OK;
}
int check_token(cd_model* m, uint32_t tok) {
    if (tok >= (uint32_t)m->cfg.vocab) return fail(m, CD_ERR_TOKEN, "token id must fit vocab for metal decode");
    return CD_OK;
}

int set_state(cd_model* m, uint32_t token) {
    // {pos, token} are the first 8 bytes of DevState: one small copy from pinned memory.
    // Every per-token entry point synchronises before returning, so the staging words are free.
    m->h_in[0] = (uint32_t)m->len;
    m->h_in[1] = token;
    CK(m, cudaMemcpyAsync(m->st, m->h_in, 8, cudaMemcpyHostToDevice, m->stream));
    return CD_OK;
}

}  // namespace

// ====================================================================== construction
namespace cd {

static int validate(const cd_config& c, int dtype) {
    if (c.dim <= 0 || c.hidden <= 0 || c.heads <= 0 || c.kv_heads <= 0 || c.hd <= 0 || c.seq <= 0 || c.nlayers <= 0 || c.vocab <= 0)
        return fail(nullptr, CD_ERR_INVALID, "config contains a non-positive dimension");
    if (c.q_dim != c.heads * c.hd || c.kv_dim != c.kv_heads * c.hd || c.heads % c.kv_heads != 0 || c.gqa_ratio != c.heads / c.kv_heads)
        return fail(nullptr, CD_ERR_INVALID, "q_dim / kv_dim / gqa_ratio inconsistent with heads, kv_heads and hd");
    if (c.hd != 64 && c.hd != 128) return fail(nullptr, CD_ERR_UNSUPPORTED, "head dimension must be 64 or 128");
    if (dtype < CD_DTYPE_F32 || dtype > CD_DTYPE_INT4_G32) return fail(nullptr, CD_ERR_INVALID, "unknown weight dtype");
    const int epc = dtype == CD_DTYPE_F32 ? 4 : dtype == CD_DTYPE_FP8_E4M3 ? 16 : dtype == CD_DTYPE_INT4_G32 ? 32 : 8;
    const int kmax = dtype >= CD_DTYPE_FP8_E4M3 ? 4 * 256 * 16 : 8 * 256 * epc;
    if (c.dim % 8 || c.q_dim % 8 || c.hidden % 8) return fail(nullptr, CD_ERR_UNSUPPORTED, "dim, q_dim and hidden must be multiples of 8");
    if (c.dim % epc || c.q_dim % epc || c.hidden % epc) return fail(nullptr, CD_ERR_UNSUPPORTED, "dim, q_dim and hidden must be multiples of the quantisation chunk (16 for FP8, 32 for INT4)");
    if (c.dim > kmax || c.q_dim > kmax || c.hidden > kmax) return fail(nullptr, CD_ERR_UNSUPPORTED, "inner dimension too large for the GEMV tiling");
    return CD_OK;
}

static int validate_moe(const cd_config& c, const cd_moe_config& mc, int dtype, int world) {
    if (c.dim <= 0 || c.hidden <= 0 || c.heads <= 0 || c.seq <= 0 || c.nlayers <= 0 || c.vocab <= 0 || mc.n_experts <= 0 || mc.top_k <= 0 ||
        mc.n_shared < 0 || mc.kv_latent <= 0 || mc.rope_dim <= 0 || mc.nope_dim <= 0 || mc.v_dim <= 0)
        return fail(nullptr, CD_ERR_INVALID, "config contains a non-positive dimension");
    if (c.hd != mc.nope_dim + mc.rope_dim || c.q_dim != c.heads * c.hd || c.kv_dim != mc.kv_latent + mc.rope_dim || c.kv_heads != 1 || c.gqa_ratio != c.heads)
        return fail(nullptr, CD_ERR_INVALID, "cd_config of a MoE + MLA model: hd = nope_dim + rope_dim, q_dim = heads * hd, kv_dim = kv_latent + rope_dim, kv_heads = 1, gqa_ratio = heads");
    if (dtype != CD_DTYPE_F32 && dtype != CD_DTYPE_F16 && dtype != CD_DTYPE_BF16) return fail(nullptr, CD_ERR_UNSUPPORTED, "MoE + MLA weights are f32, f16 or bf16");
    if (mc.top_k > mc.n_experts || mc.top_k > 16) return fail(nullptr, CD_ERR_INVALID, "top_k must not exceed n_experts (and 16)");
    if (c.heads > MLA_MAX_HEADS || mc.kv_latent > 512) return fail(nullptr, CD_ERR_UNSUPPORTED, "MLA attention supports at most 16 heads and a latent of 512");
    const int epc = dtype == CD_DTYPE_F32 ? 4 : 8;
    if (c.dim % 8 || c.hidden % 8 || mc.kv_latent % 8 || mc.rope_dim % 8 || mc.nope_dim % 8 || mc.v_dim % 8 || (c.heads * mc.v_dim) % 8)
        return fail(nullptr, CD_ERR_UNSUPPORTED, "dim, hidden and the MLA widths must be multiples of 8");
    if (c.dim > 8 * 256 * epc || c.heads * mc.v_dim > 8 * 256 * epc) return fail(nullptr, CD_ERR_UNSUPPORTED, "inner dimension too large for the GEMV tiling");
    if (world > 1 && (mc.n_experts % world || (mc.n_shared * c.hidden) % (8 * world)))
        return fail(nullptr, CD_ERR_UNSUPPORTED, "n_experts and the shared FFN's columns / 8 must be divisible by the expert-parallel world size");
    return CD_OK;
}

int model_alloc(const cd_config* cfg, const cd_options* opts_in, int untied, cd_model** out, const cd_moe_config* moe) {
    *out = nullptr;
    cd_options opts;
    memset(&opts, 0, sizeof(opts));
    opts.device = -1;
    if (opts_in) opts = *opts_in;
    int rc = moe ? validate_moe(*cfg, *moe, opts.weight_dtype, std::max(1, (int)opts.tp_world)) : validate(*cfg, opts.weight_dtype);
    if (rc) return rc;
    const int tpw = std::max(1, (int)opts.tp_world), tpr = tpw > 1 ? (int)opts.tp_rank : 0;
    // the KV cache's storage: fp32 with fp32 weights, otherwise 16 bits (fp16 unless bf16 is asked for)
    const int wdt = opts.weight_dtype;
    int kvdt;
    switch (opts.kv_dtype) {
        case CD_KV_AUTO: kvdt = wdt == CD_DTYPE_F32 ? CD_DTYPE_F32 : CD_DTYPE_F16; break;
        case CD_KV_F32: kvdt = CD_DTYPE_F32; break;
        case CD_KV_F16: kvdt = CD_DTYPE_F16; break;
        case CD_KV_BF16: kvdt = CD_DTYPE_BF16; break;
        default: return fail(nullptr, CD_ERR_INVALID, "unknown KV-cache dtype");
    }
    if ((wdt == CD_DTYPE_F32) != (kvdt == CD_DTYPE_F32) || (wdt == CD_DTYPE_F16 && kvdt != CD_DTYPE_F16))
        return fail(nullptr, CD_ERR_UNSUPPORTED, "KV-cache dtype: fp32 goes with fp32 weights, fp16 with fp16 weights, fp16 or bf16 with bf16 / FP8 / INT4 weights");
    cd_config local = *cfg;
    if (tpw > 1 && moe) {
        if (tpw > TP_MAX || tpr < 0 || tpr >= tpw) return fail(nullptr, CD_ERR_INVALID, "expert-parallel rank / world out of range");
    } else if (tpw > 1) {
        if (opts.weight_dtype == CD_DTYPE_INT4_G32 && ((cfg->q_dim / tpw) % 32 || (cfg->hidden / tpw) % 32))
            return fail(nullptr, CD_ERR_UNSUPPORTED, "INT4 groups of 32 must not straddle tensor-parallel shards (q_dim/world and hidden/world multiples of 32)");
        if (tpw > TP_MAX || tpr < 0 || tpr >= tpw) return fail(nullptr, CD_ERR_INVALID, "tensor-parallel rank / world out of range");
        if (cfg->kv_heads % tpw || cfg->heads % tpw || cfg->hidden % (8 * tpw))
            return fail(nullptr, CD_ERR_UNSUPPORTED, "heads, kv_heads and hidden/8 must be divisible by the tensor-parallel world size");
        local.heads /= tpw; local.kv_heads /= tpw; local.hidden /= tpw; local.q_dim /= tpw; local.kv_dim /= tpw;
        if ((rc = validate(local, opts.weight_dtype))) return rc;
    }
    cd_model* m = new cd_model();
    m->full_cfg = *cfg;
    m->cfg = local;
    m->tp_world = tpw;
    m->tp_rank = tpr;
    {
        // the LM head is split by vocabulary blocks under tensor parallelism and replicated under expert parallelism
        const int hw = moe ? 1 : tpw, hr = moe ? 0 : tpr;
        const int nblk = (cfg->vocab + HEAD_BLOCK - 1) / HEAD_BLOCK, per = (nblk + hw - 1) / hw;
        m->v0 = std::min(cfg->vocab, hr * per * HEAD_BLOCK);
        m->v_loc = std::min(cfg->vocab - m->v0, per * HEAD_BLOCK);
        m->tp_nb = per;  // head blocks per rank in the candidate exchange (the last rank may own fewer)
        if (m->v_loc <= 0) { delete m; return fail(nullptr, CD_ERR_UNSUPPORTED, "vocabulary too small for this tensor-parallel world size"); }
    }
    m->opt = opts;
    m->kv_dtype = kvdt;
    m->untied = untied;
    auto bail = [&](int code) { cd_model_destroy(m); return code; };
#define CKB(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { fail(nullptr, CD_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); return bail(CD_ERR_CUDA); } } while (0)
    int ndev = 0;
    CKB(cudaGetDeviceCount(&ndev));
    if (ndev == 0) { fail(nullptr, CD_ERR_CUDA, "no CUDA device"); return bail(CD_ERR_CUDA); }
    if (opts.device >= 0) CKB(cudaSetDevice(opts.device));
    CKB(cudaGetDevice(&m->device));
    cudaDeviceProp prop;
    CKB(cudaGetDeviceProperties(&prop, m->device));
    m->sm_count = prop.multiProcessorCount;
    CKB(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    CKB(cudaEventCreate(&m->ev0));
    CKB(cudaEventCreate(&m->ev1));

    const cd_config& c = m->cfg;
    const size_t es = esize(is_quant(opts.weight_dtype) ? CD_DTYPE_BF16 : opts.weight_dtype), kes = esize(kvdt);
    m->alpha = 1.0f / std::sqrt(2.0f * (float)c.nlayers);  // lib.rs:201
    m->page_tokens = opts.page_tokens > 0 ? opts.page_tokens : 64;
    m->pages_per_seq = (c.seq + m->page_tokens - 1) / m->page_tokens;
    const int max_samples = std::max(1, opts.max_samples);
    m->num_pages = m->pages_per_seq * max_samples;
    m->nsplit = std::max(1, std::min(32, m->pages_per_seq));  // a slice is at most a few pages: one or two load rounds per CTA
    m->pdl = (opts.test_flags & 1) == 0;
    if (opts.test_ring_kb > 0) m->ring_kb = std::max(16, std::min(220, (int)opts.test_ring_kb));
    m->wait_ns = (unsigned long long)(opts.wait_us > 0 ? opts.wait_us : 2000000) * 1000ull;
    m->nblocks = (m->v_loc + HEAD_BLOCK - 1) / HEAD_BLOCK;  // head blocks of this rank's vocabulary shard

    // ---- weights: one arena
    const size_t D = c.dim, Q = c.q_dim, KV = c.kv_dim, H = c.hidden, V = c.vocab;
    size_t off = 0;
    auto carve = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    const size_t o_embed = carve(V * D * es);
    const size_t o_head = untied ? carve((size_t)m->v_loc * D * es) : o_embed + (size_t)m->v0 * D * es;  // tied: rows of the embedding
    const size_t o_gf = carve(D * 4);
    struct LO { size_t wqkv, wo, w13, w2, g1, g2; };
    std::vector<LO> lo(c.nlayers);
    if (!moe) for (auto& l : lo) {
        const int dt = opts.weight_dtype;
        l.wqkv = carve((Q + 2 * KV) * lin_row_bytes(dt, c.dim)); l.wo = carve(D * lin_row_bytes(dt, c.q_dim)); l.w13 = carve(2 * H * lin_row_bytes(dt, c.dim));
        l.w2 = carve(D * lin_row_bytes(dt, c.hidden)); l.g1 = carve(D * 4); l.g2 = carve(D * 4);
    }
    m->weight_bytes = off;
    CKB(cudaMalloc(&m->weight_arena, off));
    char* wb = (char*)m->weight_arena;
    m->embed = wb + o_embed; m->lm_head = wb + o_head; m->gamma_final = (float*)(wb + o_gf);
    m->layers.resize(c.nlayers);
    for (int l = 0; l < c.nlayers && !moe; ++l) {
        m->layers[l].wqkv = wb + lo[l].wqkv; m->layers[l].wo = wb + lo[l].wo; m->layers[l].w13 = wb + lo[l].w13;
        m->layers[l].w2 = wb + lo[l].w2; m->layers[l].gamma1 = (float*)(wb + lo[l].g1); m->layers[l].gamma2 = (float*)(wb + lo[l].g2);
    }
    // ---- KV pages
    // dense: K and V of every kv head; MoE + MLA: one [latent | rope key] row per position
    m->kv_layer_bytes = moe ? align_up((size_t)m->num_pages * m->page_tokens * c.kv_dim * kes, 256)
                            : align_up((size_t)m->num_pages * 2 * c.kv_heads * m->page_tokens * c.hd * kes, 256);
    CKB(cudaMalloc(&m->kv_arena, m->kv_layer_bytes * c.nlayers));
    CKB(cudaMemsetAsync(m->kv_arena, 0, m->kv_layer_bytes * c.nlayers, m->stream));
    for (int l = 0; l < c.nlayers; ++l) m->layers[l].kv = (char*)m->kv_arena + (size_t)l * m->kv_layer_bytes;
    // ---- workspace
    off = 0;
    const size_t o_xa = carve(D * 4), o_xb = carve(D * 4), o_q = carve(Q * 4), o_attn = carve(Q * 4), o_gate = carve(H * 4);
    const size_t o_logits = carve(V * 4), o_logits2 = carve(V * 4), o_norm = carve(D * 4);
    const size_t nparts = std::max(m->nsplit, (int)MEGA_MAX_PARTS);  // attention partials per head: split-K slices, or CTAs of the persistent kernel
    const size_t o_pacc = carve((size_t)c.heads * nparts * c.hd * 4), o_pml = carve((size_t)c.heads * nparts * 2 * 4);
    const size_t o_cnt = carve((c.heads + 2) * 4);  // attention arrivals per head, head-kernel arrivals, pushing-GEMV arrivals
    const size_t o_bv = carve(m->nblocks * 4), o_bi = carve(m->nblocks * 4);
    const size_t o_tv = carve((size_t)m->nblocks * CD_MAX_GPU_TOPK * 4), o_ti = carve((size_t)m->nblocks * CD_MAX_GPU_TOPK * 4);
    const size_t o_mx = carve(m->nblocks * 4), o_sm = carve(m->nblocks * 4);
    const size_t o_tok = carve(256), o_ring = carve((c.seq + 1) * 4), o_prompt = carve((c.seq + 1) * 4);
    const size_t o_st = carve(sizeof(DevState)), o_pt = carve((size_t)m->num_pages * 4);
    const int rope_hd = moe ? moe->rope_dim : c.hd;  // width the RoPE pairs run over
    const size_t o_rope = carve((size_t)c.seq * (rope_hd / 2) * sizeof(float2));
    const size_t o_gc = carve(64), o_ml = carve((size_t)c.nlayers * sizeof(MegaLayer));
    const size_t o_tr = carve((size_t)2 * (10 * c.nlayers + 2) * 8);
    const size_t o_gv = carve((size_t)tpw * m->tp_nb * CD_MAX_GPU_TOPK * 4), o_gi = carve((size_t)tpw * m->tp_nb * CD_MAX_GPU_TOPK * 4);
    CKB(cudaMalloc(&m->ws_arena, off));
    CKB(cudaMemsetAsync(m->ws_arena, 0, off, m->stream));
    char* ws = (char*)m->ws_arena;
    m->x_a = (float*)(ws + o_xa); m->x_b = (float*)(ws + o_xb); m->q = (float*)(ws + o_q); m->attn = (float*)(ws + o_attn);
    m->gate = (float*)(ws + o_gate); m->logits = (float*)(ws + o_logits); m->logits_capped = (float*)(ws + o_logits2); m->norm_final = (float*)(ws + o_norm);
    m->part_acc = (float*)(ws + o_pacc); m->part_ml = (float*)(ws + o_pml); m->counters = (unsigned int*)(ws + o_cnt);
    m->block_vals = (float*)(ws + o_bv); m->block_idxs = (uint32_t*)(ws + o_bi);
    m->topk_vals = (float*)(ws + o_tv); m->topk_idxs = (uint32_t*)(ws + o_ti);
    m->maxes = (float*)(ws + o_mx); m->sums = (float*)(ws + o_sm);
    m->out_token = (uint32_t*)(ws + o_tok); m->out_ring = (uint32_t*)(ws + o_ring); m->prompt_dev = (uint32_t*)(ws + o_prompt);
    m->st = (DevState*)(ws + o_st); m->page_table = (int*)(ws + o_pt); m->rope = (float2*)(ws + o_rope);
    m->grid_counter = (unsigned long long*)(ws + o_gc); m->mega_layers = ws + o_ml;
    m->tp_topk_vals = (float*)(ws + o_gv); m->tp_topk_idxs = (uint32_t*)(ws + o_gi);
    if (opts.test_flags & 4) m->mega_trace = (unsigned long long*)(ws + o_tr);  // test_flags bit 2: phase stamps of the persistent kernel

    if (!moe) {   // per-layer pointer table and tiling of the persistent kernel
        std::vector<MegaLayer> ml(c.nlayers);
        for (int l = 0; l < c.nlayers; ++l) {
            const cd_layer_dev& L = m->layers[l];
            ml[l] = MegaLayer{L.wqkv, L.wo, L.w13, L.w2, L.gamma1, L.gamma2, L.kv};
        }
        CKB(cudaMemcpyAsync(m->mega_layers, ml.data(), ml.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice, m->stream));
        CKB(cudaStreamSynchronize(m->stream));
        const int epc = opts.weight_dtype == CD_DTYPE_F32 ? 4 : 8;
        const int nd = (c.dim / epc + 255) / 256, nh = (c.hidden / epc + 255) / 256;
        // (c is this rank's shard under tensor parallelism: hidden and q_dim shrink, dim does not)
        const bool combo = (nd == 1 && (nh == 1 || nh == 2)) || (nd == 2 && nh >= 3 && nh <= 6);
        if (combo && c.q_dim <= c.dim && c.gqa_ratio <= MEGA_MAX_GQA) { m->mega_nd = nd; m->mega_nh = nh == 3 ? 4 : nh == 5 ? 6 : nh; }
        // tensor parallel: measured on the 5B model, the persistent kernel wins at 2 ranks (601 against 569 tokens/s) and
        // loses at 8 (841 against 896), where a layer's data are 8 us and its fixed per-phase times dominate either way
        const bool mega_ok = !is_quant(opts.weight_dtype) && (tpw == 1 || (tpw == 2 && opts.weight_dtype != CD_DTYPE_F32));
        // one persistent kernel per token wherever its tiling covers the shape; test_flags bit 1 keeps one kernel per operator
        m->mega = (opts.test_flags & 2) == 0 && mega_ok && m->mega_nd > 0;
    }
    // identity page table; RoPE table from the host libm (sdpa_fwd.rs:18-33)
    {
        std::vector<int> pt(m->num_pages);
        for (int i = 0; i < m->num_pages; ++i) pt[i] = i;
        CKB(cudaMemcpyAsync(m->page_table, pt.data(), pt.size() * 4, cudaMemcpyHostToDevice, m->stream));
        std::vector<float2> rt((size_t)c.seq * (rope_hd / 2));
        for (int p = 0; p < c.seq; ++p)
            for (int i = 0; i < rope_hd / 2; ++i) {
                const float theta = (float)p / std::pow(10000.0f, 2.0f * (float)i / (float)rope_hd);
                rt[(size_t)p * (rope_hd / 2) + i] = make_float2(std::cos(theta), std::sin(theta));
            }
        CKB(cudaMemcpyAsync(m->rope, rt.data(), rt.size() * sizeof(float2), cudaMemcpyHostToDevice, m->stream));
        CKB(cudaStreamSynchronize(m->stream));
    }
    CKB(cudaMallocHost(&m->h_ring, (c.seq + 1) * 4));
    CKB(cudaMallocHost(&m->h_state, sizeof(DevState)));
    CKB(cudaMallocHost(&m->h_in, 16));
    if (tpw > 1) {  // the region the peers write into: its own allocation, so it can be shared through CUDA IPC
        // dense 16-bit models also run the prompt as GEMMs: two buffers of partial sums for up to seq prompt rows
        if (!moe && (opts.weight_dtype == CD_DTYPE_BF16 || opts.weight_dtype == CD_DTYPE_F16)) m->tp_pf_rows = ((size_t)c.seq + 127) / 128 * 128;
        const size_t bytes = TpRegion::bytes_with_prefill(tpw, c.dim, m->tp_nb, m->tp_pf_rows);
        CKB(cudaMalloc((void**)&m->link_region, bytes));
        CKB(cudaMemset(m->link_region, 0, bytes));
        CKB(cudaMemset(m->link_region, 0xff, TpRegion::cand_off(tpw, c.dim)));  // inbox: every word "not arrived"
        m->tp.world = tpw; m->tp.rank = tpr; m->tp.dim = c.dim; m->tp.st = m->st; m->tp.wait_ns = m->wait_ns;
        m->tp.peers[tpr] = m->link_region;
    }
    // gammas default to 1 (LayerWeights::random, layer.rs:711-712)
    {
        std::vector<float> ones(D, 1.0f);
        CKB(cudaMemcpy(m->gamma_final, ones.data(), D * 4, cudaMemcpyHostToDevice));
        for (auto& L : m->layers) {
            if (moe) break;
            CKB(cudaMemcpy(L.gamma1, ones.data(), D * 4, cudaMemcpyHostToDevice));
            CKB(cudaMemcpy(L.gamma2, ones.data(), D * 4, cudaMemcpyHostToDevice));
        }
    }
#undef CKB
    *out = m;
    return CD_OK;
}

// where a reference tensor lands in the device layout
struct Placement {
    void* dst;
    int in, out, transposed, row_mul, row_off;
    bool vec;  // fp32 vector (gamma)
    int full_in, full_out, in0, out0;  // the shard's place inside the reference's full tensor
};

static int place(cd_model* m, int layer, int which, Placement* p) {
    const cd_config& c = m->cfg;        // local (sharded) sizes
    const cd_config& f = m->full_cfg;   // reference sizes
    const int r = m->tp_rank;
    const size_t rb = lin_row_bytes(m->opt.weight_dtype, c.dim);  // a row of wqkv
    if (which == T_EMBED) { *p = {m->embed, c.dim, f.vocab, 0, 1, 0, false, f.dim, f.vocab, 0, 0}; return CD_OK; }
    if (which == T_LM_HEAD) {
        if (!m->untied) return fail(m, CD_ERR_INVALID, "model has a tied head");
        *p = {m->lm_head, c.dim, m->v_loc, 0, 1, 0, false, f.dim, f.vocab, 0, m->v0};
        return CD_OK;
    }
    if (which == T_GAMMA_FINAL) { *p = {m->gamma_final, c.dim, 1, 0, 1, 0, true, c.dim, 1, 0, 0}; return CD_OK; }
    if (layer < 0 || layer >= c.nlayers) return fail(m, CD_ERR_INVALID, "layer index out of range");
    cd_layer_dev& L = m->layers[layer];
    switch (which) {  // heads and FFN columns are split across ranks; Wo and W2 are split along their input
        case T_WQ: *p = {L.wqkv, c.dim, c.q_dim, 1, 1, 0, false, f.dim, f.q_dim, 0, r * c.q_dim}; break;
        case T_WK: *p = {(char*)L.wqkv + (size_t)c.q_dim * rb, c.dim, c.kv_dim, 1, 1, 0, false, f.dim, f.kv_dim, 0, r * c.kv_dim}; break;
        case T_WV: *p = {(char*)L.wqkv + (size_t)(c.q_dim + c.kv_dim) * rb, c.dim, c.kv_dim, 1, 1, 0, false, f.dim, f.kv_dim, 0, r * c.kv_dim}; break;
        case T_WO: *p = {L.wo, c.q_dim, c.dim, 1, 1, 0, false, f.q_dim, f.dim, r * c.q_dim, 0}; break;
        case T_W1: *p = {L.w13, c.dim, c.hidden, 1, 2, 0, false, f.dim, f.hidden, 0, r * c.hidden}; break;
        case T_W3: *p = {L.w13, c.dim, c.hidden, 1, 2, 1, false, f.dim, f.hidden, 0, r * c.hidden}; break;
        case T_W2: *p = {L.w2, c.hidden, c.dim, 0, 1, 0, false, f.hidden, f.dim, r * c.hidden, 0}; break;  // already [out=dim, in=hidden]
        case T_GAMMA1: *p = {L.gamma1, c.dim, 1, 0, 1, 0, true, c.dim, 1, 0, 0}; break;
        case T_GAMMA2: *p = {L.gamma2, c.dim, 1, 0, 1, 0, true, c.dim, 1, 0, 0}; break;
        default: return fail(m, CD_ERR_INVALID, "unknown tensor id");
    }
    return CD_OK;
}

size_t model_tensor_elems(const cd_model* m, int which) {
    const cd_config& c = m->full_cfg;  // sizes of the tensors as stored in a checkpoint
    switch (which) {
        case T_EMBED: case T_LM_HEAD: return (size_t)c.vocab * c.dim;
        case T_GAMMA_FINAL: case T_GAMMA1: case T_GAMMA2: return c.dim;
        case T_WQ: case T_WO: return (size_t)c.dim * c.q_dim;
        case T_WK: case T_WV: return (size_t)c.dim * c.kv_dim;
        default: return (size_t)c.dim * c.hidden;
    }
}

static int ensure_staging(cd_model* m, size_t bytes) {
    if (m->staging_bytes >= bytes) return CD_OK;
    if (m->staging) cudaFree(m->staging);
    m->staging = nullptr; m->staging_bytes = 0;
    CK(m, cudaMalloc(&m->staging, bytes));
    m->staging_bytes = bytes;
    return CD_OK;
}

static int ensure_staging2(cd_model* m, size_t bytes) {
    if (m->staging2_bytes >= bytes) return CD_OK;
    if (m->staging2) cudaFree(m->staging2);
    m->staging2 = nullptr; m->staging2_bytes = 0;
    CK(m, cudaMalloc(&m->staging2, bytes));
    m->staging2_bytes = bytes;
    return CD_OK;
}

// staging2 holds this rank's output rows as [out, full_in] fp32 (whole rows, so that an input-split shard of
// Wo / W2 is quantised with the scales of the unsharded matrix); write columns in0 .. in0 + in - 1 to their
// place in the quantised row format
static int quantize_rows(cd_model* m, const Placement& p) {
    const int grid = std::min(p.out, m->sm_count * 8);
    if (m->opt.weight_dtype == CD_DTYPE_FP8_E4M3)
        quantize_fp8_rows_kernel<<<grid, 256, 0, m->stream>>>((const float*)m->staging2, (unsigned char*)p.dst, p.in, p.out, p.row_mul, p.row_off, p.full_in, p.in0);
    else
        quantize_int4_rows_kernel<<<grid, 256, 0, m->stream>>>((const float*)m->staging2, (unsigned char*)p.dst, p.in, p.out, p.row_mul, p.row_off, p.full_in, p.in0);
    CK(m, cudaGetLastError());
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

int model_set_tensor_f32(cd_model* m, int layer, int which, const float* host) {
    Placement p;
    int rc = place(m, layer, which, &p);
    if (rc) return rc;
    if (!host) return fail(m, CD_ERR_INVALID, "null tensor pointer");
    if (p.vec) { CK(m, cudaMemcpy(p.dst, host, (size_t)p.in * 4, cudaMemcpyHostToDevice)); return CD_OK; }
    const size_t n = (size_t)p.full_in * p.full_out;  // the whole reference tensor is staged; the kernel picks the shard
    rc = ensure_staging(m, n * 4);
    if (rc) return rc;
    CK(m, cudaMemcpyAsync(m->staging, host, n * 4, cudaMemcpyHostToDevice, m->stream));
    const dim3 grid((p.in + 31) / 32, (p.out + 31) / 32), block(32, 8);
    if (is_quant(m->opt.weight_dtype) && which >= T_WQ && which <= T_W2) {
        // this rank's output rows, whole, in GEMV orientation as fp32 first, then quantised row by row
        rc = ensure_staging2(m, (size_t)p.full_in * p.out * 4);
        if (rc) return rc;
        const dim3 gridf((p.full_in + 31) / 32, (p.out + 31) / 32);
        relayout_kernel<float><<<gridf, block, 0, m->stream>>>((const float*)m->staging, (float*)m->staging2, p.full_in, p.out, p.transposed, 1, 0,
                                                               p.full_in, p.full_out, 0, p.out0);
        return quantize_rows(m, p);
    }
    DISPATCH_WT(m->opt.weight_dtype, WT,
                relayout_kernel<WT><<<grid, block, 0, m->stream>>>((const float*)m->staging, (WT*)p.dst, p.in, p.out, p.transposed, p.row_mul, p.row_off,
                                                                   p.full_in, p.full_out, p.in0, p.out0));
    CK(m, cudaGetLastError());
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

// Bytes of one linear as a quantised checkpoint stores it: full_out rows in GEMV orientation, each in the device's row
// format for its whole input width (FP8: codes, fp32 row scale, padding; INT4: nibbles, fp16 group scales, padding).
size_t model_quant_tensor_bytes(const cd_model* m, int which) {
    const cd_config& f = m->full_cfg;
    int in, out;
    switch (which) {
        case T_WQ: in = f.dim; out = f.q_dim; break;
        case T_WK: case T_WV: in = f.dim; out = f.kv_dim; break;
        case T_WO: in = f.q_dim; out = f.dim; break;
        case T_W1: case T_W3: in = f.dim; out = f.hidden; break;
        case T_W2: in = f.hidden; out = f.dim; break;
        default: return 0;
    }
    return (size_t)out * lin_row_bytes(m->opt.weight_dtype, in);
}

// Upload one linear from stored quantised rows (the whole matrix, see model_quant_tensor_bytes): this rank's rows, and of
// an input-split matrix (Wo, W2) this rank's columns with the whole row's scale (FP8) or its own groups' scales (INT4) -
// byte for byte what quantising the fp32 tensor at load produces.
int model_set_quant_rows(cd_model* m, int layer, int which, const void* host) {
    if (!is_quant(m->opt.weight_dtype) || which < T_WQ || which > T_W2) return fail(m, CD_ERR_INVALID, "stored quantised rows exist for the linears of a quantised model only");
    Placement p;
    int rc = place(m, layer, which, &p);
    if (rc) return rc;
    if (!host) return fail(m, CD_ERR_INVALID, "null tensor pointer");
    const int dt = m->opt.weight_dtype;
    const size_t sf = lin_row_bytes(dt, p.full_in), sl = lin_row_bytes(dt, p.in);
    const char* src = (const char*)host + (size_t)p.out0 * sf;
    char* dst = (char*)p.dst + (size_t)p.row_off * sl;
    const size_t dpitch = (size_t)p.row_mul * sl;
    if (dt == CD_DTYPE_FP8_E4M3) {
        CK(m, cudaMemcpy2DAsync(dst, dpitch, src + p.in0, sf, (size_t)p.in, (size_t)p.out, cudaMemcpyHostToDevice, m->stream));
        CK(m, cudaMemcpy2DAsync(dst + p.in, dpitch, src + p.full_in, sf, sl - (size_t)p.in, (size_t)p.out, cudaMemcpyHostToDevice, m->stream));
    } else {
        const size_t nib = (size_t)p.in / 2, sc = (size_t)p.in / 16;  // bytes of nibbles, of fp16 scales (one per 32 inputs)
        CK(m, cudaMemcpy2DAsync(dst, dpitch, src + p.in0 / 2, sf, nib, (size_t)p.out, cudaMemcpyHostToDevice, m->stream));
        CK(m, cudaMemcpy2DAsync(dst + nib, dpitch, src + p.full_in / 2 + p.in0 / 16, sf, sc, (size_t)p.out, cudaMemcpyHostToDevice, m->stream));
        if (sl > nib + sc) CK(m, cudaMemset2DAsync(dst + nib + sc, dpitch, 0, sl - nib - sc, (size_t)p.out, m->stream));
    }
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

// This rank's rows of one linear, in the device's row format for the local input width, to host memory.
int model_get_quant_rows(cd_model* m, int layer, int which, void* host, size_t cap) {
    if (!is_quant(m->opt.weight_dtype) || which < T_WQ || which > T_W2) return fail(m, CD_ERR_INVALID, "quantised rows exist for the linears of a quantised model only");
    Placement p;
    int rc = place(m, layer, which, &p);
    if (rc) return rc;
    const size_t sl = lin_row_bytes(m->opt.weight_dtype, p.in);
    if (!host || cap < (size_t)p.out * sl) return fail(m, CD_ERR_CAPACITY, "buffer too small for the tensor's rows");
    CK(m, cudaMemcpy2DAsync(host, sl, (const char*)p.dst + (size_t)p.row_off * sl, (size_t)p.row_mul * sl, sl, (size_t)p.out, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

// The embedding or the untied head (storage: 2 or 4 bytes per element) and the fp32 vectors, as stored on the device.
int model_get_plain(cd_model* m, int layer, int which, void* host, size_t cap) {
    Placement p;
    int rc = place(m, layer, which, &p);
    if (rc) return rc;
    if (!p.vec && which != T_EMBED && which != T_LM_HEAD) return fail(m, CD_ERR_INVALID, "not a plain tensor");
    const size_t bytes = p.vec ? (size_t)p.in * 4 : (size_t)p.in * p.out * esize(m->opt.weight_dtype);
    if (!host || cap < bytes) return fail(m, CD_ERR_CAPACITY, "buffer too small for the tensor");
    CK(m, cudaMemcpyAsync(host, p.dst, bytes, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

int model_set_tensor_synth(cd_model* m, int layer, int which, uint64_t seed, float std) {
    Placement p;
    int rc = place(m, layer, which, &p);
    if (rc) return rc;
    if (p.vec) return fail(m, CD_ERR_INVALID, "gammas are not synthesised");
    uint64_t uid = which == T_EMBED ? 0 : which == T_LM_HEAD ? 2 : synth_uid_layer(layer, which - T_WQ);
    const uint64_t key = synth_key(seed, uid);
    const float scale = std / 65536.0f;
    if (is_quant(m->opt.weight_dtype) && which >= T_WQ && which <= T_W2) {
        rc = ensure_staging2(m, (size_t)p.full_in * p.out * 4);
        if (rc) return rc;
        synth_kernel<float><<<m->sm_count * 8, 256, 0, m->stream>>>((float*)m->staging2, p.full_in, p.out, p.transposed, 1, 0, key, scale,
                                                                    p.full_in, p.full_out, 0, p.out0);
        return quantize_rows(m, p);
    }
    DISPATCH_WT(m->opt.weight_dtype, WT,
                synth_kernel<WT><<<m->sm_count * 8, 256, 0, m->stream>>>((WT*)p.dst, p.in, p.out, p.transposed, p.row_mul, p.row_off, key, scale,
                                                                      p.full_in, p.full_out, p.in0, p.out0));
    CK(m, cudaGetLastError());
    return CD_OK;
}

int model_finish(cd_model* m) {
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->staging) { cudaFree(m->staging); m->staging = nullptr; m->staging_bytes = 0; }
    if (m->staging2) { cudaFree(m->staging2); m->staging2 = nullptr; m->staging2_bytes = 0; }
    return CD_OK;
}

}  // namespace cd

// ====================================================================== C ABI
extern "C" {

const char* cd_last_error(const cd_model* m) { return m ? m->err.c_str() : g_error.c_str(); }

int cd_model_create(const cd_config* cfg, const cd_layer_init* layers, int nlayers, const cd_head_init* head,
                    const cd_options* opts, cd_model** out) {
    if (!cfg || !layers || !head || !out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    *out = nullptr;
    if (nlayers != cfg->nlayers) return fail(nullptr, CD_ERR_INVALID, "layer count does not match cfg.nlayers");  // lib.rs:184
    cd_model* m = nullptr;
    int rc = model_alloc(cfg, opts, head->lm_head != nullptr, &m);
    if (rc) return rc;
    auto set = [&](int l, int which, const float* p) { if (rc == CD_OK) rc = model_set_tensor_f32(m, l, which, p); };
    set(0, T_EMBED, head->embed);
    set(0, T_GAMMA_FINAL, head->gamma_final);
    if (head->lm_head) set(0, T_LM_HEAD, head->lm_head);
    for (int l = 0; l < nlayers; ++l) {
        const cd_layer_init& L = layers[l];
        set(l, T_WQ, L.wq); set(l, T_WK, L.wk); set(l, T_WV, L.wv); set(l, T_WO, L.wo);
        set(l, T_W1, L.w1); set(l, T_W3, L.w3); set(l, T_W2, L.w2); set(l, T_GAMMA1, L.gamma1); set(l, T_GAMMA2, L.gamma2);
    }
    if (rc == CD_OK) rc = model_finish(m);
    if (rc) { g_error = m->err; cd_model_destroy(m); return rc; }
    *out = m;
    return CD_OK;
}

int cd_model_create_synthetic(const cd_config* cfg, const cd_options* opts, uint64_t seed, float std, int untied_head,
                              cd_model** out) {
    if (!cfg || !out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    *out = nullptr;
    cd_model* m = nullptr;
    int rc = model_alloc(cfg, opts, untied_head != 0, &m);
    if (rc) return rc;
    auto syn = [&](int l, int which) { if (rc == CD_OK) rc = model_set_tensor_synth(m, l, which, seed, std); };
    syn(0, T_EMBED);
    if (untied_head) syn(0, T_LM_HEAD);
    for (int l = 0; l < cfg->nlayers; ++l)
        for (int w = T_WQ; w <= T_W2; ++w) syn(l, w);
    if (rc == CD_OK) rc = model_finish(m);
    if (rc) { g_error = m->err; cd_model_destroy(m); return rc; }
    *out = m;
    return CD_OK;
}

void cd_model_destroy(cd_model* m) {
    if (!m) return;
    if (m->stream) cudaStreamSynchronize(m->stream);
    prefill_release(m);
    moe_release(m);
    for (auto& kv : m->graphs) cudaGraphExecDestroy(kv.second.exec);
    for (int r = 0; r < 8; ++r) if (m->peer_maps[r]) cudaIpcCloseMemHandle(m->peer_maps[r]);
    if (m->link_region) cudaFree(m->link_region);
    if (m->weight_arena) cudaFree(m->weight_arena);
    if (m->kv_arena) cudaFree(m->kv_arena);
    if (m->ws_arena) cudaFree(m->ws_arena);
    if (m->staging) cudaFree(m->staging);
    if (m->staging2) cudaFree(m->staging2);
    if (m->h_ring) cudaFreeHost(m->h_ring);
    if (m->h_state) cudaFreeHost(m->h_state);
    if (m->h_in) cudaFreeHost(m->h_in);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
}

int cd_model_get_config(const cd_model* m, cd_config* cfg, cd_options* opts, int* untied) {
    if (!m) return CD_ERR_INVALID;
    if (cfg) *cfg = m->full_cfg;
    if (opts) *opts = m->opt;
    if (untied) *untied = m->untied;
    return CD_OK;
}

// ---- tensor parallel plumbing: one process per GPU, link regions exchanged through CUDA IPC
int cd_tp_region_handle(cd_model* m, void* out, size_t cap) {
    if (!m || !out) return fail(m, CD_ERR_INVALID, "null argument");
    if (m->tp_world <= 1) return fail(m, CD_ERR_INVALID, "model was not created tensor-parallel");
    if (cap < sizeof(cudaIpcMemHandle_t)) return fail(m, CD_ERR_CAPACITY, "handle buffer too small (64 bytes)");
    cudaIpcMemHandle_t h;
    CK(m, cudaIpcGetMemHandle(&h, m->link_region));
    memcpy(out, &h, sizeof h);
    return CD_OK;
}

int cd_tp_connect(cd_model* m, const void* handles, int world) {
    if (!m || !handles) return fail(m, CD_ERR_INVALID, "null argument");
    if (world != m->tp_world) return fail(m, CD_ERR_INVALID, "handle count does not match the tensor-parallel world size");
    CK(m, cudaSetDevice(m->device));
    for (int r = 0; r < world; ++r) {
        if (r == m->tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)r * sizeof h, sizeof h);
        void* p = nullptr;
        CK(m, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        m->peer_maps[r] = p;
        m->tp.peers[r] = (char*)p;
    }
    m->tp_connected = true;
    return CD_OK;
}

int cd_tp_region_ptr(cd_model* m, void** out) {
    if (!m || !out) return fail(m, CD_ERR_INVALID, "null argument");
    if (m->tp_world <= 1) return fail(m, CD_ERR_INVALID, "model was not created tensor-parallel");
    *out = m->link_region;
    return CD_OK;
}

int cd_tp_connect_ptrs(cd_model* m, void* const* regions, int world) {
    if (!m || !regions) return fail(m, CD_ERR_INVALID, "null argument");
    if (world != m->tp_world) return fail(m, CD_ERR_INVALID, "region count does not match the tensor-parallel world size");
    for (int r = 0; r < world; ++r) {
        if (!regions[r]) return fail(m, CD_ERR_INVALID, "null link region");
        if (r != m->tp_rank) m->tp.peers[r] = (char*)regions[r];
    }
    m->tp_connected = true;
    return CD_OK;
}

static int tp_guard(cd_model* m, bool supported) {
    if (m->tp_world <= 1) return CD_OK;
    if (!m->tp_connected) return fail(m, CD_ERR_INVALID, "tensor-parallel model is not connected to its peers (cd_tp_connect)");
    if (!supported) return fail(m, CD_ERR_UNSUPPORTED, "not available on a tensor-parallel model: use the greedy entry points");
    return CD_OK;
}

int cd_len(const cd_model* m, size_t* len) {
    if (!m || !len) return CD_ERR_INVALID;
    *len = m->len;
    return CD_OK;
}

int cd_set_len(cd_model* m, size_t len) {
    if (!m) return CD_ERR_INVALID;
    m->len = std::min(len, (size_t)m->cfg.seq);
    return CD_OK;
}

int cd_seed_layer_cache_cf(cd_model* m, int layer, size_t live_len, const float* k_cf, const float* v_cf) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !k_cf || !v_cf) return fail(m, CD_ERR_INVALID, "null argument");
    const cd_config& c = m->cfg;
    if (layer < 0 || layer >= c.nlayers) return fail(m, CD_ERR_INVALID, "layer index out of range");
    live_len = std::min(live_len, (size_t)c.seq);
    const size_t n = (size_t)c.kv_dim * c.seq;
    int rc = cd::ensure_staging(m, 2 * n * 4);
    if (rc) return rc;
    float* sk = (float*)m->staging;
    float* sv = sk + n;
    CK(m, cudaMemcpyAsync(sk, k_cf, n * 4, cudaMemcpyHostToDevice, m->stream));
    CK(m, cudaMemcpyAsync(sv, v_cf, n * 4, cudaMemcpyHostToDevice, m->stream));
    DISPATCH_WT(m->kv_dtype, KT,
                seed_kv_kernel<KT><<<m->sm_count * 4, 256, 0, m->stream>>>(sk, sv, (KT*)m->layers[layer].kv, m->page_table, c.seq,
                                                                           (int)live_len, c.kv_heads, c.hd, m->page_tokens));
    count_launch(m);
    CK(m, cudaGetLastError());
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

int cd_decode_token(cd_model* m, const float* x_in, float* x_out) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !x_in || !x_out) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    CK(m, cudaMemcpyAsync(m->x_a, x_in, (size_t)m->cfg.dim * 4, cudaMemcpyHostToDevice, m->stream));
    if ((rc = set_state(m, 0))) return rc;
    StepParams p{0, HEAD_NONE};
    if ((rc = run_step(m, p))) return rc;
    CK(m, cudaMemcpyAsync(x_out, m->x_a, (size_t)m->cfg.dim * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(&m->h_in[2], &m->st->error, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->h_in[2]) return device_wait_failed(m, (int)m->h_in[2], "");
    m->len += 1;
    return CD_OK;
}

int cd_decode_token_from_id(cd_model* m, uint32_t token, float* x_out) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !x_out) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    if ((rc = set_state(m, token))) return rc;
    StepParams p{1, HEAD_NONE};
    if ((rc = run_step(m, p))) return rc;
    CK(m, cudaMemcpyAsync(x_out, m->x_a, (size_t)m->cfg.dim * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(&m->h_in[2], &m->st->error, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->h_in[2]) return device_wait_failed(m, (int)m->h_in[2], "");
    m->len += 1;
    return CD_OK;
}

static int argmax_common(cd_model* m, int input, uint32_t token, uint32_t* out) {
    int rc = set_state(m, token);
    if (rc) return rc;
    StepParams p{input, HEAD_ARGMAX};
    if ((rc = run_step(m, p))) return rc;
    CK(m, cudaMemcpyAsync(m->h_ring, m->out_token, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(&m->h_in[2], &m->st->error, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->h_in[2]) return device_wait_failed(m, (int)m->h_in[2], "");
    *out = m->h_ring[0];
    m->len += 1;
    return CD_OK;
}

int cd_decode_token_argmax(cd_model* m, const float* x_in, uint32_t* out) {
    if (!m || !x_in || !out) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    CK(m, cudaMemcpyAsync(m->x_a, x_in, (size_t)m->cfg.dim * 4, cudaMemcpyHostToDevice, m->stream));
    return argmax_common(m, 0, 0, out);
}

int cd_decode_token_argmax_from_id(cd_model* m, uint32_t token, uint32_t* out) {
    if (!m || !out) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    return argmax_common(m, 1, token, out);
}

int cd_decode_token_topk_from_id(cd_model* m, uint32_t token, size_t top_k, float* out_vals, uint32_t* out_idxs, size_t cap,
                                 size_t* count) {
    if (m) { int g_ = tp_guard(m, true); if (g_) return g_; }  // tensor parallel: every rank returns all ranks' candidates
    if (!m || !out_vals || !out_idxs || !count) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    if (top_k == 0) return fail(m, CD_ERR_INVALID, "top_k must be positive");
    if (top_k > CD_MAX_GPU_TOPK) return fail(m, CD_ERR_INVALID, "top_k exceeds metal decode top-k capacity");
    const int nblk_all = (m->full_cfg.vocab + HEAD_BLOCK - 1) / HEAD_BLOCK;  // == m->nblocks on one GPU
    const size_t n = (size_t)nblk_all * top_k;
    if (cap < n) return fail(m, CD_ERR_CAPACITY, "out_vals too small for top-k candidates");
    if ((rc = set_state(m, token))) return rc;
    StepParams p{1, HEAD_TOPK};
    p.k = (int)top_k;
    if ((rc = run_step(m, p))) return rc;
    if (m->tp_world > 1) {
        for (int r = 0; r < m->tp_world; ++r) {  // rank r's row of the gathered candidates holds its blocks, k entries each
            const int nb_r = std::min(m->tp_nb, nblk_all - r * m->tp_nb);
            if (nb_r <= 0) break;
            const size_t src = (size_t)r * m->tp_nb * 32, dst = (size_t)r * m->tp_nb * top_k, cnt = (size_t)nb_r * top_k * 4;
            CK(m, cudaMemcpyAsync(out_vals + dst, m->tp_topk_vals + src, cnt, cudaMemcpyDeviceToHost, m->stream));
            CK(m, cudaMemcpyAsync(out_idxs + dst, m->tp_topk_idxs + src, cnt, cudaMemcpyDeviceToHost, m->stream));
        }
    } else {
        CK(m, cudaMemcpyAsync(out_vals, m->topk_vals, n * 4, cudaMemcpyDeviceToHost, m->stream));
        CK(m, cudaMemcpyAsync(out_idxs, m->topk_idxs, n * 4, cudaMemcpyDeviceToHost, m->stream));
    }
    CK(m, cudaMemcpyAsync(&m->h_in[2], &m->st->error, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->h_in[2]) return device_wait_failed(m, (int)m->h_in[2], "");
    *count = n;
    m->len += 1;
    return CD_OK;
}

int cd_decode_token_block_stats_from_id(cd_model* m, uint32_t token, float inv_temperature, float softcap, float* out_maxes,
                                        float* out_sums, size_t cap, size_t* nblocks) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !out_maxes || !out_sums || !nblocks) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    if (cap < (size_t)m->nblocks) return fail(m, CD_ERR_CAPACITY, "out_maxes too small");
    if ((rc = set_state(m, token))) return rc;
    StepParams p{1, HEAD_STATS};
    p.inv_t = inv_temperature;
    p.softcap = softcap;
    if ((rc = run_step(m, p))) return rc;
    CK(m, cudaMemcpyAsync(out_maxes, m->maxes, (size_t)m->nblocks * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(out_sums, m->sums, (size_t)m->nblocks * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(&m->h_in[2], &m->st->error, 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    if (m->h_in[2]) return device_wait_failed(m, (int)m->h_in[2], "");
    *nblocks = (size_t)m->nblocks;
    m->len += 1;
    return CD_OK;
}

int cd_materialize_current_logits_block(cd_model* m, size_t block_idx, float softcap, float* out, size_t cap, size_t* valid) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !out || !valid) return fail(m, CD_ERR_INVALID, "null argument");
    if (block_idx >= (size_t)m->nblocks) return fail(m, CD_ERR_INVALID, "block_idx out of range");
    const size_t n = std::min<size_t>(HEAD_BLOCK, (size_t)m->cfg.vocab - block_idx * HEAD_BLOCK);
    if (cap < n) return fail(m, CD_ERR_CAPACITY, "out_logits too small");
    // The logits of the last step are still resident (the reference recomputes them from the
    // resident normalised hidden, lib.rs:997); softcap without temperature as lib.rs:1716-1719.
    const float* src = m->logits + block_idx * HEAD_BLOCK;
    if (softcap > 0.0f) {
        float* tmp = m->logits_capped;
        softcap_copy_kernel<<<1, 256, 0, m->stream>>>(src, tmp, (int)n, softcap);
        count_launch(m);
        CK(m, cudaGetLastError());
        src = tmp;
    }
    CK(m, cudaMemcpyAsync(out, src, n * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    *valid = n;
    return CD_OK;
}

static int fetch_logits(cd_model* m, float softcap, float* out) {
    const int V = m->cfg.vocab;
    const float* src = m->logits;
    if (softcap > 0.0f) {
        float* capped = m->logits_capped;
        softcap_copy_kernel<<<m->sm_count, 256, 0, m->stream>>>(m->logits, capped, V, softcap);
        count_launch(m);
        CK(m, cudaGetLastError());
        src = capped;
    }
    CK(m, cudaMemcpyAsync(out, src, (size_t)V * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    return CD_OK;
}

int cd_decode_token_logits_from_id(cd_model* m, uint32_t token, float softcap, float* out_logits) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !out_logits) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    if ((rc = set_state(m, token))) return rc;
    StepParams p{1, HEAD_LOGITS};
    if ((rc = run_step(m, p))) return rc;
    if ((rc = fetch_logits(m, softcap, out_logits))) return rc;
    m->len += 1;
    return CD_OK;
}

int cd_prefill(cd_model* m, const uint32_t* ids, size_t n, float softcap, float* last_logits) {
    if (m) { int g_ = tp_guard(m, last_logits == nullptr); if (g_) return g_; }
    if (!m || !ids || n == 0) return fail(m, CD_ERR_INVALID, "prompt must contain at least one token");
    int rc = check_room(m, n);
    if (rc) return rc;
    for (size_t i = 0; i < n; ++i)
        if ((rc = check_token(m, ids[i]))) return rc;
    CK(m, cudaMemcpyAsync(m->prompt_dev, ids, n * 4, cudaMemcpyHostToDevice, m->stream));
    // Prompts of a few tokens and up go through the batched tensor-core pass where the model
    // allows it (CD_PREFILL=token keeps the one-token-at-a-time path of inference.rs:650-670).
    const char* mode = getenv("CD_PREFILL");
    if (n >= 8 && !(mode && !strcmp(mode, "token"))) {
        CK(m, cudaEventRecord(m->ev0, m->stream));
        rc = prefill_batched(m, n);
        if (rc == CD_OK) {
            begin_loop_kernel<<<1, 1, 0, m->stream>>>(m->st, (int)(m->len + n), 0u, 0ull);
            count_launch(m);
            if (last_logits) {
                cudaError_t e = enqueue_head_only(m);
                if (e != cudaSuccess) return fail(m, CD_ERR_CUDA, std::string("head launch: ") + cudaGetErrorString(e));
            }
            CK(m, cudaEventRecord(m->ev1, m->stream));
            CK(m, cudaMemcpyAsync(m->h_state, m->st, sizeof(DevState), cudaMemcpyDeviceToHost, m->stream));
            if (last_logits) {
                if ((rc = fetch_logits(m, softcap, last_logits))) return rc;
            } else {
                CK(m, cudaStreamSynchronize(m->stream));
            }
            CK(m, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
            if (m->h_state->error) return device_wait_failed(m, m->h_state->error, " during the batched prompt pass");
            m->len += n;
            return CD_OK;
        }
        if (rc != CD_ERR_UNSUPPORTED) return rc;
    }
    begin_loop_kernel<<<1, 1, 0, m->stream>>>(m->st, (int)m->len, 0u, 0ull);
    count_launch(m);
    CK(m, cudaEventRecord(m->ev0, m->stream));
    for (size_t i = 0; i < n; ++i) {
        StepParams p{2, (i + 1 == n && last_logits) ? HEAD_LOGITS : HEAD_NONE};
        if ((rc = run_step(m, p))) return rc;
    }
    CK(m, cudaEventRecord(m->ev1, m->stream));
    if (last_logits) {
        if ((rc = fetch_logits(m, softcap, last_logits))) return rc;
    } else {
        CK(m, cudaStreamSynchronize(m->stream));
    }
    CK(m, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    m->len += n;
    return CD_OK;
}

static int decode_loop(cd_model* m, uint32_t first, size_t nsteps, StepParams p, uint64_t* rng, uint32_t* out_ids) {
    if (!m || !out_ids) return fail(m, CD_ERR_INVALID, "null argument");
    int rc = check_room(m, nsteps);
    if (rc) return rc;
    if ((rc = check_token(m, first))) return rc;
    if (nsteps == 0) return CD_OK;
    begin_loop_kernel<<<1, 1, 0, m->stream>>>(m->st, (int)m->len, first, rng ? *rng : 0ull);
    count_launch(m);
    CK(m, cudaGetLastError());
    CK(m, cudaEventRecord(m->ev0, m->stream));
    for (size_t i = 0; i < nsteps; ++i)
        if ((rc = run_step(m, p))) return rc;
    CK(m, cudaEventRecord(m->ev1, m->stream));
    CK(m, cudaMemcpyAsync(m->h_ring, m->out_ring, nsteps * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaMemcpyAsync(m->h_state, m->st, sizeof(DevState), cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    CK(m, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
    if (m->h_state->error) return device_wait_failed(m, m->h_state->error, "");
    memcpy(out_ids, m->h_ring, nsteps * 4);
    if (rng) *rng = m->h_state->rng;
    m->len += nsteps;
    return CD_OK;
}

int cd_decode_steps_greedy(cd_model* m, uint32_t first, size_t nsteps, uint32_t* out_ids) {
    StepParams p{1, LOOP_GREEDY};
    return decode_loop(m, first, nsteps, p, nullptr, out_ids);
}

int cd_decode_steps_topk(cd_model* m, uint32_t first, size_t nsteps, size_t top_k, float t, float softcap, uint64_t* rng,
                         uint32_t* out_ids) {
    if (m) { int g_ = tp_guard(m, true); if (g_) return g_; }  // tensor parallel: candidates are exchanged between the ranks
    if (!m || !rng) return fail(m, CD_ERR_INVALID, "null argument");
    if (top_k == 0 || top_k > CD_MAX_GPU_TOPK) return fail(m, CD_ERR_INVALID, "top_k exceeds metal decode top-k capacity");
    StepParams p{1, LOOP_TOPK};
    p.k = (int)std::min<size_t>(top_k, (size_t)m->cfg.vocab);  // decode.rs:140
    p.t = t;
    p.softcap = softcap;
    return decode_loop(m, first, nsteps, p, rng, out_ids);
}

int cd_decode_steps_fullvocab(cd_model* m, uint32_t first, size_t nsteps, float t, float softcap, uint64_t* rng,
                              uint32_t* out_ids) {
    if (m) { int g_ = tp_guard(m, true); if (g_) return g_; }  // tensor parallel: block statistics are exchanged between the ranks
    if (!m || !rng) return fail(m, CD_ERR_INVALID, "null argument");
    // (a vocabulary-sharded head exchanges one (max, sum) per block of every rank; the MoE model's head is replicated)
    if (m->nblocks > 256 || (m->moe == nullptr && m->tp_world * m->tp_nb > 256)) return fail(m, CD_ERR_UNSUPPORTED, "full-vocab block sampler supports at most 65536 vocabulary rows");
    StepParams p{1, LOOP_FULLVOCAB};
    p.t = t;
    p.inv_t = 1.0f / std::max(t, 1.17549435e-38f);  // decode.rs:174
    p.softcap = softcap;
    return decode_loop(m, first, nsteps, p, rng, out_ids);
}

int cd_decode_steps_samples(cd_model* m, const uint32_t* first_tokens, size_t nsamples, size_t nsteps, int mode, size_t top_k,
                            float temperature, float softcap, uint64_t* rng_states, uint32_t* out_ids) {
    if (m) { int g_ = tp_guard(m, false); if (g_) return g_; }
    if (!m || !first_tokens || !out_ids) return fail(m, CD_ERR_INVALID, "null argument");
    if (nsamples == 0 || nsamples > 16 || nsamples > (size_t)(m->num_pages / m->pages_per_seq))
        return fail(m, CD_ERR_CAPACITY, "sample count exceeds cd_options.max_samples (at most 16)");
    if (mode < CD_SAMPLES_GREEDY || mode > CD_SAMPLES_FULLVOCAB) return fail(m, CD_ERR_INVALID, "unknown sampling mode");
    if (mode != CD_SAMPLES_GREEDY && !rng_states) return fail(m, CD_ERR_INVALID, "null argument");
    if (mode == CD_SAMPLES_TOPK && (top_k == 0 || top_k > CD_MAX_GPU_TOPK)) return fail(m, CD_ERR_INVALID, "top_k exceeds metal decode top-k capacity");
    if (mode == CD_SAMPLES_FULLVOCAB && m->nblocks > 256) return fail(m, CD_ERR_UNSUPPORTED, "full-vocab block sampler supports at most 65536 vocabulary rows");
    int rc = check_room(m, nsteps);
    if (rc) return rc;
    for (size_t s = 0; s < nsamples; ++s)
        if ((rc = check_token(m, first_tokens[s]))) return rc;
    if (nsteps == 0) return CD_OK;
    rc = decode_samples(m, first_tokens, (int)nsamples, nsteps, mode, (int)std::min<size_t>(top_k, (size_t)m->cfg.vocab), temperature, softcap,
                        rng_states, out_ids);
    if (rc == CD_ERR_UNSUPPORTED) return fail(m, rc, "multi-sample decode needs a bf16 / fp16 single-GPU model");
    return rc;
}

int cd_profile_decode_step(cd_model* m, uint32_t token, float* ms_by_class, uint32_t* launches_by_class, size_t nclasses) {
    if (!m || !ms_by_class || !launches_by_class || nclasses < CLS_COUNT) return fail(m, CD_ERR_INVALID, "need room for 8 classes");
    int rc = check_room(m, 1);
    if (rc) return rc;
    if ((rc = check_token(m, token))) return rc;
    if ((rc = set_state(m, token))) return rc;
    CK(m, cudaStreamSynchronize(m->stream));
    m->profiling = true;
    m->prof_events.clear();
    m->prof_classes.clear();
    m->cur_cls = CLS_MISC;
    cudaEvent_t start;
    cudaEventCreate(&start);
    cudaEventRecord(start, m->stream);
    StepParams p{1, HEAD_ARGMAX};
    cudaError_t e = enqueue_step(m, p);
    m->profiling = false;
    cudaError_t e2 = cudaStreamSynchronize(m->stream);
    for (size_t i = 0; i < nclasses; ++i) { ms_by_class[i] = 0.f; launches_by_class[i] = 0; }
    cudaEvent_t prev = start;
    for (size_t i = 0; i < m->prof_events.size(); ++i) {
        float ms = 0.f;
        if (e == cudaSuccess && e2 == cudaSuccess) cudaEventElapsedTime(&ms, prev, m->prof_events[i]);
        ms_by_class[m->prof_classes[i]] += ms;
        launches_by_class[m->prof_classes[i]] += 1;
        if (prev != start) cudaEventDestroy(prev);
        prev = m->prof_events[i];
    }
    if (prev != start) cudaEventDestroy(prev);
    cudaEventDestroy(start);
    m->prof_events.clear();
    m->prof_classes.clear();
    if (e != cudaSuccess || e2 != cudaSuccess)
        return fail(m, CD_ERR_CUDA, std::string("profiled step: ") + cudaGetErrorString(e != cudaSuccess ? e : e2));
    m->len += 1;
    return CD_OK;
}

int cd_debug_phase_trace(cd_model* m, unsigned long long* out, size_t cap, size_t* n) {
    if (!m || !out || !n) return CD_ERR_INVALID;
    const size_t count = (size_t)2 * (10 * m->cfg.nlayers + 2);
    if (!m->mega_trace) return fail(m, CD_ERR_UNSUPPORTED, "phase tracing is off (cd_options.test_flags bit 2 when the model is created)");
    if (cap < count) return fail(m, CD_ERR_CAPACITY, "trace buffer too small");
    CK(m, cudaMemcpy(out, m->mega_trace, count * 8, cudaMemcpyDeviceToHost));
    *n = count;
    return CD_OK;
}

int cd_last_device_ms(const cd_model* m, float* ms) {
    if (!m || !ms) return CD_ERR_INVALID;
    *ms = m->last_ms;
    return CD_OK;
}

int cd_kernel_launches(const cd_model* m, uint64_t* n) {
    if (!m || !n) return CD_ERR_INVALID;
    *n = m->launches;
    return CD_OK;
}

}  // extern "C"
