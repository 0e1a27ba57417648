// Batch-1 decode kernels for sm_100a.  Every kernel here is HBM-bound: the design
// rule is "each weight / KV byte crosses HBM once per token, as 16-byte coalesced
// loads with enough of them in flight per SM", with all element-wise work
// (RMSNorm, RoPE, KV append, SwiGLU, residuals) folded into GEMV prologues and
// epilogues so that activations never make a separate trip.
#pragma once
#include "common.cuh"

namespace cd {

// ====================================================================== GEMV
// y[r] = sum_k W[r, k] * x[k] over a [N, K] matrix stored K-contiguous.
//
// A CTA owns a contiguous range of rows.  Its consumer threads walk each row
// together: thread t owns the 16-byte chunks t, t+256, ... of every row, so its
// slice of x lives in registers for the whole kernel and one row is read as one
// contiguous burst.  Per-warp partial sums go through shared memory once per row;
// the last phase adds them and runs the epilogue functor on UNIT consecutive rows.
//
// NORM fuses rmsnorm_single (lib.rs:1354-1378): x * rsqrt(mean(x^2)+eps) * gamma.

struct EpiStore {  // plain y (LM head logits)
    float* out;
    __device__ void operator()(int unit, const float (&y)[1]) const { out[unit] = y[0]; }
};

struct EpiResidual {  // residual_add, lib.rs:1491-1502 / w2_proj beta=1, :1189-1201
    const float* res;
    float* out;
    float alpha;
    __device__ void operator()(int unit, const float (&y)[1]) const { out[unit] = __ldcg(res + unit) + alpha * y[0]; }
};

struct EpiGate {  // silu_gate, lib.rs:1504-1513; rows (2j, 2j+1) hold w1 and w3 column j
    float* gate;
    int act;
    __device__ void operator()(int unit, const float (&y)[2]) const {
        float a;
        if (act == 1) {  // LeakyReLU^2 (layer.rs:826-830)
            const float l = fmaxf(y[0], 0.5f * y[0]);
            a = l * l;
        } else {
            const float sig = 1.0f / (1.0f + expf(-y[0]));
            a = y[0] * sig;
        }
        gate[unit] = a * y[1];
    }
};

// rope_inplace + append_kv (lib.rs:1392-1424) on the fused [q | k | v] rows.
// cos/sin come from a host-built table [seq, hd/2] (the formula of
// sdpa_fwd.rs:18-33 evaluated once with the host libm).  K and V go straight
// into the paged cache: page = [2 (k,v)][kv_heads][page_tokens][hd].
template <typename KT> struct EpiQKV {
    float* q_out;
    KT* kv_pool;  // this layer's pages
    const int* page_table;
    const DevState* st;
    const float2* rope;  // [seq, hd/2] (cos, sin)
    int Q, KV, hd, kv_heads, page_tokens;
    __device__ void operator()(int unit, const float (&y)[2]) const {
        const int r = unit * 2;
        const int pos = __ldcg(&st->pos);
        if (r < Q + KV) {
            const int i = (r % hd) >> 1;
            const float2 cs = rope[(size_t)pos * (hd >> 1) + i];
            const float e = y[0] * cs.x - y[1] * cs.y;
            const float o = y[1] * cs.x + y[0] * cs.y;
            if (r < Q) {
                q_out[r] = e;
                q_out[r + 1] = o;
                return;
            }
            const int rk = r - Q, head = rk / hd, d = rk % hd;
            const int page = page_table[pos / page_tokens], off = pos % page_tokens;
            KT* dst = kv_pool + ((((size_t)page * 2 + 0) * kv_heads + head) * page_tokens + off) * hd + d;
            dst[0] = Elem<KT>::from_f32(e);
            dst[1] = Elem<KT>::from_f32(o);
        } else {
            const int rv = r - Q - KV, head = rv / hd, d = rv % hd;
            const int page = page_table[pos / page_tokens], off = pos % page_tokens;
            KT* dst = kv_pool + ((((size_t)page * 2 + 1) * kv_heads + head) * page_tokens + off) * hd + d;
            dst[0] = Elem<KT>::from_f32(y[0]);
            dst[1] = Elem<KT>::from_f32(y[1]);
        }
    }
};

// Tensor parallel: the partial vector of a row-sharded Wo / W2 product goes straight into
// every rank's inbox (own included); see TpRegion.
struct EpiPush {
    TpLink tp;
    __device__ void operator()(int unit, const float (&y)[1]) const {
        const unsigned int seq = __ldcg(&tp.st->ar_base) + (unsigned int)tp.ar_out;
        const size_t at = ((size_t)(seq % 3u) * tp.world + tp.rank) * tp.dim + unit;
        const float v = tp_sanitize(y[0]);
        for (int p = 0; p < tp.world; ++p) reinterpret_cast<float*>(tp.peers[p])[at] = v;
    }
};

// silu_gate over the chosen experts of a mixture-of-experts FFN: unit u belongs to entry u / hidden of the
// compact list of chosen local experts (its router weight multiplies the gate) or, past the list, to the
// shared FFN (weight 1).
struct EpiGateMoe {
    float* gate;
    const float* loc_w;
    const int* n_loc;
    int hidden;
    __device__ void operator()(int unit, const float (&y)[2]) const {
        const int s = unit / hidden;
        const float w = s < __ldcg(n_loc) ? __ldcg(loc_w + s) : 1.0f;
        gate[unit] = (y[0] / (1.0f + expf(-y[0]))) * y[1] * w;
    }
};

// ---------------------------------------------------------------------- where the rows of a GEMV come from
// SrcPlain: one matrix, row r at W + r * row_bytes.  The two expert sources assemble a virtual matrix from
// the experts the router chose for this token (a device-side list, so the kernel reads its shape after
// waiting for the previous kernel): the producer's copies gather it, the consumers see plain rows.
constexpr int SRC_MAX_LIST = 16;  // entries of a chosen-expert list (top_k at most)
struct SrcPlain {
    static constexpr bool DYNAMIC = false;
};
// Rows in blocks: entry s of the list contributes seg_rows rows (expert list[s] of W), then tail_rows rows of `tail`.
// `list` is the CTA's shared-memory copy of loc_ids, nl its length.
struct SrcExpertRows {
    static constexpr bool DYNAMIC = true;
    const int* loc_ids;
    const int* n_loc;
    const void* tail;
    int seg_rows, tail_rows;
    __device__ int rows(int, int nl) const { return nl * seg_rows + tail_rows; }
    __device__ int cols(int K, int) const { return K; }
    __device__ void copy(uint32_t dst, const char* W, int row0, int nrows, uint32_t row_bytes, uint32_t bar, uint64_t policy, const int* list, int nl) const {
        auto addr = [&](int v) -> const char* {
            const int sg = v / seg_rows;
            return sg < nl ? W + ((size_t)list[sg] * seg_rows + (size_t)(v - sg * seg_rows)) * row_bytes
                           : reinterpret_cast<const char*>(tail) + (size_t)(v - nl * seg_rows) * row_bytes;
        };
        const int last = row0 + nrows - 1;
        if (row0 >= nl * seg_rows || row0 / seg_rows == last / seg_rows) {
            bulk_g2s_stream(dst, addr(row0), (uint32_t)nrows * row_bytes, bar, policy);
        } else {
            for (int j = 0; j < nrows; ++j) bulk_g2s_stream(dst + (uint32_t)j * row_bytes, addr(row0 + j), row_bytes, bar, policy);
        }
    }
};
// Columns in blocks: row r is the concatenation of row r of expert list[s] (seg_bytes each, the expert's matrix has
// mat_rows rows) for every list entry, then row r of `tail` (tail_bytes).
struct SrcExpertCols {
    static constexpr bool DYNAMIC = true;
    const int* loc_ids;
    const int* n_loc;
    const void* tail;
    int seg_cols, tail_cols, mat_rows;
    uint32_t seg_bytes, tail_bytes;
    __device__ int rows(int N, int) const { return N; }
    __device__ int cols(int, int nl) const { return nl * seg_cols + tail_cols; }
    __device__ void copy(uint32_t dst, const char* W, int row0, int nrows, uint32_t row_bytes, uint32_t bar, uint64_t policy, const int* list, int nl) const {
        for (int j = 0; j < nrows; ++j) {
            const uint32_t d = dst + (uint32_t)j * row_bytes;
            for (int sg = 0; sg < nl; ++sg)
                bulk_g2s_stream(d + (uint32_t)sg * seg_bytes, W + ((size_t)list[sg] * mat_rows + (size_t)(row0 + j)) * seg_bytes, seg_bytes, bar, policy);
            if (tail_bytes) bulk_g2s_stream(d + (uint32_t)nl * seg_bytes, reinterpret_cast<const char*>(tail) + (size_t)(row0 + j) * tail_bytes, tail_bytes, bar, policy);
        }
    }
};

// ---------------------------------------------------------------------- the weight stream
// The weight stream is decoupled from the math: one producer thread keeps a ring of
// shared-memory stages full with 1-D bulk copies (cp.async.bulk, completion on an
// mbarrier), eight consumer warps drain it.  One persistent CTA per SM owns a
// contiguous row range; a stage is R whole rows, i.e. one contiguous burst of
// R * row_stride bytes.  The ring takes most of the SM's shared memory (about 30 MB
// in flight across the GPU, several times HBM latency times bandwidth).  Under
// programmatic dependent launch the producer starts filling the ring as soon as the
// CTA is resident, before the previous kernel's results are visible; consumers wait
// (griddepcontrol.wait) before touching x.
constexpr int GEMV_CONSUMERS = 256;
constexpr int GEMV_TMA_THREADS = GEMV_CONSUMERS + 32;

// Consumers come in G groups of 256 threads.  Every group holds the same slice layout of x
// and takes every G-th row of a stage, so G = 2 doubles the warps that decode a stage
// (the quantised formats need the issue slots; the plain formats run with G = 1).
__device__ inline void gemv_group_bar(int group) { asm volatile("bar.sync %0, 256;" ::"r"(group + 1) : "memory"); }
__device__ inline void all_consumers_bar(int nthreads) { asm volatile("bar.sync 8, %0;" ::"r"(nthreads) : "memory"); }
__device__ inline float consumer_sum(float v, float* red, int group = 0) {  // red: 8 floats of this group
    const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & 7;
    v = warp_sum(v);
    gemv_group_bar(group);
    if (lane == 0) red[warp] = v;
    gemv_group_bar(group);
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < GEMV_CONSUMERS / 32; ++i) t += red[i];
    return t;
}

template <typename WT, int NITER, int R, int UNIT, bool NORM, class Epi, int G = 1, class Src = SrcPlain>
__global__ void __launch_bounds__(G * GEMV_CONSUMERS + 32, 1)
gemv_tma_kernel(const WT* __restrict__ W, const float* __restrict__ x, const float* __restrict__ gamma,
                float* __restrict__ norm_out, int N, int K, int rows_cap, int nstages, int* err, NextStream next,
                TpLink tp, Epi epi, Src src) {
    using F = Wfmt<WT>;
    __shared__ int src_list[SRC_MAX_LIST];
    int src_n = 0;
    if constexpr (Src::DYNAMIC) {  // the shape is the previous kernel's result; N and K arrive as its upper bounds
        pdl_wait();
        src_n = min(__ldcg(src.n_loc), SRC_MAX_LIST);
        if ((int)threadIdx.x < src_n) src_list[threadIdx.x] = __ldcg(src.loc_ids + threadIdx.x);  // visible after the barrier below
        N = src.rows(N, src_n);
        K = src.cols(K, src_n);
    }
    constexpr int EPC = F::EPC;
    constexpr int NW = GEMV_CONSUMERS / 32;  // warps per group: one partial sum per row from each
    constexpr int RG = R / G;                // rows of a stage per group
    static_assert(R % G == 0, "a stage must split evenly over the consumer groups");
    extern __shared__ __align__(128) unsigned char smraw[];
    const uint32_t row_bytes = F::row_stride(K);
    const uint32_t stage_bytes = R * row_bytes;
    float* partial = reinterpret_cast<float*>(smraw + (size_t)nstages * stage_bytes);  // [rows_cap][NW]
    float* red = partial + (size_t)rows_cap * NW;                                       // 32
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 32);                             // full[ns], empty[ns]
    const uint32_t ring = smem_addr(smraw);
    const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8u * nstages;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool producer = warp == G * NW;
    const int group = G == 1 ? 0 : warp / NW;  // a compile-time zero for the single-group kernels
    const int tid = G == 1 ? (int)threadIdx.x : (int)(threadIdx.x & (GEMV_CONSUMERS - 1));
    const int gwarp = G == 1 ? warp : (warp & (NW - 1));
    const int nchunks = K / EPC;
    const int nunits = N / UNIT;
    const int u0 = (int)((long long)blockIdx.x * nunits / gridDim.x);
    const int u1 = (int)((long long)(blockIdx.x + 1) * nunits / gridDim.x);
    const int r0 = u0 * UNIT, r1 = u1 * UNIT;
    const int ngroups = K > 0 ? (r1 - r0 + R - 1) / R : 0;  // K == 0 (an empty expert list and no tail): every output is zero

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, G * NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (producer) {  // ---- producer: weights do not depend on the previous kernel
        if (lane == 0) {
            const char* Wb = reinterpret_cast<const char*>(W) + (size_t)r0 * row_bytes;
            const uint64_t policy = l2_evict_first_policy();
            for (int g = 0; g < ngroups; ++g) {
                if (next.test_drop && blockIdx.x == 0 && g == ngroups - 1) break;  // test hook: this stage never arrives
                const int s = g % nstages;
                if (g >= nstages && !mbar_wait(empty0 + 8u * s, ((g / nstages) - 1) & 1)) {
                    atomicExch(err, DEV_ERR_EMPTY_WAIT);
                    break;
                }
                const int rows = min(R, (r1 - r0) - g * R);
                const uint32_t bytes = (uint32_t)rows * row_bytes;
                mbar_arrive_expect_tx(full0 + 8u * s, bytes);
                if constexpr (Src::DYNAMIC) src.copy(ring + (uint32_t)s * stage_bytes, reinterpret_cast<const char*>(W), r0 + g * R, rows, row_bytes, full0 + 8u * s, policy, src_list, src_n);
                else bulk_g2s_stream(ring + (uint32_t)s * stage_bytes, Wb + (size_t)g * stage_bytes, bytes, full0 + 8u * s, policy);
            }
            if (next.w != nullptr) {  // queue the next kernel's first bytes behind our own last loads
                const long long nu0 = (long long)blockIdx.x * next.nunits / gridDim.x;
                const long long nu1 = (long long)(blockIdx.x + 1) * next.nunits / gridDim.x;
                const char* nb = reinterpret_cast<const char*>(next.w) + (size_t)nu0 * next.unit * next.row_bytes;
                const size_t avail = (size_t)(nu1 - nu0) * next.unit * next.row_bytes;
                const uint32_t total = (uint32_t)min((size_t)next.bytes, avail) & ~15u;
                for (uint32_t off = 0; off < total; off += 16384u) bulk_prefetch_l2(nb + off, min(16384u, total - off));
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    float xr[NITER][EPC];
    float ss = 0.0f;
    const float* inbox = nullptr;  // tensor parallel: the input is res + alpha * (sum of the peers' partial vectors)
    if (tp.world > 1 && tp.in_reduce) {
        const unsigned int seq = __ldcg(&tp.st->ar_base) + (unsigned int)tp.in_reduce;
        float* base = reinterpret_cast<float*>(tp.peers[tp.rank]);
        inbox = base + (size_t)(seq % 3u) * tp.world * tp.dim;
        // re-arm the slot two all-reduces ahead (nobody reads or writes it now), split over the CTAs
        uint4* rearm = reinterpret_cast<uint4*>(base + (size_t)((seq + 2u) % 3u) * tp.world * tp.dim);
        const int n4 = group == 0 ? tp.world * tp.dim / 4 : 0;
        for (int j = blockIdx.x * GEMV_CONSUMERS + tid; j < n4; j += gridDim.x * GEMV_CONSUMERS)
            rearm[j] = make_uint4(TP_SENTINEL, TP_SENTINEL, TP_SENTINEL, TP_SENTINEL);
    }
#pragma unroll
    for (int i = 0; i < NITER; ++i) {
        const int c = tid + i * GEMV_CONSUMERS;
#pragma unroll
        for (int e = 0; e < EPC; e += 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < nchunks) {
                if (inbox != nullptr) {
                    float4 a;  // summed in fixed rank order: identical on every rank
                    if (!tp_gather4(inbox, tp.world, tp.dim, (size_t)c * EPC + e, a, tp.st, tp.wait_ns)) atomicCAS(err, 0, DEV_ERR_TP_WAIT);
                    const float4 r4 = __ldcg(reinterpret_cast<const float4*>(tp.res + (size_t)c * EPC + e));
                    v = make_float4(r4.x + tp.alpha * a.x, r4.y + tp.alpha * a.y, r4.z + tp.alpha * a.z, r4.w + tp.alpha * a.w);
                    if (blockIdx.x == 0 && group == 0) *reinterpret_cast<float4*>(tp.x_out + (size_t)c * EPC + e) = v;
                } else {
                    v = __ldcg(reinterpret_cast<const float4*>(x + (size_t)c * EPC + e));
                }
            }
            xr[i][e] = v.x; xr[i][e + 1] = v.y; xr[i][e + 2] = v.z; xr[i][e + 3] = v.w;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
    if (NORM) {
        const float tot = consumer_sum(ss, red + 8 * group, group);
        const float inv = 1.0f / sqrtf(tot * (1.0f / (float)K) + RMS_EPS);
#pragma unroll
        for (int i = 0; i < NITER; ++i) {
            const int c = tid + i * GEMV_CONSUMERS;
            if (c < nchunks) {
#pragma unroll
                for (int e = 0; e < EPC; e += 4) {
                    const float4 g = *reinterpret_cast<const float4*>(gamma + (size_t)c * EPC + e);
                    xr[i][e] = xr[i][e] * inv * g.x;
                    xr[i][e + 1] = xr[i][e + 1] * inv * g.y;
                    xr[i][e + 2] = xr[i][e + 2] * inv * g.z;
                    xr[i][e + 3] = xr[i][e + 3] * inv * g.w;
                    if (norm_out != nullptr && blockIdx.x == 0 && group == 0)
                        *reinterpret_cast<float4*>(norm_out + (size_t)c * EPC + e) =
                            make_float4(xr[i][e], xr[i][e + 1], xr[i][e + 2], xr[i][e + 3]);
                }
            }
        }
    }

    bool ok = true;
    const int wait_limit = next.test_drop ? (1 << 12) : MBAR_WAIT_LIMIT;  // the test hook's wait runs out in milliseconds
    for (int g = 0; g < ngroups; ++g) {
        const int s = g % nstages;
        if (!mbar_wait(full0 + 8u * s, (g / nstages) & 1, wait_limit)) {
            atomicExch(err, DEV_ERR_FULL_WAIT);
            ok = false;
            break;
        }
        const uint32_t base = ring + (uint32_t)s * stage_bytes;
        uint4 w[RG][NITER];
        uint32_t aux[RG][NITER];  // per-chunk scale bits
        float rs[RG];             // per-row scale
#pragma unroll
        for (int jj = 0; jj < RG; ++jj) {
            const int j = jj * G + group;  // this group's rows of the stage
#pragma unroll
            for (int i = 0; i < NITER; ++i) {
                const int c = tid + i * GEMV_CONSUMERS;
                w[jj][i] = make_uint4(0, 0, 0, 0);
                aux[jj][i] = 0;
                if (c < nchunks) {
                    if constexpr (F::CHUNK_BYTES == 16) {
                        w[jj][i] = lds128(base + (uint32_t)j * row_bytes + (uint32_t)c * 16u);
                    } else {
                        const uint2 t = *reinterpret_cast<const uint2*>(smraw + (size_t)s * stage_bytes + (size_t)j * row_bytes + (size_t)c * 8);
                        w[jj][i].x = t.x; w[jj][i].y = t.y;
                    }
                    if (F::CHUNK_SCALE)
                        aux[jj][i] = *reinterpret_cast<const unsigned short*>(smraw + (size_t)s * stage_bytes + (size_t)j * row_bytes + F::scale_off(K) + (size_t)(c >> F::SCALE_SHIFT) * 2);
                }
            }
            rs[jj] = 1.0f;
            if (F::ROW_SCALE) rs[jj] = *reinterpret_cast<const float*>(smraw + (size_t)s * stage_bytes + (size_t)j * row_bytes + F::scale_off(K));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8u * s);  // this warp holds its slice in registers: stage may be refilled
        float acc[RG];
#pragma unroll
        for (int j = 0; j < RG; ++j) {
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < NITER; ++i) a = F::dot(w[j][i], aux[j][i], xr[i], a);
            acc[j] = F::ROW_SCALE ? a * rs[j] : a;
        }
        int rr;
        const float tot = warp_reduce_rows<RG>(acc, lane, rr);
        const int row = g * R + rr * G + group;  // rows past the range were never copied: their sums are dropped
        if ((lane & (32 / RG - 1)) == 0 && row < r1 - r0) partial[row * NW + gwarp] = tot;
    }
    if (!ok) {
        // leave only once the copies that may still be in flight have landed (bounded)
        for (int s = 0; s < nstages; ++s) mbar_wait(full0 + 8u * s, 0, wait_limit);
    }
    all_consumers_bar(G * GEMV_CONSUMERS);
    if (!ok) return;
    for (int u = threadIdx.x; u < u1 - u0; u += G * GEMV_CONSUMERS) {
        float y[UNIT];
#pragma unroll
        for (int k = 0; k < UNIT; ++k) {
            float sacc = 0.0f;
#pragma unroll
            for (int wi = 0; wi < NW; ++wi) sacc += partial[(u * UNIT + k) * NW + wi];
            y[k] = ngroups > 0 ? sacc : 0.0f;
        }
        epi(u0 + u, y);
    }
}

// ====================================================================== embedding gather
// embed_lookup, lib.rs:1380-1390; the token id is read from the device state.
template <typename WT>
__global__ void embed_kernel(const WT* __restrict__ embed, DevState* st, float* __restrict__ x, int D, int vocab) {
    const uint32_t tok = checked_token(st->token, vocab, &st->error);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < D; i += gridDim.x * blockDim.x)
        x[i] = Elem<WT>::to_f32(embed[(size_t)tok * D + i]);
}

// ====================================================================== split-K flash-decode attention
// sdpa_causal (lib.rs:1426-1489) for one query token over the paged cache.
// grid = (heads, nsplit): each CTA takes one head and one contiguous slice of the
// context (a whole number of pages) in a single pass with a running softmax
// (max, sum, weighted V) per token lane-group; groups are merged in shared memory
// and the slice result goes to scratch.  The CTA that arrives last for a head
// (atomic counter, no waiting) merges the slices, normalises and writes
// attn_out[head*hd ..].  A token's key (or value) row for one head is hd contiguous
// elements: LPT lanes load it as 16-byte chunks, 128/LPT tokens side by side, UNR
// tokens deep, so K and V of a 64-token page are in flight at once.
template <typename KT, int HD>
__device__ __forceinline__ void
attn_decode_body(const float* __restrict__ q, const KT* __restrict__ kv_pool, const int* __restrict__ page_table,
                 const DevState* st, float* __restrict__ part_acc, float* __restrict__ part_ml,
                 unsigned int* __restrict__ counters, float* __restrict__ attn_out, int kv_heads, int gqa,
                 int page_tokens, int nsplit, float scale) {
    constexpr int EPC = Elem<KT>::EPC;
    constexpr int LPT = HD / EPC;   // lanes per token row
    constexpr int NG = 128 / LPT;   // tokens side by side
    constexpr int UNR = 8;
    constexpr float NEG = -3.402823466e+38f;
    __shared__ float accs[NG * HD];
    __shared__ float gm[NG], gl[NG];
    __shared__ int is_last;

    const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
    const int g = tid / LPT, l = tid % LPT;
    const int kvh = h / gqa;
    const size_t head_stride = (size_t)page_tokens * HD;        // one head's rows inside a page
    const size_t page_stride = (size_t)2 * kv_heads * head_stride;
    pdl_wait();  // q, the new K/V row and the position come from the previous kernel
    pdl_launch_dependents();
    const int attn_len = __ldcg(&st->pos) + 1;
    int per = (attn_len + nsplit - 1) / nsplit;
    per = ((per + page_tokens - 1) / page_tokens) * page_tokens;
    const int t0 = s * per, t1 = min(attn_len, t0 + per);

    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; e += 4) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(q + (size_t)h * HD + l * EPC + e));
        qf[e] = v.x; qf[e + 1] = v.y; qf[e + 2] = v.z; qf[e + 3] = v.w;
    }

    float m = NEG, lsum = 0.0f;
    float acc[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) acc[e] = 0.0f;
    for (int tb = t0; tb < t1; tb += NG * UNR) {  // bounds are uniform across the CTA (shuffles inside)
        uint4 kw[UNR], vw[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int t = tb + g + u * NG;
            if (t < t1) {
                const int page = page_table[t / page_tokens], off = t % page_tokens;
                const KT* kp = kv_pool + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)off * HD + l * EPC;
                kw[u] = ldg_stream_coherent(kp);
                vw[u] = ldg_stream_coherent(kp + (size_t)kv_heads * head_stride);
            } else {
                kw[u] = make_uint4(0, 0, 0, 0);
                vw[u] = make_uint4(0, 0, 0, 0);
            }
        }
        float sc[UNR];
        float mnew = m;
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            float f[EPC];
            Elem<KT>::unpack(kw[u], f);
            float d = 0.0f;
#pragma unroll
            for (int e = 0; e < EPC; ++e) d = fmaf(qf[e], f[e], d);
#pragma unroll
            for (int o = LPT / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            sc[u] = (tb + g + u * NG < t1) ? d * scale : NEG;
            mnew = fmaxf(mnew, sc[u]);
        }
        if (mnew > NEG) {
            const float corr = expf(m - mnew);
            lsum *= corr;
#pragma unroll
            for (int e = 0; e < EPC; ++e) acc[e] *= corr;
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                if (tb + g + u * NG < t1) {
                    const float p = expf(sc[u] - mnew);
                    lsum += p;
                    float f[EPC];
                    Elem<KT>::unpack(vw[u], f);
#pragma unroll
                    for (int e = 0; e < EPC; ++e) acc[e] = fmaf(p, f[e], acc[e]);
                }
            }
            m = mnew;
        }
    }
    // ---- merge the NG lane-groups
#pragma unroll
    for (int e = 0; e < EPC; ++e) accs[g * HD + l * EPC + e] = acc[e];
    if (l == 0) { gm[g] = m; gl[g] = lsum; }
    __syncthreads();
    const size_t slot = (size_t)h * nsplit + s;
    if (tid < HD) {
        float M = NEG;
#pragma unroll
        for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, gm[gg]);
        float L = 0.0f, a = 0.0f;
#pragma unroll
        for (int gg = 0; gg < NG; ++gg) {
            if (gl[gg] > 0.0f) {
                const float wgt = expf(gm[gg] - M);
                L += gl[gg] * wgt;
                a += accs[gg * HD + tid] * wgt;
            }
        }
        part_acc[slot * HD + tid] = a;
        if (tid == 0) {
            part_ml[slot * 2 + 0] = M;
            part_ml[slot * 2 + 1] = L;
        }
    }

    // ---- last CTA of this head merges the slices
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(&counters[h], 1u);
        is_last = (prev == (unsigned)nsplit - 1u);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // slice weights first (one thread per slice, loads in parallel), then every output
    // lane sums its column with independent, unconditional loads
    float* wsl = accs;            // [nsplit] weight exp(m_s - M) (0 for empty slices)
    float* lsl = accs + 64;       // [nsplit] weight * sum
    float ms = NEG, ls = 0.0f;
    if (tid < nsplit) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + ((size_t)h * nsplit + tid) * 2));
        ms = ml.x;
        ls = ml.y;
    }
    float M = ls > 0.0f ? ms : NEG;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if ((tid & 31) == 0 && tid < 64) gl[tid >> 5] = M;  // nsplit <= 64: two warps can hold slices
    __syncthreads();
    M = fmaxf(gl[0], gl[1]);
    if (tid < nsplit) {
        const float wgt = ls > 0.0f ? expf(ms - M) : 0.0f;
        wsl[tid] = wgt;
        lsl[tid] = ls * wgt;
    }
    __syncthreads();
    if (tid < HD) {
        float L = 0.0f, o = 0.0f;
        const float* pa = part_acc + (size_t)h * nsplit * HD + tid;
#pragma unroll 8
        for (int ss = 0; ss < nsplit; ++ss) {
            L += lsl[ss];
            o += __ldcg(pa + (size_t)ss * HD) * wsl[ss];
        }
        attn_out[(size_t)h * HD + tid] = L > 0.0f ? o / L : 0.0f;
    }
    if (tid == 0) counters[h] = 0u;  // ready for the next layer / step
}

template <typename KT, int HD>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const float* __restrict__ q, const KT* __restrict__ kv_pool, const int* __restrict__ page_table,
                   const DevState* st, float* __restrict__ part_acc, float* __restrict__ part_ml,
                   unsigned int* __restrict__ counters, float* __restrict__ attn_out, int kv_heads, int gqa,
                   int page_tokens, int nsplit, float scale) {
    attn_decode_body<KT, HD>(q, kv_pool, page_table, st, part_acc, part_ml, counters, attn_out, kv_heads, gqa, page_tokens, nsplit, scale);
}

// Several samples that share a prompt and sit at the same position, NS of them per CTA (blockIdx.z
// picks the group): each sample has its own query, page table (prompt pages shared, later pages its
// own) and scratch [sample][head][slice].  A K/V tile that lies wholly inside the shared prompt
// pages (tokens < shared_tokens) is loaded once and applied to the NS queries; tiles that reach
// into the samples' own pages are loaded per sample.  Slices are multiples of the 32- or 64-token
// tile rather than of a page; the last-arriver merge runs per sample.
template <typename KT, int HD, int NS>
__global__ void __launch_bounds__(128)
attn_decode_group_kernel(const float* __restrict__ q, const KT* __restrict__ kv_pool, const int* __restrict__ page_table,
                         const DevState* st, float* __restrict__ part_acc, float* __restrict__ part_ml,
                         unsigned int* __restrict__ counters, float* __restrict__ attn_out, int kv_heads, int gqa,
                         int page_tokens, int nsplit, float scale, int pages_per_seq, int nsamples, int shared_tokens) {
    constexpr int EPC = Elem<KT>::EPC;
    constexpr int LPT = HD / EPC;
    constexpr int NG = 128 / LPT;
    constexpr int UNR = 4;
    constexpr int TILE = NG * UNR;
    constexpr float NEG = -3.402823466e+38f;
    __shared__ float accs[NG * HD];
    __shared__ float gm[NG], gl[NG];
    __shared__ int is_last;

    const int h = blockIdx.x, s = blockIdx.y, tid = threadIdx.x, heads = gridDim.x;
    const int z0 = blockIdx.z * NS, cnt = min(NS, nsamples - z0);
    const int g = tid / LPT, l = tid % LPT;
    const int kvh = h / gqa;
    const size_t head_stride = (size_t)page_tokens * HD;
    const size_t page_stride = (size_t)2 * kv_heads * head_stride;
    const int attn_len = __ldcg(&st->pos) + 1;
    int per = (attn_len + nsplit - 1) / nsplit;
    per = ((per + TILE - 1) / TILE) * TILE;
    const int t0 = s * per, t1 = min(attn_len, t0 + per);

    float qf[NS][EPC], acc[NS][EPC], m[NS], lsum[NS];
#pragma unroll
    for (int z = 0; z < NS; ++z) {
        m[z] = NEG;
        lsum[z] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPC; ++e) { acc[z][e] = 0.0f; qf[z][e] = 0.0f; }
        if (z < cnt) {
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(q + ((size_t)(z0 + z) * heads + h) * HD + l * EPC + e));
                qf[z][e] = v.x; qf[z][e + 1] = v.y; qf[z][e + 2] = v.z; qf[z][e + 3] = v.w;
            }
        }
    }
    for (int tb = t0; tb < t1; tb += TILE) {  // bounds are uniform across the CTA (shuffles inside)
        const bool shared = tb + TILE <= shared_tokens;
        uint4 kw[UNR], vw[UNR];
#pragma unroll
        for (int z = 0; z < NS; ++z) {
            if (z >= cnt) break;
            if (z == 0 || !shared) {
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const int t = tb + g + u * NG;
                    if (t < t1) {
                        const int page = page_table[(size_t)(z0 + z) * pages_per_seq + t / page_tokens], off = t % page_tokens;
                        const KT* kp = kv_pool + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)off * HD + l * EPC;
                        kw[u] = ldg_stream_coherent(kp);
                        vw[u] = ldg_stream_coherent(kp + (size_t)kv_heads * head_stride);
                    } else {
                        kw[u] = make_uint4(0, 0, 0, 0);
                        vw[u] = make_uint4(0, 0, 0, 0);
                    }
                }
            }
            float sc[UNR];
            float mnew = m[z];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                float f[EPC];
                Elem<KT>::unpack(kw[u], f);
                float d = 0.0f;
#pragma unroll
                for (int e = 0; e < EPC; ++e) d = fmaf(qf[z][e], f[e], d);
#pragma unroll
                for (int o = LPT / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                sc[u] = (tb + g + u * NG < t1) ? d * scale : NEG;
                mnew = fmaxf(mnew, sc[u]);
            }
            if (mnew > NEG) {
                const float corr = expf(m[z] - mnew);
                lsum[z] *= corr;
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[z][e] *= corr;
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    if (tb + g + u * NG < t1) {
                        const float p = expf(sc[u] - mnew);
                        lsum[z] += p;
                        float f[EPC];
                        Elem<KT>::unpack(vw[u], f);
#pragma unroll
                        for (int e = 0; e < EPC; ++e) acc[z][e] = fmaf(p, f[e], acc[z][e]);
                    }
                }
                m[z] = mnew;
            }
        }
    }
    // ---- per sample: merge the NG lane-groups, store this slice's partial
#pragma unroll
    for (int z = 0; z < NS; ++z) {
        if (z >= cnt) break;
        __syncthreads();
#pragma unroll
        for (int e = 0; e < EPC; ++e) accs[g * HD + l * EPC + e] = acc[z][e];
        if (l == 0) { gm[g] = m[z]; gl[g] = lsum[z]; }
        __syncthreads();
        const size_t slot = ((size_t)(z0 + z) * heads + h) * nsplit + s;
        if (tid < HD) {
            float M = NEG;
#pragma unroll
            for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, gm[gg]);
            float L = 0.0f, a = 0.0f;
#pragma unroll
            for (int gg = 0; gg < NG; ++gg) {
                if (gl[gg] > 0.0f) {
                    const float wgt = expf(gm[gg] - M);
                    L += gl[gg] * wgt;
                    a += accs[gg * HD + tid] * wgt;
                }
            }
            part_acc[slot * HD + tid] = a;
            if (tid == 0) {
                part_ml[slot * 2 + 0] = M;
                part_ml[slot * 2 + 1] = L;
            }
        }
    }
    // ---- the last CTA of this head (and group) merges the slices of every sample of the group
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(&counters[blockIdx.z * heads + h], 1u);
        is_last = (prev == (unsigned)nsplit - 1u);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float* wsl = accs;
    float* lsl = accs + 64;
    for (int z = 0; z < cnt; ++z) {
        const size_t base = ((size_t)(z0 + z) * heads + h) * nsplit;
        float ms = NEG, ls = 0.0f;
        if (tid < nsplit) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (base + tid) * 2));
            ms = ml.x;
            ls = ml.y;
        }
        float M = ls > 0.0f ? ms : NEG;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        __syncthreads();
        if ((tid & 31) == 0 && tid < 64) gl[tid >> 5] = M;
        __syncthreads();
        M = fmaxf(gl[0], gl[1]);
        if (tid < nsplit) {
            const float wgt = ls > 0.0f ? expf(ms - M) : 0.0f;
            wsl[tid] = wgt;
            lsl[tid] = ls * wgt;
        }
        __syncthreads();
        if (tid < HD) {
            float L = 0.0f, o = 0.0f;
            const float* pa = part_acc + base * HD + tid;
#pragma unroll 8
            for (int ss = 0; ss < nsplit; ++ss) {
                L += lsl[ss];
                o += __ldcg(pa + (size_t)ss * HD) * wsl[ss];
            }
            attn_out[((size_t)(z0 + z) * heads + h) * HD + tid] = L > 0.0f ? o / L : 0.0f;
        }
    }
    if (tid == 0) counters[blockIdx.z * heads + h] = 0u;
}

// ====================================================================== LM-head reductions
// The head GEMV leaves raw logits [vocab] in HBM (128 KB at vocab 32000); these
// kernels restate the reference's per-256-row block reductions on them.
__device__ inline bool better(float v, uint32_t i, float bv, uint32_t bi) {  // lib.rs:1553
    return v > bv || (v == bv && i < bi);
}

// block-wide (val, idx) arg-max under `better`; result valid in every thread.
__device__ inline void block_argmax(float& v, uint32_t& i, float* sv, uint32_t* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    v = sv[0]; i = si[0];
    for (int w = 1; w < nw; ++w)
        if (better(sv[w], si[w], v, i)) { v = sv[w]; i = si[w]; }
}

// logits_argmax_blocks + logits_argmax_finalize (lib.rs:1515-1565, :1725-1760).
// The last block to finish reduces the block winners; `advance` makes it also
// publish the token as the next input and append it to the output ring.
static __global__ void __launch_bounds__(256)
head_argmax_kernel(const float* __restrict__ logits, int V, float* block_vals, uint32_t* block_idxs,
                   unsigned int* counter, uint32_t* out_token, DevState* st, uint32_t* out_ring, int advance,
                   int idx_offset, TpLink tp, size_t logits_stride = 0, size_t block_stride = 0, size_t token_stride = 0,
                   size_t ring_stride = 0) {  // strides: blockIdx.y = sample of a multi-sample step
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    __shared__ int is_last;
    logits += blockIdx.y * logits_stride; block_vals += blockIdx.y * block_stride; block_idxs += blockIdx.y * block_stride;
    counter += blockIdx.y; out_token += blockIdx.y * token_stride; st += blockIdx.y; out_ring += blockIdx.y * ring_stride;
    const int row = blockIdx.x * HEAD_BLOCK + threadIdx.x;
    float v = -INFINITY;
    uint32_t i = 0xffffffffu;
    if (row < V) { v = logits[row]; i = (uint32_t)(row + idx_offset); }  // idx_offset: first row of this rank's vocabulary shard
    block_argmax(v, i, sv, si);
    if (threadIdx.x == 0) {
        block_vals[blockIdx.x] = v;
        block_idxs[blockIdx.x] = i;
        __threadfence();
        is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    v = -INFINITY; i = 0xffffffffu;
    for (int b = threadIdx.x; b < (int)gridDim.x; b += blockDim.x) {
        const float bv = __ldcg(block_vals + b);
        const uint32_t bi = __ldcg(block_idxs + b);
        if (better(bv, bi, v, i)) { v = bv; i = bi; }
    }
    block_argmax(v, i, sv, si);
    if (threadIdx.x == 0 && tp.world > 1) {
        // tensor parallel: hand this shard's winner to every rank; tp_pick_kernel chooses
        *counter = 0u;
        const unsigned int seq = tp.st->cand_seq + 1;
        const int slot = seq & 1;
        for (int p = 0; p < tp.world; ++p) {
            uint2* cand = reinterpret_cast<uint2*>(tp.peers[p] + TpRegion::cand_off(tp.world, tp.dim)) + slot * tp.world + tp.rank;
            *cand = make_uint2(__float_as_uint(v), i);
        }
        __threadfence_system();
        for (int p = 0; p < tp.world; ++p)
            st_release_sys(reinterpret_cast<unsigned int*>(tp.peers[p] + TpRegion::cflags_off(tp.world, tp.dim)) + slot * tp.world + tp.rank, seq);
        tp.st->cand_seq = seq;
        return;
    }
    if (threadIdx.x == 0) {
        *out_token = i;
        *counter = 0u;
        if (advance) {
            st->token = i;
            out_ring[st->nout] = i;
            st->nout += 1;
        }
        st->pos += 1;
    }
}

// Tensor parallel: pick the best of the ranks' shard winners (larger logit, ties to the lower
// token id — the same rule as inside a shard, so the result equals the single-GPU arg-max).
// Tensor-parallel top-k sampling: every rank hands its shard's per-block candidates (token ids made
// global) to every rank; with all candidates and the same LCG state each rank then draws the same
// token in sample_topk_kernel.  nb = blocks per rank in the exchange layout, nb_local = this rank's.
static __global__ void __launch_bounds__(256)
tp_push_topk_kernel(TpLink tp, const float* __restrict__ vals, const uint32_t* __restrict__ idxs, int nb_local, int nb, int k, int idx_offset) {
    const unsigned int seq = tp.st->cand_seq + 1;
    const int slot = seq & 1, per_rank = nb * 32;
    const size_t slot_off = TpRegion::topk_off(tp.world, tp.dim) + (size_t)slot * TpRegion::topk_slot_bytes(tp.world, nb);
    for (int j = threadIdx.x; j < per_rank; j += blockDim.x) {
        float v = -INFINITY;
        uint32_t i = 0xffffffffu;
        if (j < nb_local * k) {
            v = vals[j];
            i = idxs[j];
            if (i != 0xffffffffu) i += (uint32_t)idx_offset;
        }
        for (int p = 0; p < tp.world; ++p) {
            float* pv = reinterpret_cast<float*>(tp.peers[p] + slot_off) + (size_t)tp.rank * per_rank;
            uint32_t* pi = reinterpret_cast<uint32_t*>(tp.peers[p] + slot_off) + (size_t)tp.world * per_rank + (size_t)tp.rank * per_rank;
            pv[j] = v;
            pi[j] = i;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int p = 0; p < tp.world; ++p)
            st_release_sys(reinterpret_cast<unsigned int*>(tp.peers[p] + TpRegion::cflags_off(tp.world, tp.dim)) + slot * tp.world + tp.rank, seq);
        tp.st->cand_seq = seq;
    }
}
// wait (bounded) for every rank's candidates of this exchange, then copy them to fixed buffers
static __global__ void __launch_bounds__(256)
tp_wait_topk_kernel(TpLink tp, DevState* st, float* __restrict__ out_vals, uint32_t* __restrict__ out_idxs, int nb, int take) {
    const unsigned int seq = __ldcg(&st->cand_seq);
    const int slot = seq & 1, n = tp.world * nb * 32;  // `take` leading entries of every rank's row are kept, packed
    if ((int)threadIdx.x < tp.world) {
        const unsigned int* cf = reinterpret_cast<const unsigned int*>(tp.peers[tp.rank] + TpRegion::cflags_off(tp.world, tp.dim));
        if (!tp_wait_flag(cf + slot * tp.world + threadIdx.x, seq, st, tp.wait_ns)) atomicCAS(&st->error, 0, DEV_ERR_TP_WAIT);
    }
    __syncthreads();
    const char* base = tp.peers[tp.rank] + TpRegion::topk_off(tp.world, tp.dim) + (size_t)slot * TpRegion::topk_slot_bytes(tp.world, nb);
    const float* sv = reinterpret_cast<const float*>(base);
    const uint32_t* si = reinterpret_cast<const uint32_t*>(base) + n;
    for (int j = threadIdx.x; j < tp.world * take; j += blockDim.x) {
        const int r = j / take, e = j % take;
        out_vals[j] = __ldcg(sv + (size_t)r * nb * 32 + e);
        out_idxs[j] = __ldcg(si + (size_t)r * nb * 32 + e);
    }
}

static __global__ void tp_count_allreduces_kernel(DevState* st, unsigned int ars) { st->ar_base += ars; }

static __global__ void tp_pick_kernel(TpLink tp, uint32_t* out_token, DevState* st, uint32_t* out_ring, int advance, unsigned int ars) {
    const int lane = threadIdx.x;
    const unsigned int seq = __ldcg(&st->cand_seq);
    const int slot = seq & 1;
    float v = -INFINITY;
    uint32_t i = 0xffffffffu;
    if (lane < tp.world) {
        const unsigned int* cf = reinterpret_cast<const unsigned int*>(tp.peers[tp.rank] + TpRegion::cflags_off(tp.world, tp.dim));
        if (!tp_wait_flag(cf + slot * tp.world + lane, seq, st, tp.wait_ns)) atomicCAS(&st->error, 0, DEV_ERR_TP_WAIT);
        const uint2 c = __ldcg(reinterpret_cast<const uint2*>(tp.peers[tp.rank] + TpRegion::cand_off(tp.world, tp.dim)) + slot * tp.world + lane);
        v = __uint_as_float(c.x);
        i = c.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (lane == 0) {
        *out_token = i;
        if (advance) {
            st->token = i;
            out_ring[st->nout] = i;
            st->nout += 1;
        }
        st->pos += 1;
        st->ar_base += ars;
    }
}

// Tensor parallel: consume an all-reduce nobody else reads (the last one of a token that
// computes no logits): finish x = res + alpha * sum and re-arm the ring slot.
static __global__ void __launch_bounds__(256) tp_consume_kernel(TpLink tp, int* err) {
    const unsigned int seq = __ldcg(&tp.st->ar_base) + (unsigned int)tp.in_reduce;
    float* base = reinterpret_cast<float*>(tp.peers[tp.rank]);
    const float* inbox = base + (size_t)(seq % 3u) * tp.world * tp.dim;
    uint4* rearm = reinterpret_cast<uint4*>(base + (size_t)((seq + 2u) % 3u) * tp.world * tp.dim);
    const int n4 = tp.world * tp.dim / 4;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n4; j += gridDim.x * blockDim.x)
        rearm[j] = make_uint4(TP_SENTINEL, TP_SENTINEL, TP_SENTINEL, TP_SENTINEL);
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < tp.dim / 4; c += gridDim.x * blockDim.x) {
        float4 a;
        if (!tp_gather4(inbox, tp.world, tp.dim, (size_t)c * 4, a, tp.st, tp.wait_ns)) atomicCAS(err, 0, DEV_ERR_TP_WAIT);
        const float4 r4 = __ldcg(reinterpret_cast<const float4*>(tp.res + (size_t)c * 4));
        *reinterpret_cast<float4*>(tp.x_out + (size_t)c * 4) =
            make_float4(r4.x + tp.alpha * a.x, r4.y + tp.alpha * a.y, r4.z + tp.alpha * a.z, r4.w + tp.alpha * a.w);
    }
}

// logits_topk_blocks (lib.rs:1567-1635): k rounds of arg-max-and-remove per block.
static __global__ void __launch_bounds__(256)
head_topk_kernel(const float* __restrict__ logits, int V, int top_k, float* out_vals, uint32_t* out_idxs,
                 size_t logits_stride = 0, size_t cand_stride = 0) {  // strides: blockIdx.y = sample of a multi-sample step
    __shared__ float sv[8];
    __shared__ uint32_t si[8];
    logits += blockIdx.y * logits_stride; out_vals += blockIdx.y * cand_stride; out_idxs += blockIdx.y * cand_stride;
    const int row = blockIdx.x * HEAD_BLOCK + threadIdx.x;
    float cv = -INFINITY;
    uint32_t ci = 0xffffffffu;
    if (row < V) { cv = logits[row]; ci = (uint32_t)row; }
    for (int rank = 0; rank < top_k; ++rank) {
        float v = cv;
        uint32_t i = ci;
        block_argmax(v, i, sv, si);
        if (threadIdx.x == 0) {
            out_vals[blockIdx.x * top_k + rank] = v;
            out_idxs[blockIdx.x * top_k + rank] = i;
        }
        if (ci == i) { cv = -INFINITY; ci = 0xffffffffu; }
        __syncthreads();
    }
}

__device__ inline float softcap_apply(float z, float c) { return c > 0.0f ? c * tanhf(z / c) : z; }

// logits_block_stats (lib.rs:1637-1700): per block max of z = softcap(logit)*inv_T and sum exp(z - max).
static __global__ void __launch_bounds__(256)
head_stats_kernel(const float* __restrict__ logits, int V, float inv_t, float softcap, float* maxes, float* sums,
                  size_t logits_stride = 0, size_t stat_stride = 0) {  // strides: blockIdx.y = sample of a multi-sample step
    __shared__ float red[32];
    logits += blockIdx.y * logits_stride; maxes += blockIdx.y * stat_stride; sums += blockIdx.y * stat_stride;
    const int row = blockIdx.x * HEAD_BLOCK + threadIdx.x;
    float z = -INFINITY;
    if (row < V) z = softcap_apply(logits[row], softcap) * inv_t;
    const float mx = block_max(z, red);
    const float e = row < V ? expf(z - mx) : 0.0f;
    const float s = block_sum(e, red);
    if (threadIdx.x == 0) { maxes[blockIdx.x] = mx; sums[blockIdx.x] = s; }
}

// Advance the position after a step whose last kernel does not do it itself.
static __global__ void advance_kernel(DevState* st, unsigned int ars) {
    st->pos += 1;
    st->ar_base += ars;  // tensor parallel: all-reduces this token issued
}

static __global__ void set_state_kernel(DevState* st, int pos, uint32_t token) {
    st->pos = pos;
    st->token = token;
}
static __global__ void begin_loop_kernel(DevState* st, int pos, uint32_t token, uint64_t rng) {
    st->pos = pos;
    st->token = token;
    st->rng = rng;
    st->nout = 0;
    st->cursor = 0;
}
// Prefill feeds prompt tokens from a device array: take the next one.
static __global__ void next_prompt_kernel(DevState* st, const uint32_t* prompt) {
    st->token = prompt[st->cursor];
    st->cursor += 1;
}

// ====================================================================== on-device samplers
__device__ inline float lcg_next_f32(uint64_t& s) {  // inference.rs:759-768
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    return (float)(s >> 40) / 16777216.0f;
}

// decode.rs:218-253 (merge of nblocks*k candidates, ties to the lower index, non-finite
// dropped), decode.rs:155-159 (softcap), then sample_topk_candidates (inference.rs:823-849).
// One CTA; the k winners are extracted by k rounds of arg-max, the draw is sequential.
static __global__ void __launch_bounds__(1024)
sample_topk_kernel(const float* __restrict__ cand_vals, const uint32_t* __restrict__ cand_idxs, int ncand,
                   int top_k, float temperature, float softcap, DevState* st, uint32_t* out_ring,
                   size_t cand_stride = 0, size_t ring_stride = 0) {  // strides: blockIdx.x = sample of a multi-sample step
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    __shared__ float mv[32];
    __shared__ uint32_t mi[32];
    cand_vals += blockIdx.x * cand_stride; cand_idxs += blockIdx.x * cand_stride; st += blockIdx.x; out_ring += blockIdx.x * ring_stride;
    constexpr int PER = 8;  // 1024 threads * 8 >= 256 blocks * 32
    float cv[PER];
    uint32_t ci[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = threadIdx.x + j * 1024;
        cv[j] = -INFINITY; ci[j] = 0xffffffffu;
        if (c < ncand) {
            const float v = cand_vals[c];
            const uint32_t i = cand_idxs[c];
            if (i != 0xffffffffu && isfinite(v)) { cv[j] = v; ci[j] = i; }
        }
    }
    int merged = 0;
    for (int rank = 0; rank < top_k; ++rank) {
        float v = -INFINITY;
        uint32_t i = 0xffffffffu;
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (better(cv[j], ci[j], v, i)) { v = cv[j]; i = ci[j]; }
        block_argmax(v, i, sv, si);
        if (i == 0xffffffffu) break;
        if (threadIdx.x == 0) { mv[rank] = v; mi[rank] = i; }
#pragma unroll
        for (int j = 0; j < PER; ++j)
            if (ci[j] == i) { cv[j] = -INFINITY; ci[j] = 0xffffffffu; }
        merged = rank + 1;
        __syncthreads();
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    uint64_t rng = st->rng;
    uint32_t next = 0;
    if (merged > 0) {
        if (softcap > 0.0f)
            for (int j = 0; j < merged; ++j) mv[j] = softcap * tanhf(mv[j] / softcap);
        next = mi[0];
        if (!(temperature <= 0.0f || merged == 1)) {
            float mx = -INFINITY;
            for (int j = 0; j < merged; ++j) mx = fmaxf(mx, mv[j]);
            float sum = 0.0f;
            for (int j = 0; j < merged; ++j) sum += expf((mv[j] - mx) / temperature);
            if (isfinite(sum) && sum > 0.0f) {
                float draw = lcg_next_f32(rng) * sum;
                next = mi[merged - 1];
                for (int j = 0; j < merged; ++j) {
                    draw -= expf((mv[j] - mx) / temperature);
                    if (draw <= 0.0f) { next = mi[j]; break; }
                }
            }
        }
    }
    st->rng = rng;
    st->token = next;
    out_ring[st->nout] = next;
    st->nout += 1;
    st->pos += 1;
}

// sample_block_from_stats (inference.rs:851-891), then materialize (lib.rs:1702-1723:
// softcap, no temperature) and sample_softmax_index over that block (inference.rs:893-917).
// exp() of the 256 entries is evaluated in parallel; every accumulation and both
// inverse-CDF scans run on one thread in index order, as the reference does.
static __global__ void __launch_bounds__(256)
sample_fullvocab_kernel(const float* __restrict__ logits, int V, const float* __restrict__ maxes,
                        const float* __restrict__ sums, int nblocks, float temperature, float softcap,
                        DevState* st, uint32_t* out_ring, size_t logits_stride = 0, size_t stat_stride = 0,
                        size_t ring_stride = 0) {  // strides: blockIdx.x = sample of a multi-sample step
    __shared__ float w[256];
    __shared__ float red[32];
    __shared__ int sblock;
    const int tid = threadIdx.x;
    logits += blockIdx.x * logits_stride; maxes += blockIdx.x * stat_stride; sums += blockIdx.x * stat_stride;
    st += blockIdx.x; out_ring += blockIdx.x * ring_stride;
    // block weights exp(max_b - gmax) * sum_b
    float gm = -INFINITY;
    for (int b = tid; b < nblocks; b += 256)
        if (isfinite(maxes[b])) gm = fmaxf(gm, maxes[b]);
    gm = block_max(gm, red);
    uint64_t rng = st->rng;
    for (int base = 0; base < nblocks; base += 256) {  // nblocks <= 256 in every supported vocab
        const int b = base + tid;
        float wt = 0.0f;
        if (b < nblocks && isfinite(maxes[b]) && isfinite(sums[b]) && sums[b] > 0.0f) wt = expf(maxes[b] - gm) * sums[b];
        w[tid] = wt;
    }
    __syncthreads();
    if (tid == 0) {
        int chosen = 0;
        if (isfinite(gm)) {
            float total = 0.0f;
            for (int b = 0; b < nblocks; ++b) total += w[b];
            if (isfinite(total) && total > 0.0f) {
                float draw = lcg_next_f32(rng) * total;
                chosen = nblocks - 1;
                for (int b = 0; b < nblocks; ++b) {
                    draw -= w[b];
                    if (draw <= 0.0f) { chosen = b; break; }
                }
            }
        }
        sblock = chosen;
    }
    __syncthreads();
    const int blk = sblock;
    const int valid = min(256, V - blk * 256);
    float lg = -INFINITY;
    if (tid < valid) lg = softcap_apply(logits[blk * 256 + tid], softcap);
    const float mx = block_max(lg, red);
    __syncthreads();
    w[tid] = tid < valid ? expf((lg - mx) / temperature) : 0.0f;
    // ties for the non-finite fallback: last maximum, as Rust's max_by (inference.rs:901-906)
    __shared__ float lgs[256];
    lgs[tid] = lg;
    __syncthreads();
    if (tid != 0) return;
    float sum = 0.0f;
    for (int i = 0; i < valid; ++i) sum += w[i];
    int pick;
    if (!isfinite(sum) || sum <= 0.0f) {
        pick = 0;
        for (int i = 1; i < valid; ++i)
            if (!(lgs[i] < lgs[pick])) pick = i;
    } else {
        float draw = lcg_next_f32(rng) * sum;
        pick = valid - 1;
        for (int i = 0; i < valid; ++i) {
            draw -= w[i];
            if (draw <= 0.0f) { pick = i; break; }
        }
    }
    const uint32_t next = (uint32_t)(blk * 256 + pick);
    st->rng = rng;
    st->block_idx = blk;
    st->token = next;
    out_ring[st->nout] = next;
    st->nout += 1;
    st->pos += 1;
}

// Tensor-parallel full-vocabulary sampler (sample_fullvocab_kernel's arithmetic): every rank picks the
// same 256-row block from the gathered per-block (max, sum); the rank whose vocabulary shard holds that
// block draws the token from its logits and hands (token, whether it consumed a second draw) to all
// ranks, which advance their LCG state alike.  maxes / sums: [world * nb] in vocabulary order.
static __global__ void __launch_bounds__(256)
tp_sample_fullvocab_kernel(const float* __restrict__ local_logits, int v0, int V, const float* __restrict__ maxes,
                           const uint32_t* __restrict__ sum_bits, int nb, float temperature, float softcap, DevState* st,
                           uint32_t* out_ring, TpLink tp, unsigned int ars) {
    __shared__ float w[256];
    __shared__ float red[32];
    __shared__ float lgs[256];
    __shared__ int sblock;
    const int tid = threadIdx.x, nblocks = tp.world * nb;
    const float* sums = reinterpret_cast<const float*>(sum_bits);
    float gm = -INFINITY;
    for (int b = tid; b < nblocks; b += 256)
        if (isfinite(maxes[b])) gm = fmaxf(gm, maxes[b]);
    gm = block_max(gm, red);
    uint64_t rng = st->rng;
    {
        const int b = tid;
        float wt = 0.0f;
        if (b < nblocks && isfinite(maxes[b]) && isfinite(sums[b]) && sums[b] > 0.0f) wt = expf(maxes[b] - gm) * sums[b];
        w[tid] = wt;
    }
    __syncthreads();
    if (tid == 0) {
        int chosen = 0;
        if (isfinite(gm)) {
            float total = 0.0f;
            for (int b = 0; b < nblocks; ++b) total += w[b];
            if (isfinite(total) && total > 0.0f) {
                float draw = lcg_next_f32(rng) * total;
                chosen = nblocks - 1;
                for (int b = 0; b < nblocks; ++b) {
                    draw -= w[b];
                    if (draw <= 0.0f) { chosen = b; break; }
                }
            }
        }
        if (chosen * 256 >= V) chosen = (V - 1) / 256;  // rows past the vocabulary carry zero weight; keep the index valid
        sblock = chosen;
    }
    __syncthreads();
    const int blk = sblock, owner = blk / nb;
    const unsigned int seq = st->cand_seq + 1;
    const int slot = seq & 1;
    uint32_t next = 0, drew = 0;
    if (owner == tp.rank) {
        const int valid = min(256, V - blk * 256);
        float lg = -INFINITY;
        if (tid < valid) lg = softcap_apply(local_logits[blk * 256 - v0 + tid], softcap);
        const float mx = block_max(lg, red);
        __syncthreads();
        w[tid] = tid < valid ? expf((lg - mx) / temperature) : 0.0f;
        lgs[tid] = lg;
        __syncthreads();
        if (tid != 0) return;
        float sum = 0.0f;
        for (int i = 0; i < valid; ++i) sum += w[i];
        int pick;
        if (!isfinite(sum) || sum <= 0.0f) {
            pick = 0;
            for (int i = 1; i < valid; ++i)
                if (!(lgs[i] < lgs[pick])) pick = i;
        } else {
            float draw = lcg_next_f32(rng) * sum;
            drew = 1;
            pick = valid - 1;
            for (int i = 0; i < valid; ++i) {
                draw -= w[i];
                if (draw <= 0.0f) { pick = i; break; }
            }
        }
        next = (uint32_t)(blk * 256 + pick);
        for (int p = 0; p < tp.world; ++p) {
            uint2* cand = reinterpret_cast<uint2*>(tp.peers[p] + TpRegion::cand_off(tp.world, tp.dim)) + slot * tp.world + tp.rank;
            *cand = make_uint2(drew, next);
        }
        __threadfence_system();
        for (int p = 0; p < tp.world; ++p)
            st_release_sys(reinterpret_cast<unsigned int*>(tp.peers[p] + TpRegion::cflags_off(tp.world, tp.dim)) + slot * tp.world + tp.rank, seq);
    } else {
        if (tid != 0) return;
        const unsigned int* cf = reinterpret_cast<const unsigned int*>(tp.peers[tp.rank] + TpRegion::cflags_off(tp.world, tp.dim));
        if (!tp_wait_flag(cf + slot * tp.world + owner, seq, st, tp.wait_ns)) atomicCAS(&st->error, 0, DEV_ERR_TP_WAIT);
        const uint2 c = __ldcg(reinterpret_cast<const uint2*>(tp.peers[tp.rank] + TpRegion::cand_off(tp.world, tp.dim)) + slot * tp.world + owner);
        drew = c.x;
        next = c.y;
        if (drew) lcg_next_f32(rng);
    }
    st->cand_seq = seq;
    st->rng = rng;
    st->block_idx = blk;
    st->token = next;
    out_ring[st->nout] = next;
    st->nout += 1;
    st->pos += 1;
    st->ar_base += ars;
}

// ====================================================================== weight preparation
// dst[(o*row_mul + row_off) * in + i] = convert(src[transposed ? i*out + o : o*in + i]).
// The reference keeps wq/wk/wv/wo/w1/w3 as [in, out]; every GEMV here wants [out, in].
template <typename WT>
__global__ void relayout_kernel(const float* __restrict__ src, WT* __restrict__ dst, int in, int out, int transposed,
                                int row_mul, int row_off, int full_in, int full_out, int in0, int out0) {
    __shared__ float tile[32][33];
    const int bi = blockIdx.x * 32, bo = blockIdx.y * 32;
    if (transposed) {
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int i = bi + j, o = bo + threadIdx.x;
            if (i < in && o < out) tile[j][threadIdx.x] = src[(size_t)(i + in0) * full_out + (o + out0)];
        }
        __syncthreads();
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int o = bo + j, i = bi + threadIdx.x;
            if (i < in && o < out) dst[((size_t)o * row_mul + row_off) * in + i] = Elem<WT>::from_f32(tile[threadIdx.x][j]);
        }
    } else {
        for (int j = threadIdx.y; j < 32; j += blockDim.y) {
            const int o = bo + j, i = bi + threadIdx.x;
            if (i < in && o < out) dst[((size_t)o * row_mul + row_off) * in + i] = Elem<WT>::from_f32(src[(size_t)(o + out0) * full_in + (i + in0)]);
        }
    }
}

// The same mapping with values drawn from the counter-based generator.
template <typename WT>
__global__ void synth_kernel(WT* __restrict__ dst, int in, int out, int transposed, int row_mul, int row_off,
                             uint64_t key, float scale, int full_in, int full_out, int in0, int out0) {
    const size_t total = (size_t)in * out;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (size_t)gridDim.x * blockDim.x) {
        const size_t o = j / in, i = j % in;
        const size_t logical = transposed ? (i + in0) * (size_t)full_out + (o + out0) : (o + out0) * (size_t)full_in + (i + in0);
        dst[(o * row_mul + row_off) * in + i] = Elem<WT>::from_f32(synth_value(key, logical, scale));
    }
}

// ---------------------------------------------------------------------- weight quantisation
// src is a [out, ld] fp32 matrix already in GEMV orientation, of which columns col0 .. col0 + in - 1
// are kept (a tensor-parallel rank that holds a slice of the inputs sees the whole rows, so that its
// scales are those of the unsharded matrix); row o lands in destination row o * row_mul + row_off in
// the Wfmt row format.  One CTA per row (grid-stride).  No reference counterpart (the reference
// stores fp32 only).
static __global__ void __launch_bounds__(256)
quantize_fp8_rows_kernel(const float* __restrict__ src, unsigned char* __restrict__ dst, int in, int out, int row_mul, int row_off, int ld, int col0) {
    __shared__ float red[32];
    const uint32_t stride = Wfmt<Fp8Row>::row_stride(in);
    for (int o = blockIdx.x; o < out; o += gridDim.x) {
        const float* full = src + (size_t)o * ld;
        float amax = 0.0f;
        for (int i = threadIdx.x; i < ld; i += blockDim.x) amax = fmaxf(amax, fabsf(full[i]));  // the scale of the whole row
        amax = block_max(amax, red);
        const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
        const float* row = full + col0;
        unsigned char* drow = dst + ((size_t)o * row_mul + row_off) * stride;
        for (int i = threadIdx.x; i < in; i += blockDim.x)
            drow[i] = (unsigned char)__nv_cvt_float_to_fp8(row[i] / scale, __NV_SATFINITE, __NV_E4M3);
        if (threadIdx.x < 4) reinterpret_cast<float*>(drow + in)[threadIdx.x] = threadIdx.x == 0 ? scale : 0.0f;
        __syncthreads();
    }
}

static __global__ void __launch_bounds__(256)
quantize_int4_rows_kernel(const float* __restrict__ src, unsigned char* __restrict__ dst, int in, int out, int row_mul, int row_off, int ld, int col0) {
    const uint32_t stride = Wfmt<Int4G32>::row_stride(in), soff = Wfmt<Int4G32>::scale_off(in);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5, ngroups = in / 32;
    for (int o = blockIdx.x; o < out; o += gridDim.x) {
        const float* row = src + (size_t)o * ld + col0;  // col0 is a multiple of 32: the groups are those of the whole row
        unsigned char* drow = dst + ((size_t)o * row_mul + row_off) * stride;
        for (int g = warp; g < ngroups; g += nwarps) {
            const float v = row[g * 32 + lane];
            const float amax = warp_max(fabsf(v));
            const __half sh = __float2half_rn(amax / 7.0f);
            const float s = __half2float(sh);
            const float q = s > 0.0f ? fminf(fmaxf(rintf(v / s), -8.0f), 7.0f) : 0.0f;
            const uint32_t n = (uint32_t)((int)q + 8);
            const int e = lane & 7, nib = (e >> 1) + 4 * (e & 1);  // position inside the 32-bit word (see Wfmt<Int4G32>)
            const uint32_t word = __reduce_or_sync(0xffu << (lane & 24), n << (4 * nib));
            if (e == 0) reinterpret_cast<uint32_t*>(drow + g * 16)[lane >> 3] = word;
            if (lane == 0) reinterpret_cast<__half*>(drow + soff)[g] = sh;
        }
        for (uint32_t b = soff + (uint32_t)ngroups * 2u + threadIdx.x; b < stride; b += blockDim.x) drow[b] = 0;  // padding
    }
}

// Model::seed_layer_cache_from_channel_first (lib.rs:217-237): [kv_dim, seq] fp32 -> pages.
template <typename KT>
__global__ void seed_kv_kernel(const float* __restrict__ k_cf, const float* __restrict__ v_cf, KT* __restrict__ kv_pool,
                               const int* __restrict__ page_table, int seq, int live_len, int kv_heads, int hd,
                               int page_tokens) {
    const int KV = kv_heads * hd;
    const size_t total = (size_t)seq * KV;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (size_t)gridDim.x * blockDim.x) {
        const int pos = (int)(j % seq), d = (int)(j / seq);  // coalesced reads of the channel-first source
        const int head = d / hd, dd = d % hd;
        const int page = page_table[pos / page_tokens], off = pos % page_tokens;
        const float kk = pos < live_len ? k_cf[(size_t)d * seq + pos] : 0.0f;
        const float vv = pos < live_len ? v_cf[(size_t)d * seq + pos] : 0.0f;
        kv_pool[((((size_t)page * 2 + 0) * kv_heads + head) * page_tokens + off) * hd + dd] = Elem<KT>::from_f32(kk);
        kv_pool[((((size_t)page * 2 + 1) * kv_heads + head) * page_tokens + off) * hd + dd] = Elem<KT>::from_f32(vv);
    }
}

}  // namespace cd
