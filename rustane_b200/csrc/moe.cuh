// Kernels of the MoE + MLA decoder (a mixture-of-experts FFN behind multi-head latent attention),
// one token per step.  The reference has neither (no router, expert or latent-cache code anywhere
// in it): the model is defined by this repository (include/cuda_decode.h, cd_moe_config) and what
// it shares with the dense model - RMSNorm (lib.rs:1354-1378), interleaved-pair RoPE
// (lib.rs:1392-1408), SwiGLU (lib.rs:1504-1513), the scaled residuals (lib.rs:1491-1502) - is
// computed exactly as there.
//
// Per layer (H heads, C latent width, R RoPE width, N / V per-head no-position / value widths):
//   gemv_tma_kernel      RMSNorm + [q | latent | rope key] = W_qa xn            (the dense GEMV, plain store)
//   mla_post_kernel      RoPE on the q heads' RoPE parts and on the key; RMSNorm of the latent; the
//                        cache row [latent | rope key] into its page; per head the absorbed query
//                        q'_h = W_uk_h^T q_nope_h, so that a score is one 576-wide dot with a cache row
//   mla_attn_kernel      split over cached positions: every CTA reads its positions once for all heads
//                        (the cache is shared by the heads), running softmax, partial latent sums
//   mla_out_kernel       merges the slices (fixed order) and applies W_uv_h: the head's output
//   gemv_tma_kernel      Wo + scaled residual
//   moe_router_kernel    RMSNorm, router logits, softmax over all experts, top-k (ties: lower index)
//   moe_w13_kernel       gate = silu(xn W1) * (xn W3) * p for the chosen experts and the shared ones
//   moe_w2_kernel        x = x2 + alpha * sum over experts of W2 gate; expert parallel: the rank's partial
//                        sum is pushed to every rank's inbox instead (the dense model's all-reduce)
// All of them are HBM-bound streams of weight rows (or cache rows) with fp32 accumulation.
#pragma once
#include "common.cuh"

namespace cd {

constexpr int MLA_MAX_HEADS = 16;   // heads whose state one attention thread keeps
constexpr int MLA_TILE = 16;        // cached positions per attention tile

// dot of one weight row (K elements, storage WT) with x (fp32, shared memory): the lanes of a warp take
// 16-byte chunks round robin; result valid in every lane
template <typename WT> __device__ inline float warp_row_dot(const WT* __restrict__ row, const float* xs, int K, int lane) {
    constexpr int EPC = Elem<WT>::EPC;
    float a = 0.0f;
#pragma unroll 4
    for (int c = lane; c < K / EPC; c += 32) {
        const uint4 w = ldg_stream(reinterpret_cast<const char*>(row) + (size_t)c * 16);
        float f[EPC];
        Elem<WT>::unpack(w, f);
#pragma unroll
        for (int e = 0; e < EPC; e += 4) {  // x in 16-byte pieces: one shared-memory transaction per four elements
            const float4 x4 = *reinterpret_cast<const float4*>(xs + c * EPC + e);
            a = fmaf(f[e], x4.x, a); a = fmaf(f[e + 1], x4.y, a); a = fmaf(f[e + 2], x4.z, a); a = fmaf(f[e + 3], x4.w, a);
        }
    }
    return warp_sum(a);
}

struct MlaDims {
    int heads, latent, rope, nope, vdim, page_tokens;
};

// ---------------------------------------------------------------------- after the q | latent | key GEMV
// grid = heads + 1.  CTA h: RoPE on q_h's RoPE part, absorbed query q'_h[c] = sum_d W_uk[c, h N + d] q_nope_h[d];
// both into qabs[h] = [q' (C) | rope(q_rope) (R)].  CTA `heads`: the cache row of this position.
template <typename WT, typename KT>
__global__ void __launch_bounds__(256)
mla_post_kernel(const float* __restrict__ qa, const WT* __restrict__ wuk_t, const float* __restrict__ gamma_kv, const float2* __restrict__ rope,
                const int* __restrict__ page_table, const DevState* st, KT* __restrict__ lat_pool, float* __restrict__ qabs, MlaDims d) {
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int C = d.latent, R = d.rope, N = d.nope, QH = N + R, h = blockIdx.x;
    const int pos = __ldcg(&st->pos);
    if (h < d.heads) {
        float* qn = sm;  // [N]
        for (int i = tid; i < N; i += blockDim.x) qn[i] = __ldcg(qa + (size_t)h * QH + i);
        for (int i = tid; i < R / 2; i += blockDim.x) {
            const float e = __ldcg(qa + (size_t)h * QH + N + 2 * i), o = __ldcg(qa + (size_t)h * QH + N + 2 * i + 1);
            const float2 cs = rope[(size_t)pos * (R / 2) + i];
            qabs[(size_t)h * (C + R) + C + 2 * i] = e * cs.x - o * cs.y;
            qabs[(size_t)h * (C + R) + C + 2 * i + 1] = o * cs.x + e * cs.y;
        }
        __syncthreads();
        const WT* base = wuk_t + (size_t)h * C * N;
        for (int c = warp; c < C; c += nw) {
            const float v = warp_row_dot<WT>(base + (size_t)c * N, qn, N, lane);
            if (lane == 0) qabs[(size_t)h * (C + R) + c] = v;
        }
        return;
    }
    // the cache row: rmsnorm(latent) | rope(key)
    const float* craw = qa + (size_t)d.heads * QH;
    float ss = 0.0f;
    for (int i = tid; i < C; i += blockDim.x) {
        const float v = __ldcg(craw + i);
        sm[i] = v;
        ss += v * v;
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot * (1.0f / (float)C) + RMS_EPS);
    const int page = page_table[pos / d.page_tokens], off = pos % d.page_tokens;
    KT* row = lat_pool + ((size_t)page * d.page_tokens + off) * (C + R);
    for (int i = tid; i < C; i += blockDim.x) row[i] = Elem<KT>::from_f32(sm[i] * inv * gamma_kv[i]);
    for (int i = tid; i < R / 2; i += blockDim.x) {
        const float e = __ldcg(craw + C + 2 * i), o = __ldcg(craw + C + 2 * i + 1);
        const float2 cs = rope[(size_t)pos * (R / 2) + i];
        row[C + 2 * i] = Elem<KT>::from_f32(e * cs.x - o * cs.y);
        row[C + 2 * i + 1] = Elem<KT>::from_f32(o * cs.x + e * cs.y);
    }
}

// ---------------------------------------------------------------------- latent attention, one slice of cached positions per CTA
// score_h(t) = qabs_h . row(t) * scale over the C + R wide cache row; out_h = sum_t p_h(t) row(t)[0 .. C).
// Shared memory: qs [H][W + 1], rows [MLA_TILE][W + 1] (W = C + R; the pad keeps the columns on
// different banks), sc [H][MLA_TILE], state [3][H].  256 threads; thread t owns latent dimensions
// t and t + 256 of every head.
template <typename KT>
__global__ void __launch_bounds__(256)
mla_attn_kernel(const float* __restrict__ qabs, const KT* __restrict__ lat_pool, const int* __restrict__ page_table, const DevState* st,
                float* __restrict__ part_acc, float* __restrict__ part_ml, MlaDims d, int nsplit, float scale) {
    extern __shared__ float sm[];
    constexpr float NEG = -3.402823466e+38f;
    const int tid = threadIdx.x, H = d.heads, C = d.latent, W = d.latent + d.rope, LD = W + 1, s = blockIdx.x;
    float* qs = sm;                          // [H][LD]
    float* rows = qs + (size_t)H * LD;       // [MLA_TILE][LD]
    float* sc = rows + (size_t)MLA_TILE * LD;  // [H][MLA_TILE] probabilities of the tile
    float* mrun = sc + H * MLA_TILE;         // [H] running maximum
    float* lrun = mrun + H;                  // [H] running sum
    float* corr = lrun + H;                  // [H] rescale factor of the tile
    const int attn_len = __ldcg(&st->pos) + 1;
    int per = (attn_len + nsplit - 1) / nsplit;
    per = (per + MLA_TILE - 1) / MLA_TILE * MLA_TILE;
    const int t0 = s * per, t1 = min(attn_len, t0 + per);
    for (int i = tid; i < H * W; i += 256) qs[(i / W) * LD + (i % W)] = __ldcg(qabs + i);
    if (tid < H) { mrun[tid] = NEG; lrun[tid] = 0.0f; }
    float acc[MLA_MAX_HEADS][2];
#pragma unroll
    for (int h = 0; h < MLA_MAX_HEADS; ++h) acc[h][0] = acc[h][1] = 0.0f;
    __syncthreads();
    for (int tb = t0; tb < t1; tb += MLA_TILE) {
        const int nt = min(MLA_TILE, t1 - tb);
        for (int i = tid; i < nt * W; i += 256) {  // the tile's cache rows, widened to fp32
            const int j = i / W, k = i % W, t = tb + j;
            const int page = page_table[t / d.page_tokens], off = t % d.page_tokens;
            rows[j * LD + k] = Elem<KT>::to_f32(lat_pool[((size_t)page * d.page_tokens + off) * W + k]);
        }
        __syncthreads();
        for (int base = 0; base < H * MLA_TILE; base += 256) {  // one (head, position) score per thread; whole warps take part in the shuffles
            const int item = base + tid;
            const bool live = item < H * MLA_TILE;
            const int h = live ? item / MLA_TILE : 0, j = item % MLA_TILE;
            float v = NEG;
            if (live && j < nt) {
                const float* q = qs + h * LD;
                const float* r = rows + j * LD;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                int k = 0;
                for (; k + 4 <= W; k += 4) {
                    a0 = fmaf(q[k], r[k], a0); a1 = fmaf(q[k + 1], r[k + 1], a1);
                    a2 = fmaf(q[k + 2], r[k + 2], a2); a3 = fmaf(q[k + 3], r[k + 3], a3);
                }
                for (; k < W; ++k) a0 = fmaf(q[k], r[k], a0);
                v = ((a0 + a1) + (a2 + a3)) * scale;
            }
            // the MLA_TILE lanes of a head sit side by side in one warp: maximum and sum by shuffles
            float mx = v;
#pragma unroll
            for (int o = MLA_TILE / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mold = mrun[h], mnew = fmaxf(mold, mx);
            const float p = (live && j < nt) ? expf(v - mnew) : 0.0f;
            float ps = p;
#pragma unroll
            for (int o = MLA_TILE / 2; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            if (live) sc[item] = p;
            __syncwarp();
            if (live && j == 0) {
                const float c = expf(mold - mnew);
                corr[h] = c;
                lrun[h] = lrun[h] * c + ps;
                mrun[h] = mnew;
            }
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < MLA_MAX_HEADS; ++h) {
            if (h < H) {
                const float c = corr[h];
                float a0 = acc[h][0] * c, a1 = acc[h][1] * c;
                for (int j = 0; j < nt; ++j) {
                    const float p = sc[h * MLA_TILE + j];
                    if (tid < C) a0 = fmaf(p, rows[j * LD + tid], a0);
                    if (tid + 256 < C) a1 = fmaf(p, rows[j * LD + tid + 256], a1);
                }
                acc[h][0] = a0; acc[h][1] = a1;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < MLA_MAX_HEADS; ++h) {
        if (h < H) {
            float* pa = part_acc + ((size_t)s * H + h) * C;
            if (tid < C) pa[tid] = acc[h][0];
            if (tid + 256 < C) pa[tid + 256] = acc[h][1];
        }
    }
    if (tid < H) {
        part_ml[((size_t)s * H + tid) * 2 + 0] = mrun[tid];
        part_ml[((size_t)s * H + tid) * 2 + 1] = lrun[tid];
    }
}

// ---------------------------------------------------------------------- merge the slices, apply W_uv: grid = heads
template <typename WT>
__global__ void __launch_bounds__(256)
mla_out_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, const WT* __restrict__ wuv_t, float* __restrict__ attn_out,
               MlaDims d, int nsplit) {
    extern __shared__ float sm[];  // [C] the head's latent-space output, then [nsplit] slice weights
    constexpr float NEG = -3.402823466e+38f;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int H = d.heads, C = d.latent, V = d.vdim, h = blockIdx.x;
    float* lat = sm;
    float* wsl = sm + C;
    __shared__ float s_inv;
    if (warp == 0) {
        float M = NEG;
        for (int s = lane; s < nsplit; s += 32) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + (size_t)s * H + h);
            if (ml.y > 0.0f) M = fmaxf(M, ml.x);
        }
        M = warp_max(M);
        for (int s = lane; s < nsplit; s += 32) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + (size_t)s * H + h);
            wsl[s] = ml.y > 0.0f ? expf(ml.x - M) : 0.0f;
        }
        // the slices' sums are added in slice order by one lane, so the result does not depend on the lane count
        __syncwarp();
        if (lane == 0) {
            float tot = 0.0f;
            for (int s = 0; s < nsplit; ++s) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + (size_t)s * H + h);
                tot += ml.y * wsl[s];
            }
            s_inv = tot > 0.0f ? 1.0f / tot : 0.0f;
        }
    }
    __syncthreads();
    for (int c = tid; c < C; c += blockDim.x) {
        float a = 0.0f;
        for (int s = 0; s < nsplit; ++s) a += __ldcg(part_acc + ((size_t)s * H + h) * C + c) * wsl[s];
        lat[c] = a * s_inv;
    }
    __syncthreads();
    for (int dv = warp; dv < V; dv += nw) {
        const float v = warp_row_dot<WT>(wuv_t + ((size_t)h * V + dv) * C, lat, C, lane);
        if (lane == 0) attn_out[(size_t)h * V + dv] = v;
    }
}

// ---------------------------------------------------------------------- router: one CTA
// xn = rmsnorm(x, gamma) (kept for the expert kernels), p = softmax(W_r xn), the top_k largest p
// (k rounds of arg-max, ties to the lower expert index) with their weights, not renormalised.
template <typename WT>
__global__ void __launch_bounds__(1024)
moe_router_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const WT* __restrict__ wr, float* __restrict__ xn_out,
                  int* __restrict__ sel_ids, float* __restrict__ sel_w, int dim, int n_experts, int top_k) {
    extern __shared__ float sm[];  // [dim] xn, then [n_experts] logits / probabilities
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    float* xn = sm;
    float* pr = sm + dim;
    float ss = 0.0f;
    for (int i = tid; i < dim; i += blockDim.x) {
        const float v = __ldcg(x + i);
        xn[i] = v;
        ss += v * v;
    }
    const float tot = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(tot * (1.0f / (float)dim) + RMS_EPS);
    for (int i = tid; i < dim; i += blockDim.x) {
        const float v = xn[i] * inv * gamma[i];
        xn[i] = v;
        xn_out[i] = v;
    }
    __syncthreads();
    for (int e = warp; e < n_experts; e += nw) {
        const float v = warp_row_dot<WT>(wr + (size_t)e * dim, xn, dim, lane);
        if (lane == 0) pr[e] = v;
    }
    __syncthreads();
    if (warp != 0) return;
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, pr[e]);
    mx = warp_max(mx);
    __syncwarp();
    if (lane == 0) {  // exponentials and their sum in expert order by one lane: the oracle's order
        float sum = 0.0f;
        for (int e = 0; e < n_experts; ++e) {
            const float p = expf(pr[e] - mx);
            pr[e] = p;
            sum += p;
        }
        for (int e = 0; e < n_experts; ++e) pr[e] = pr[e] / sum;
    }
    __syncwarp();
    for (int k = 0; k < top_k; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = pr[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            sel_ids[k] = bi;
            sel_w[k] = bv;
            pr[bi] = -INFINITY;  // removed from the later rounds
        }
        __syncwarp();
    }
}

struct MoeDims {
    int dim, hidden, top_k;
    int e0, n_local;      // routed experts this rank holds: e0 .. e0 + n_local - 1
    int shared_cols;      // columns of the shared FFN this rank holds
};

// ---------------------------------------------------------------------- gate = silu(xn W1) * (xn W3) * weight
// Units: for each of the top_k chosen experts `hidden` column pairs, then `shared_cols` pairs of the shared
// FFN; one warp per unit (rows 2j and 2j + 1 of an interleaved [2 hidden, dim] matrix are adjacent in memory).
// A chosen expert another rank holds is skipped here and in moe_w2_kernel.
template <typename WT>
__global__ void __launch_bounds__(256)
moe_w13_kernel(const float* __restrict__ xn, const WT* __restrict__ w13, const WT* __restrict__ ws13, const int* __restrict__ sel_ids,
               const float* __restrict__ sel_w, float* __restrict__ gate, MoeDims d) {
    extern __shared__ float xs[];  // [dim]
    const int tid = threadIdx.x, lane = tid & 31;
    for (int i = tid; i < d.dim; i += blockDim.x) xs[i] = __ldcg(xn + i);
    __syncthreads();
    const int units = d.top_k * d.hidden + d.shared_cols;
    const int gw = (blockIdx.x * blockDim.x + tid) >> 5, total = (gridDim.x * blockDim.x) >> 5;
    for (int u = gw; u < units; u += total) {
        const WT* rows;
        float weight = 1.0f;
        if (u < d.top_k * d.hidden) {
            const int s = u / d.hidden, j = u % d.hidden, le = __ldcg(sel_ids + s) - d.e0;
            if (le < 0 || le >= d.n_local) continue;  // uniform across the warp
            rows = w13 + ((size_t)le * d.hidden + j) * 2 * d.dim;
            weight = __ldcg(sel_w + s);
        } else {
            rows = ws13 + (size_t)(u - d.top_k * d.hidden) * 2 * d.dim;
        }
        const float y1 = warp_row_dot<WT>(rows, xs, d.dim, lane);
        const float y3 = warp_row_dot<WT>(rows + d.dim, xs, d.dim, lane);
        if (lane == 0) gate[u] = (y1 / (1.0f + expf(-y1))) * y3 * weight;
    }
}

// ---------------------------------------------------------------------- y = sum of W2 gate over the local experts and the shared FFN
// One warp per output row.  Single GPU: out = res + alpha y.  Expert parallel: y goes to every rank's inbox
// (the dense model's push all-reduce, TpRegion); the next GEMV's prologue adds the ranks' rows in rank order.
template <typename WT>
__global__ void __launch_bounds__(256)
moe_w2_kernel(const float* __restrict__ gate, const WT* __restrict__ w2, const WT* __restrict__ ws2, const int* __restrict__ sel_ids,
              const float* __restrict__ res, float* __restrict__ out, float alpha, MoeDims d, TpLink tp) {
    extern __shared__ float gs[];  // [top_k * hidden + shared_cols]
    const int tid = threadIdx.x, lane = tid & 31;
    const int units = d.top_k * d.hidden + d.shared_cols;
    for (int i = tid; i < units; i += blockDim.x) gs[i] = __ldcg(gate + i);
    __syncthreads();
    const int gw = (blockIdx.x * blockDim.x + tid) >> 5, total = (gridDim.x * blockDim.x) >> 5;
    for (int r = gw; r < d.dim; r += total) {
        float y = 0.0f;
        for (int s = 0; s < d.top_k; ++s) {
            const int le = __ldcg(sel_ids + s) - d.e0;
            if (le < 0 || le >= d.n_local) continue;
            y += warp_row_dot<WT>(w2 + ((size_t)le * d.dim + r) * d.hidden, gs + s * d.hidden, d.hidden, lane);
        }
        if (d.shared_cols > 0) y += warp_row_dot<WT>(ws2 + (size_t)r * d.shared_cols, gs + d.top_k * d.hidden, d.shared_cols, lane);
        if (lane == 0) {
            if (tp.world > 1) {
                const unsigned int seq = __ldcg(&tp.st->ar_base) + (unsigned int)tp.ar_out;
                const size_t at = ((size_t)(seq % 3u) * tp.world + tp.rank) * tp.dim + r;
                const float v = tp_sanitize(y);
                for (int p = 0; p < tp.world; ++p) reinterpret_cast<float*>(tp.peers[p])[at] = v;
            } else {
                out[r] = __ldcg(res + r) + alpha * y;
            }
        }
    }
}

}  // namespace cd
