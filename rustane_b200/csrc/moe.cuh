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

// The same for NR rows `stride` elements apart: the loads of all rows are in flight together (a single row per
// warp is bound by one memory latency per row)
template <typename WT, int NR>
__device__ inline void warp_rows_dot(const WT* __restrict__ rows, size_t stride, const float* xs, int K, int lane, float (&out)[NR]) {
    constexpr int EPC = Elem<WT>::EPC;
    float a[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) a[r] = 0.0f;
#pragma unroll 2
    for (int c = lane; c < K / EPC; c += 32) {
        uint4 w[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) w[r] = ldg_stream(reinterpret_cast<const char*>(rows + (size_t)r * stride) + (size_t)c * 16);
        float x[EPC];
#pragma unroll
        for (int e = 0; e < EPC; e += 4) {
            const float4 x4 = *reinterpret_cast<const float4*>(xs + c * EPC + e);
            x[e] = x4.x; x[e + 1] = x4.y; x[e + 2] = x4.z; x[e + 3] = x4.w;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            float f[EPC];
            Elem<WT>::unpack(w[r], f);
#pragma unroll
            for (int e = 0; e < EPC; ++e) a[r] = fmaf(f[e], x[e], a[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(a[r]);
}

struct MlaDims {
    int heads, latent, rope, nope, vdim, page_tokens;
};

// ---------------------------------------------------------------------- after the q | latent | key GEMV
// grid = ceil(heads * C / 128) + 1 CTAs of 128 threads.  The first CTAs: one thread per row (h, c) of the absorbed-key matrix,
// q'_h[c] = sum_d W_uk[c, h N + d] q_nope_h[d] (a row is N elements: every thread has its whole row in flight);
// the last CTA: RoPE on the heads' RoPE parts of q, and the cache row of this position
// [rmsnorm(latent) | rope(key)].  qabs[h] = [q'_h (C) | rope(q_rope_h) (R)].
template <typename WT, typename KT>
__global__ void __launch_bounds__(128)
mla_post_kernel(const float* __restrict__ qa, const WT* __restrict__ wuk_t, const float* __restrict__ gamma_kv, const float2* __restrict__ rope,
                const int* __restrict__ page_table, const DevState* st, KT* __restrict__ lat_pool, float* __restrict__ qabs, KT* __restrict__ qsplit,
                MlaDims d) {
    extern __shared__ float sm[];  // [heads * N] the no-position parts of q (absorb CTAs) or [C] the raw latent (last CTA)
    __shared__ float red[32];
    constexpr int EPC = Elem<WT>::EPC;
    const int tid = threadIdx.x;
    const int H = d.heads, C = d.latent, R = d.rope, N = d.nope, QH = N + R;
    // qsplit (16-bit cache only): [2][16][C + R], the 16-bit head of qabs and the 16-bit remainder, the tensor-core
    // attention's A operand
    auto put = [&](int h, int k, float v) {
        qabs[(size_t)h * (C + R) + k] = v;
        if (qsplit != nullptr) {
            const KT hi = Elem<KT>::from_f32(v);
            qsplit[(size_t)h * (C + R) + k] = hi;
            qsplit[(size_t)(16 + h) * (C + R) + k] = Elem<KT>::from_f32(v - Elem<KT>::to_f32(hi));
        }
    };
    if (blockIdx.x + 1 < gridDim.x) {
        const int r = min((int)(blockIdx.x * blockDim.x) + tid, H * C - 1);  // row (h, c)
        const char* row = reinterpret_cast<const char*>(wuk_t + (size_t)r * N);
        constexpr int PRE = 16;  // chunks of the row requested before anything else (a whole 128-wide 16-bit row)
        uint4 w[PRE];
#pragma unroll
        for (int j = 0; j < PRE; ++j) w[j] = j < N / EPC ? ldg_stream(row + (size_t)j * 16) : make_uint4(0, 0, 0, 0);
        pdl_wait();  // the weights above do not depend on the previous kernel, q does
        pdl_launch_dependents();
        for (int i = tid; i < H * N; i += blockDim.x) sm[i] = __ldcg(qa + (size_t)(i / N) * QH + (i % N));
        __syncthreads();
        if ((int)(blockIdx.x * blockDim.x) + tid >= H * C) return;
        const int h = r / C;
        const float* qn = sm + h * N;
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            if (j < N / EPC) {
                float f[EPC];
                Elem<WT>::unpack(w[j], f);
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc = fmaf(f[e], qn[j * EPC + e], acc);
            }
        }
        for (int c0 = PRE; c0 < N / EPC; c0 += 8) {  // wider rows: eight more chunks in flight at a time
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = c0 + j < N / EPC ? ldg_stream(row + (size_t)(c0 + j) * 16) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (c0 + j < N / EPC) {
                    float f[EPC];
                    Elem<WT>::unpack(v[j], f);
#pragma unroll
                    for (int e = 0; e < EPC; ++e) acc = fmaf(f[e], qn[(c0 + j) * EPC + e], acc);
                }
            }
        }
        put(h, r % C, acc);
        return;
    }
    pdl_wait();
    pdl_launch_dependents();
    const int pos = __ldcg(&st->pos);
    for (int i = tid; i < H * (R / 2); i += blockDim.x) {  // RoPE on q's RoPE parts
        const int h = i / (R / 2), k = i % (R / 2);
        const float e = __ldcg(qa + (size_t)h * QH + N + 2 * k), o = __ldcg(qa + (size_t)h * QH + N + 2 * k + 1);
        const float2 cs = rope[(size_t)pos * (R / 2) + k];
        put(h, C + 2 * k, e * cs.x - o * cs.y);
        put(h, C + 2 * k + 1, o * cs.x + e * cs.y);
    }
    // the cache row: rmsnorm(latent) | rope(key)
    const float* craw = qa + (size_t)H * QH;
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
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
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
            rows[j * LD + k] = Elem<KT>::to_f32(__ldcg(lat_pool + ((size_t)page * d.page_tokens + off) * W + k));  // the newest row was written this token
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

// ---------------------------------------------------------------------- merge the slices, apply W_uv: grid = (heads, ceil(V / 32))
template <typename WT>
__global__ void __launch_bounds__(256)
mla_out_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, const WT* __restrict__ wuv_t, float* __restrict__ attn_out,
               const DevState* st, MlaDims d, int nsplit_max, int tile) {
    extern __shared__ float sm[];  // [C] the head's latent-space output, then [nsplit] slice weights
    constexpr float NEG = -3.402823466e+38f;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    const int H = d.heads, C = d.latent, V = d.vdim, h = blockIdx.x;
    float* lat = sm;
    float* wsl = sm + C;
    __shared__ float s_inv;
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    // the attention kernel's split of this context: slices of `per` positions, the first `nsplit` of them hold any
    const int attn_len = __ldcg(&st->pos) + 1;
    int per = (attn_len + nsplit_max - 1) / nsplit_max;
    per = (per + tile - 1) / tile * tile;
    const int nsplit = (attn_len + per - 1) / per;
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
    for (int c = 2 * tid; c < C; c += 2 * blockDim.x) {  // C is even
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 16
        for (int s = 0; s < nsplit; ++s) {  // slice order
            const float2 v = __ldcg(reinterpret_cast<const float2*>(part_acc + ((size_t)s * H + h) * C + c));
            a0 = fmaf(v.x, wsl[s], a0);
            a1 = fmaf(v.y, wsl[s], a1);
        }
        lat[c] = a0 * s_inv;
        lat[c + 1] = a1 * s_inv;
    }
    __syncthreads();
    // this CTA's 32 output rows of the head: four rows per warp, their loads in flight together
    const int dv0 = blockIdx.y * 32 + warp * 4;
    if (nw == 8 && dv0 + 4 <= V) {
        float y[4];
        warp_rows_dot<WT, 4>(wuv_t + ((size_t)h * V + dv0) * C, (size_t)C, lat, C, lane, y);
        if (lane < 4) attn_out[(size_t)h * V + dv0 + lane] = lane == 0 ? y[0] : lane == 1 ? y[1] : lane == 2 ? y[2] : y[3];
    } else {
        for (int dv = blockIdx.y * 32 + warp; dv < min(V, (int)blockIdx.y * 32 + 32); dv += nw) {
            const float v = warp_row_dot<WT>(wuv_t + ((size_t)h * V + dv) * C, lat, C, lane);
            if (lane == 0) attn_out[(size_t)h * V + dv] = v;
        }
    }
}

// ---------------------------------------------------------------------- latent attention on the tensor cores
// The absorbed form is a GEMM with M = heads: scores S[h, t] = qabs[h, :] . row(t) over the C + R wide
// cache row, output O[h, :] = sum_t p[h, t] row(t)[0 .. C).  mma.sync m16n8k16 with fp32 accumulation;
// the fp32 operands (q, p) are split into a 16-bit head and a 16-bit remainder (two MMAs), so only the
// cache itself carries its storage rounding.  One CTA of four warps per slice of cached positions, 64
// positions at a time: the tile's rows arrive by one bulk copy each (row stride padded by 16 bytes: ldmatrix
// without bank conflicts); warp w scores positions 16 w .. 16 w + 15, then owns latent columns
// 128 w .. 128 w + 127 of every head.  Geometry: 16-bit cache, C = 512, (C + R) % 16 == 0, heads <= 16.
constexpr int MLA_MMA_TILE = 64, MLA_MMA_C = 512, MLA_MMA_THREADS = 128;

template <typename KT> struct Mma16;
template <> struct Mma16<__half> {
    __device__ static inline void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Mma16<__nv_bfloat16> {
    __device__ static inline void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
__device__ inline void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ inline void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__host__ __device__ inline size_t mla_mma_smem_bytes(int W) {
    const size_t ldb = (size_t)W * 2 + 16;
    return (size_t)(MLA_MMA_TILE + 32) * ldb            // rows, q head, q remainder
           + (size_t)16 * (MLA_MMA_TILE + 1) * 4         // scores
           + (size_t)2 * 16 * (MLA_MMA_TILE + 8) * 2     // p head, p remainder
           + 3 * 16 * 4 + 16;                            // running max, sum, rescale; mbarrier
}

template <typename KT>
__global__ void __launch_bounds__(MLA_MMA_THREADS)
mla_attn_mma_kernel(const KT* __restrict__ qsplit, const KT* __restrict__ lat_pool, const int* __restrict__ page_table, const DevState* st,
                    float* __restrict__ part_acc, float* __restrict__ part_ml, MlaDims d, int nsplit, float scale, int* err) {
    extern __shared__ __align__(128) unsigned char smraw[];
    constexpr float NEG = -3.402823466e+38f;
    constexpr int T = MLA_MMA_TILE, C = MLA_MMA_C, LDS = T + 1, LDP = T + 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, H = d.heads, W = d.latent + d.rope, s = blockIdx.x;
    const uint32_t LDB = (uint32_t)W * 2u + 16u;
    unsigned char* rows_p = smraw;                                   // [T][LDB]
    unsigned char* qh_p = rows_p + (size_t)T * LDB;                  // [16][LDB]
    unsigned char* ql_p = qh_p + (size_t)16 * LDB;                   // [16][LDB], directly behind qh
    float* sc = reinterpret_cast<float*>(ql_p + (size_t)16 * LDB);   // [16][LDS]
    KT* ph = reinterpret_cast<KT*>(sc + 16 * LDS);                   // [16][LDP]
    KT* pl = ph + 16 * LDP;                                          // [16][LDP]
    float* mrun = reinterpret_cast<float*>(pl + 16 * LDP);           // [16]
    float* lrun = mrun + 16;
    float* corr = lrun + 16;
    uint64_t* bar_p = reinterpret_cast<uint64_t*>(corr + 16);
    const uint32_t rows = smem_addr(rows_p), qh = smem_addr(qh_p), ql = smem_addr(ql_p), bar = smem_addr(bar_p);
    const uint32_t pha = smem_addr(ph), pla = smem_addr(pl);

    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    const int attn_len = __ldcg(&st->pos) + 1;
    int per = (attn_len + nsplit - 1) / nsplit;
    per = (per + T - 1) / T * T;
    const int t0 = s * per, t1 = min(attn_len, t0 + per);
    if (t0 >= t1) return;  // a slice past the context: mla_out_kernel merges ceil(attn_len / per) slices only
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    if (tid < 16) { mrun[tid] = NEG; lrun[tid] = 0.0f; corr[tid] = 0.0f; }
    __syncthreads();
    auto fetch = [&](int tb, bool with_q) {  // warp 0: one bulk copy per cached row of the tile (and per row of q)
        const int nt = min(T, t1 - tb);
        if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(nt + (with_q ? 32 : 0)) * (uint32_t)W * 2u);
        __syncwarp();
        // q as mla_post_kernel left it: 16 rows of 16-bit heads, 16 rows of remainders (rows of heads that do not exist are zero)
        if (with_q) bulk_g2s(qh + (uint32_t)lane * LDB, qsplit + (size_t)lane * W, (uint32_t)W * 2u, bar);
        for (int j = lane; j < nt; j += 32) {
            const int t = tb + j, page = page_table[t / d.page_tokens], off = t % d.page_tokens;
            bulk_g2s(rows + (uint32_t)j * LDB, lat_pool + ((size_t)page * d.page_tokens + off) * W, (uint32_t)W * 2u, bar);
        }
    };
    if (warp == 0) fetch(t0, true);
    float acc[16][4];  // columns 128 warp + 8 nb + 2 (lane % 4) + {0, 1} of heads lane / 4 and lane / 4 + 8
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.0f;
    const int g = lane >> 2, tq = lane & 3;
    uint32_t phase = 0;
    for (int tb = t0; tb < t1; tb += T) {
        const int nt = min(T, t1 - tb);
        // rows past the slice's end are multiplied by p = 0: they must hold finite values
        for (int i = tid; i < (T - nt) * (int)(LDB / 16); i += MLA_MMA_THREADS)
            *reinterpret_cast<uint4*>(rows_p + (size_t)(nt + i / (int)(LDB / 16)) * LDB + (size_t)(i % (int)(LDB / 16)) * 16) = make_uint4(0, 0, 0, 0);
        if (!mbar_wait(bar, phase)) atomicCAS(err, 0, DEV_ERR_FULL_WAIT);
        phase ^= 1u;
        __syncthreads();  // the zero rows are in place
        // ---- scores of positions 16 warp .. 16 warp + 15
        const int j0 = 16 * warp;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        if (j0 < nt) {
            const uint32_t a_off = (uint32_t)(lane & 15) * LDB + (uint32_t)(lane >> 4) * 16u;
            const uint32_t b_off = (uint32_t)(j0 + (lane & 7) + 8 * (lane >> 4)) * LDB + (uint32_t)((lane >> 3) & 1) * 16u;
#pragma unroll 4
            for (int ks = 0; ks < W / 16; ++ks) {
                uint32_t ah[4], al[4], b[4];
                ldsm_x4(ah, qh + a_off + (uint32_t)ks * 32u);
                ldsm_x4(al, ql + a_off + (uint32_t)ks * 32u);
                ldsm_x4(b, rows + b_off + (uint32_t)ks * 32u);
                Mma16<KT>::mma(c0, ah, b[0], b[1]);
                Mma16<KT>::mma(c0, al, b[0], b[1]);
                Mma16<KT>::mma(c1, ah, b[2], b[3]);
                Mma16<KT>::mma(c1, al, b[2], b[3]);
            }
        }
        {
            const int ja = j0 + 2 * tq, jb = j0 + 8 + 2 * tq;
            sc[g * LDS + ja] = c0[0] * scale;       sc[g * LDS + ja + 1] = c0[1] * scale;
            sc[(g + 8) * LDS + ja] = c0[2] * scale; sc[(g + 8) * LDS + ja + 1] = c0[3] * scale;
            sc[g * LDS + jb] = c1[0] * scale;       sc[g * LDS + jb + 1] = c1[1] * scale;
            sc[(g + 8) * LDS + jb] = c1[2] * scale; sc[(g + 8) * LDS + jb + 1] = c1[3] * scale;
        }
        __syncthreads();
        // ---- running softmax: eight threads per head, eight positions each
        {
            const int h = tid >> 3, sub = tid & 7;
            float v[8], mx = NEG;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int j = sub * 8 + i;
                v[i] = j < nt ? sc[h * LDS + j] : NEG;
                mx = fmaxf(mx, v[i]);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mold = mrun[h], mnew = fmaxf(mold, mx);
            float ps = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int j = sub * 8 + i;
                const float p = j < nt ? expf(v[i] - mnew) : 0.0f;
                ps += p;
                const KT hi = Elem<KT>::from_f32(p);
                ph[h * LDP + j] = hi;
                pl[h * LDP + j] = Elem<KT>::from_f32(p - Elem<KT>::to_f32(hi));
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            __syncwarp();
            if (sub == 0) {
                const float cr = expf(mold - mnew);
                corr[h] = cr;
                lrun[h] = lrun[h] * cr + ps;
                mrun[h] = mnew;
            }
        }
        __syncthreads();
        // ---- O += P V over this warp's 128 latent columns
        {
            const float ca = corr[g], cb = corr[g + 8];
#pragma unroll
            for (int nb = 0; nb < 16; ++nb) { acc[nb][0] *= ca; acc[nb][1] *= ca; acc[nb][2] *= cb; acc[nb][3] *= cb; }
            const uint32_t a_off = (uint32_t)(lane & 15) * (uint32_t)(LDP * 2) + (uint32_t)(lane >> 4) * 16u;
            const uint32_t v_off = (uint32_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * LDB + (uint32_t)(128 * warp + 8 * (lane >> 4)) * 2u;
            for (int ks = 0; ks < T / 16; ++ks) {
                if (16 * ks >= nt) break;
                uint32_t ah[4], al[4];
                ldsm_x4(ah, pha + a_off + (uint32_t)ks * 32u);
                ldsm_x4(al, pla + a_off + (uint32_t)ks * 32u);
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, rows + v_off + (uint32_t)(16 * ks) * LDB + (uint32_t)np * 32u);
                    Mma16<KT>::mma(acc[2 * np], ah, b[0], b[1]);
                    Mma16<KT>::mma(acc[2 * np], al, b[0], b[1]);
                    Mma16<KT>::mma(acc[2 * np + 1], ah, b[2], b[3]);
                    Mma16<KT>::mma(acc[2 * np + 1], al, b[2], b[3]);
                }
            }
        }
        __syncthreads();  // every warp is done with the tile's rows
        if (warp == 0 && tb + T < t1) fetch(tb + T, false);
    }
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) {
        const int col = 128 * warp + 8 * nb + 2 * tq;
        if (g < H) *reinterpret_cast<float2*>(part_acc + ((size_t)s * H + g) * C + col) = make_float2(acc[nb][0], acc[nb][1]);
        if (g + 8 < H) *reinterpret_cast<float2*>(part_acc + ((size_t)s * H + g + 8) * C + col) = make_float2(acc[nb][2], acc[nb][3]);
    }
    if (tid < H) {
        part_ml[((size_t)s * H + tid) * 2 + 0] = mrun[tid];
        part_ml[((size_t)s * H + tid) * 2 + 1] = lrun[tid];
    }
}

// ---------------------------------------------------------------------- router: one warp per expert, the last CTA picks
// xn = rmsnorm(x, gamma) (every CTA, CTA 0 keeps it for the expert kernels), logit_e = W_r[e] . xn;
// the CTA that finishes last (a counter, nobody waits) computes p = softmax(logits) and the top_k
// largest p (k rounds of arg-max, ties to the lower expert index) with their weights, not
// renormalised.  Besides the choice (sel_ids, sel_w) it writes the compact list of the chosen experts
// this rank holds (local index, weight, count): the expert kernels walk that list.
template <typename WT>
__global__ void __launch_bounds__(128)
moe_router_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const WT* __restrict__ wr, float* __restrict__ xn_out,
                  float* __restrict__ logits, unsigned int* __restrict__ counter, int* __restrict__ sel_ids, float* __restrict__ sel_w,
                  int* __restrict__ loc_ids, float* __restrict__ loc_w, int* __restrict__ n_loc, int dim, int n_experts, int top_k, int e0,
                  int n_local) {
    extern __shared__ float sm[];  // [dim] x * gamma; the last CTA: [n_experts] probabilities on top of it
    __shared__ float red[32];
    __shared__ int s_last;
    constexpr int EPC = Elem<WT>::EPC, PRE = 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    float* xg = sm;
    // this warp's expert row: its first chunks are requested before anything else (x, gamma and the row arrive together)
    const int e = min(blockIdx.x * nw + warp, n_experts - 1);
    const char* row = reinterpret_cast<const char*>(wr + (size_t)e * dim);
    const int nchunks = dim / EPC;
    uint4 w[PRE];
#pragma unroll
    for (int j = 0; j < PRE; ++j) w[j] = lane + 32 * j < nchunks ? ldg_stream(row + (size_t)(lane + 32 * j) * 16) : make_uint4(0, 0, 0, 0);
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    float ss = 0.0f;
    for (int i = tid; i < dim; i += blockDim.x) {
        const float v = __ldcg(x + i);
        xg[i] = v * gamma[i];
        ss += v * v;
    }
    const float tot = block_sum(ss, red);  // (its barriers also publish xg)
    const float inv = 1.0f / sqrtf(tot * (1.0f / (float)dim) + RMS_EPS);
    if (blockIdx.x == 0)
        for (int i = tid; i < dim; i += blockDim.x) xn_out[i] = xg[i] * inv;
    // logit = inv * (row . (x * gamma))
    float a = 0.0f;
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
        const int c = lane + 32 * j;
        if (c < nchunks) {
            float f[EPC];
            Elem<WT>::unpack(w[j], f);
#pragma unroll
            for (int k = 0; k < EPC; ++k) a = fmaf(f[k], xg[c * EPC + k], a);
        }
    }
    for (int c = lane + 32 * PRE; c < nchunks; c += 32) {
        float f[EPC];
        Elem<WT>::unpack(ldg_stream(row + (size_t)c * 16), f);
#pragma unroll
        for (int k = 0; k < EPC; ++k) a = fmaf(f[k], xg[c * EPC + k], a);
    }
    a = warp_sum(a) * inv;
    if (lane == 0 && blockIdx.x * nw + warp < n_experts) logits[e] = a;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(counter, 1u) == gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (!s_last || warp != 0) return;
    __threadfence();
    float* pr = sm;  // x * gamma is no longer needed: the other warps have left, this one has its logit
    float mx = -INFINITY;
    for (int k = lane; k < n_experts; k += 32) {
        const float v = __ldcg(logits + k);
        pr[k] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    __syncwarp();
    for (int k = lane; k < n_experts; k += 32) pr[k] = expf(pr[k] - mx);
    __syncwarp();
    float sum = 0.0f;  // in expert order, the same in every lane
    for (int k = 0; k < n_experts; ++k) sum += pr[k];
    __syncwarp();
    for (int k = lane; k < n_experts; k += 32) pr[k] = pr[k] / sum;
    __syncwarp();
    int nl = 0;
    for (int k = 0; k < top_k; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane; i < n_experts; i += 32) {
            const float v = pr[i];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
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
            if (bi >= e0 && bi < e0 + n_local) { loc_ids[nl] = bi - e0; loc_w[nl] = bv; }
        }
        if (bi >= e0 && bi < e0 + n_local) ++nl;  // bi is the same in every lane after the exchange
        __syncwarp();
    }
    if (lane == 0) {
        *n_loc = nl;
        *counter = 0u;  // for the next launch
    }
}

struct MoeDims {
    int dim, hidden;
    int shared_cols;      // columns of the shared FFN this rank holds
};
// the chosen experts this rank holds, in the router's order: local index, weight; their count
struct MoePick {
    const int* loc_ids;
    const float* loc_w;
    const int* n_loc;
};

// ---------------------------------------------------------------------- gate = silu(xn W1) * (xn W3) * weight
// Units: for each chosen local expert `hidden` column pairs, then `shared_cols` pairs of the shared FFN; one
// warp per unit (rows 2j and 2j + 1 of an interleaved [2 hidden, dim] matrix are adjacent in memory).
// This and moe_w2_kernel are the plain-load forms, for shapes the streamed GEMV does not take.
template <typename WT>
__global__ void __launch_bounds__(256)
moe_w13_kernel(const float* __restrict__ xn, const WT* __restrict__ w13, const WT* __restrict__ ws13, MoePick pick,
               float* __restrict__ gate, MoeDims d) {
    extern __shared__ float xs[];  // [dim]
    const int tid = threadIdx.x, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    for (int i = tid; i < d.dim; i += blockDim.x) xs[i] = __ldcg(xn + i);
    __syncthreads();
    const int nl = __ldcg(pick.n_loc);
    const int units = nl * d.hidden + d.shared_cols;
    const int gw = (blockIdx.x * blockDim.x + tid) >> 5, total = (gridDim.x * blockDim.x) >> 5;
    for (int u = gw; u < units; u += total) {
        const WT* rows;
        float weight = 1.0f;
        if (u < nl * d.hidden) {
            const int s = u / d.hidden, j = u % d.hidden;
            rows = w13 + ((size_t)__ldcg(pick.loc_ids + s) * d.hidden + j) * 2 * d.dim;
            weight = __ldcg(pick.loc_w + s);
        } else {
            rows = ws13 + (size_t)(u - nl * d.hidden) * 2 * d.dim;
        }
        float y[2];
        warp_rows_dot<WT, 2>(rows, (size_t)d.dim, xs, d.dim, lane, y);
        if (lane == 0) gate[u] = (y[0] / (1.0f + expf(-y[0]))) * y[1] * weight;
    }
}

// ---------------------------------------------------------------------- y = sum of W2 gate over the local experts and the shared FFN
// One warp per output row.  Single GPU: out = res + alpha y.  Expert parallel: y goes to every rank's inbox
// (the dense model's push all-reduce, TpRegion); the next GEMV's prologue adds the ranks' rows in rank order.
template <typename WT>
__global__ void __launch_bounds__(256)
moe_w2_kernel(const float* __restrict__ gate, const WT* __restrict__ w2, const WT* __restrict__ ws2, MoePick pick,
              const float* __restrict__ res, float* __restrict__ out, float alpha, MoeDims d, TpLink tp) {
    extern __shared__ float gs[];  // [n_loc * hidden + shared_cols]
    const int tid = threadIdx.x, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();  // after the wait: at most this kernel and the next one overlap
    const int nl = __ldcg(pick.n_loc);
    const int units = nl * d.hidden + d.shared_cols;
    for (int i = tid; i < units; i += blockDim.x) gs[i] = __ldcg(gate + i);
    __syncthreads();
    const int gw = (blockIdx.x * blockDim.x + tid) >> 5, total = (gridDim.x * blockDim.x) >> 5;
    constexpr int EPC = Elem<WT>::EPC;
    for (int r = gw; r < d.dim; r += total) {
        float a = 0.0f;  // this lane's share of the row's sum over every segment: one reduction at the end, loads of all segments independent
        for (int s = 0; s <= nl; ++s) {
            const WT* seg;
            const float* g = gs + s * d.hidden;
            int K;
            if (s < nl) {
                seg = w2 + ((size_t)__ldcg(pick.loc_ids + s) * d.dim + r) * d.hidden; K = d.hidden;
            } else {
                if (d.shared_cols == 0) continue;
                seg = ws2 + (size_t)r * d.shared_cols; K = d.shared_cols;
            }
#pragma unroll 4
            for (int c = lane; c < K / EPC; c += 32) {
                const uint4 w = ldg_stream(reinterpret_cast<const char*>(seg) + (size_t)c * 16);
                float f[EPC];
                Elem<WT>::unpack(w, f);
#pragma unroll
                for (int e = 0; e < EPC; e += 4) {
                    const float4 x4 = *reinterpret_cast<const float4*>(g + c * EPC + e);
                    a = fmaf(f[e], x4.x, a); a = fmaf(f[e + 1], x4.y, a); a = fmaf(f[e + 2], x4.z, a); a = fmaf(f[e + 3], x4.w, a);
                }
            }
        }
        const float y = warp_sum(a);
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
