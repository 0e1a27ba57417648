// Shared device/host helpers for the cuda_decode library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cd {

constexpr float RMS_EPS = 1e-5f;  // metal-decode/src/lib.rs:14, cpu/rmsnorm.rs:10
constexpr int HEAD_BLOCK = 256;   // vocab rows per head block, lib.rs:156

// Device-resident per-sequence state.  Kernels read position and token from here
// so that one captured graph can be replayed for every step.
struct DevState {
    int32_t pos;         // slot the current token is written to (= cached length)
    uint32_t token;      // token fed to the embedding gather
    uint64_t rng;        // LCG state of the running sample (inference.rs:759)
    int32_t nout;        // tokens appended to the output ring so far
    int32_t error;       // first device-side error code (0 = none)
    int32_t block_idx;   // last block chosen by the full-vocab sampler
    int32_t cursor;      // next prompt token to feed during prefill
};

// ------------------------------------------------------------------ synthetic tensors
// Counter-based generator: three SplitMix64 outputs per element, their twelve 16-bit
// fields summed (Irwin–Hall: mean 393210, variance 65536^2), centred and scaled.
// Integer arithmetic up to one final multiply, so host and device agree bit for bit.
constexpr uint64_t GOLDEN = 0x9E3779B97F4A7C15ull;
__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}
__host__ __device__ inline uint32_t sum16(uint64_t a) {
    return (uint32_t)(a & 0xffff) + (uint32_t)((a >> 16) & 0xffff) + (uint32_t)((a >> 32) & 0xffff) +
           (uint32_t)(a >> 48);
}
__host__ __device__ inline uint64_t synth_key(uint64_t seed, uint64_t uid) { return mix64(seed ^ mix64(uid + GOLDEN)); }
__host__ __device__ inline float synth_value(uint64_t key, uint64_t idx, float scale) {
    const uint64_t base = key + 3 * idx * GOLDEN;
    const uint32_t s = sum16(mix64(base + GOLDEN)) + sum16(mix64(base + 2 * GOLDEN)) + sum16(mix64(base + 3 * GOLDEN));
    return (float)((int32_t)s - 393210) * scale;
}
// tensor uids: 0 embed, 2 lm_head, 16 + 16*layer + {0 wq,1 wk,2 wv,3 wo,4 w1,5 w3,6 w2}
__host__ __device__ inline uint64_t synth_uid_layer(int layer, int which) { return 16 + (uint64_t)layer * 16 + (uint64_t)which; }

// ------------------------------------------------------------------ storage types
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int EPC = 4;  // elements per 16-byte chunk
    __device__ static inline void unpack(const uint4& w, float (&f)[4]) {
        f[0] = __uint_as_float(w.x); f[1] = __uint_as_float(w.y); f[2] = __uint_as_float(w.z); f[3] = __uint_as_float(w.w);
    }
    __host__ __device__ static inline float from_f32(float v) { return v; }
    __device__ static inline float to_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int EPC = 8;
    __device__ static inline void unpack(const uint4& w, float (&f)[8]) {
        f[0] = __uint_as_float(w.x << 16); f[1] = __uint_as_float(w.x & 0xffff0000u);
        f[2] = __uint_as_float(w.y << 16); f[3] = __uint_as_float(w.y & 0xffff0000u);
        f[4] = __uint_as_float(w.z << 16); f[5] = __uint_as_float(w.z & 0xffff0000u);
        f[6] = __uint_as_float(w.w << 16); f[7] = __uint_as_float(w.w & 0xffff0000u);
    }
    __device__ static inline __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
    __device__ static inline float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct Elem<__half> {
    static constexpr int EPC = 8;
    __device__ static inline void unpack(const uint4& w, float (&f)[8]) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&w.w));
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    }
    __device__ static inline __half from_f32(float v) { return __float2half_rn(v); }
    __device__ static inline float to_f32(__half v) { return __half2float(v); }
};

// 16-byte streaming load: read-only path, no L1 allocation (weights and KV are
// touched once per token).
__device__ inline uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum R per-lane values across the warp with R + log2(32/R) ... shuffles instead of
// 5R: each halving step trades half of the rows for the other half-warp's copy.
// Afterwards every lane of an aligned group of 32/R lanes holds the total of row
// `row`; callers let the first lane of each group write.
template <int R> __device__ inline float warp_reduce_rows(float (&v)[R], int lane, int& row) {
    row = 0;
    int width = 16;
#pragma unroll
    for (int n = R; n > 1; n >>= 1, width >>= 1) {
        const bool hi = (lane & width) != 0;
#pragma unroll
        for (int j = 0; j < n / 2; ++j) {
            const float send = hi ? v[j] : v[j + n / 2];
            const float keep = hi ? v[j + n / 2] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, width);
        }
        if (hi) row += n / 2;
    }
#pragma unroll
    for (; width >= 1; width >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], width);
    return v[0];
}

// Block-wide sum / max for up to 1024 threads; `red` is 32 floats of shared memory.
__device__ inline float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}
__device__ inline float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = red[0];
    for (int i = 1; i < nw; ++i) t = fmaxf(t, red[i]);
    return t;
}

}  // namespace cd
