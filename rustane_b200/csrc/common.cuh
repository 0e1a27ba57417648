// Shared device/host helpers for the cuda_decode library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
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
    unsigned long long epoch;  // persistent-kernel launches completed (grid-barrier bookkeeping)
    uint32_t ar_base;    // tensor-parallel all-reduces issued by the tokens completed so far (same on every rank)
    uint32_t cand_seq;   // tensor-parallel head exchanges issued so far
};

// ------------------------------------------------------------------ tensor-parallel link
// Every rank owns one "link region" in its HBM that its peers map through CUDA IPC:
//   inbox  [3 slots][world][dim] fp32   partial vectors pushed by the peers (and by itself)
//   cand   [2 slots][world] (f32, u32)  best (logit, token) of each rank's vocabulary shard
//   cflags [2 slots][world] u32         sequence number of the head exchange a cand row holds
// An all-reduce is push-based and one-shot: the GEMV that produces a partial vector stores
// it straight into every peer's inbox from its epilogue (plain 4-byte peer stores over
// NVLink).  There is no flag and no fence: an inbox word that has not arrived yet holds a
// sentinel bit pattern no result can have, and the consuming GEMV polls the words it needs
// (bounded) until none is the sentinel, then adds the world rows in fixed rank order, so
// every rank computes a bit-identical residual stream.  Slots rotate over three buffers:
// the consumer of all-reduce k re-arms slot (k+2) mod 3, which every rank finished reading
// before any rank can push all-reduce k+2 (a rank pushes k+2 only after it consumed k+1,
// i.e. after every rank pushed k+1, i.e. after every rank ran the consumer of k).
// Data always lands in the consumer's own memory before it is used.
constexpr int TP_MAX = 8;
struct TpRegion {
    __host__ __device__ static size_t inbox_off() { return 0; }
    __host__ __device__ static size_t cand_off(int world, int dim) { return (size_t)3 * world * dim * 4; }
    __host__ __device__ static size_t cflags_off(int world, int dim) { return cand_off(world, dim) + 256; }
    __host__ __device__ static size_t bytes(int world, int dim) { return cflags_off(world, dim) + 256; }
    // top-k exchange (sampled decoding): [2 slots] { vals [world][nb * 32] f32, idxs [world][nb * 32] u32 },
    // nb = head blocks per rank (the same number on every rank), announced through the same cflags
    __host__ __device__ static size_t topk_off(int world, int dim) { return bytes(world, dim); }
    __host__ __device__ static size_t topk_slot_bytes(int world, int nb) { return (size_t)2 * world * nb * 32 * 4; }
    __host__ __device__ static size_t bytes_with_topk(int world, int dim, int nb) { return topk_off(world, dim) + 2 * topk_slot_bytes(world, nb); }
    // batched prompt pass: [2 buffers][world] u32 sequence numbers a rank's peers write ("my partial sums of all-reduce
    // seq are in my buffer"), then this rank's two buffers of [rows][dim] fp32 partial sums, which the peers read
    __host__ __device__ static size_t pf_flags_off(int world, int dim, int nb) { return (bytes_with_topk(world, dim, nb) + 255) & ~(size_t)255; }
    __host__ __device__ static size_t pf_buf_off(int world, int dim, int nb) { return pf_flags_off(world, dim, nb) + 256; }
    __host__ __device__ static size_t bytes_with_prefill(int world, int dim, int nb, size_t rows) {
        return pf_buf_off(world, dim, nb) + 2 * rows * (size_t)dim * 4;
    }
};
struct TpLink {          // world <= 1: single GPU, nothing below is used
    int world, rank, dim;
    char* peers[TP_MAX];  // link region of every rank as mapped into this process (peers[rank] = own)
    DevState* st;
    int ar_out;           // pushing kernel: index (1-based within the token) of the all-reduce it issues
    // consumer side of a GEMV whose input is an all-reduced vector: x = res + alpha * sum(inbox rows)
    int in_reduce;        // index (1-based within the token) of the all-reduce to consume, 0 = none
    const float* res;
    float alpha;
    float* x_out;
    unsigned long long wait_ns;  // bound of every wait on a peer (cd_options.wait_us)
};
// Waits on a peer are bounded by time (globaltimer), not by iterations, and they are sticky: once
// any wait of this rank has run out (DevState::error != 0) every later wait returns at once, so a
// peer that stopped costs one budget per call, not one per all-reduce of every remaining token.
__device__ inline unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ inline bool dev_failed(const DevState* st) { return *reinterpret_cast<const volatile int32_t*>(&st->error) != 0; }
constexpr int TP_POLLS_PER_CLOCK_READ = 64;
constexpr uint32_t TP_SENTINEL = 0xffffffffu;  // "not arrived": a NaN payload no kernel here produces
__device__ inline float tp_sanitize(float v) {
    return __float_as_uint(v) == TP_SENTINEL ? __uint_as_float(0x7fffffffu) : v;
}
// Sum over ranks (in rank order) of the four words at offset `at` of every rank's inbox row.  All
// loads of a round are issued before any is looked at, so a round costs one memory latency
// instead of one per rank; rows that have not arrived are polled again until the time budget is
// spent.  false on expiry, and at once when this rank has already failed.
__device__ inline bool tp_gather4(const float* inbox, int world, int dim, size_t at, float4& sum, const DevState* st, unsigned long long budget_ns) {
    uint4 v[TP_MAX];
#pragma unroll
    for (int r = 0; r < TP_MAX; ++r) v[r] = make_uint4(0u, 0u, 0u, 0u);
    unsigned pending = (1u << world) - 1u;
    if (dev_failed(st)) { sum = make_float4(0.f, 0.f, 0.f, 0.f); return false; }
    unsigned long long t0 = 0;
    for (int i = 0; pending; ++i) {
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
            if (pending >> r & 1u)
                asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(inbox + (size_t)r * dim + at) : "memory");
#pragma unroll
        for (int r = 0; r < TP_MAX; ++r)
            if ((pending >> r & 1u) && v[r].x != TP_SENTINEL && v[r].y != TP_SENTINEL && v[r].z != TP_SENTINEL && v[r].w != TP_SENTINEL)
                pending &= ~(1u << r);
        if (pending && (i % TP_POLLS_PER_CLOCK_READ) == TP_POLLS_PER_CLOCK_READ - 1) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > budget_ns || dev_failed(st)) break;
        }
    }
    sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < TP_MAX; ++r)
        if (r < world) {
            sum.x += __uint_as_float(v[r].x); sum.y += __uint_as_float(v[r].y);
            sum.z += __uint_as_float(v[r].z); sum.w += __uint_as_float(v[r].w);
        }
    return pending == 0;
}
enum { DEV_ERR_TP_WAIT = 4, DEV_ERR_BAD_TOKEN = 5 };
// The token id a step starts from, as a row of the embedding table.  An id past the vocabulary cannot come from a
// caller (the host checks) but it can come from the device's own arg-max over logits that are all NaN: it is
// replaced by row 0 and recorded, never used as an address.
__device__ inline uint32_t checked_token(uint32_t tok, int vocab, int* err) {
    if (tok < (uint32_t)vocab) return tok;
    atomicCAS(err, 0, DEV_ERR_BAD_TOKEN);
    return 0u;
}

__device__ inline void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ inline unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// wait until *p (written by a peer GPU into local memory) reaches `want`; false on expiry, and at
// once when this rank has already failed
__device__ inline bool tp_wait_flag(const unsigned int* p, unsigned int want, const DevState* st, unsigned long long budget_ns) {
    if (dev_failed(st)) return false;
    unsigned long long t0 = 0;
    for (int i = 0;; ++i) {
        if ((int)(ld_acquire_sys(p) - want) >= 0) return true;
        if ((i % TP_POLLS_PER_CLOCK_READ) == TP_POLLS_PER_CLOCK_READ - 1) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > budget_ns || dev_failed(st)) return false;
        }
    }
}

// Where the next weight-streaming kernel of the token will start reading, so that a CTA
// can pull the head of that stream into L2 while its own tail and the launch gap pass.
struct NextStream {
    const void* w;       // nullptr: nothing to prefetch
    uint32_t row_bytes;
    int nunits, unit;    // the next kernel's row partition (same grid size assumed)
    uint32_t bytes;      // per CTA
    int test_drop;       // test hook (cd_options.test_flags bit 3): CTA 0 withholds its last stage and waits only briefly for it
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

// ------------------------------------------------------------------ weight-row formats of the GEMV
// How one matrix row is laid out in HBM and how a 16-byte chunk of it meets the
// thread's slice of x.  Plain element types: K elements, nothing else.  The two
// quantised formats keep their scales inside the row, so one bulk copy brings a
// row and everything needed to decode it (no reference counterpart):
//   Fp8Row   K e4m3 bytes, then the row's fp32 scale (row padded to 16 bytes);
//            w = e4m3 * scale, scale = max|row| / 448
//   Int4G32  K/2 bytes of nibbles (value q + 8), then K/32 fp16 group scales, padded to
//            16 bytes; w = q * scale, q in [-8, 7], scale = fp16(max|group| / 7); 16 bytes
//            of nibbles = one group.  Inside each little-endian 32-bit word, element
//            e (0..7) sits in nibble (e >> 1) + 4 * (e & 1): nibbles j and j + 4 are
//            neighbours, so one mask yields a pair that meets an adjacent pair of x
// packed fp32 FMA (two lanes per instruction): acc += a * b
__device__ inline void ffma2(float2& acc, const float2 a, const float2 b) {
    unsigned long long c = *reinterpret_cast<unsigned long long*>(&acc);
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(*reinterpret_cast<const unsigned long long*>(&a)), "l"(*reinterpret_cast<const unsigned long long*>(&b)));
    acc = *reinterpret_cast<float2*>(&c);
}
struct Fp8Row { unsigned char b; };
struct Int4G32 { unsigned char b; };

template <typename T> struct Wfmt {
    static constexpr int EPC = Elem<T>::EPC;
    static constexpr bool QUANT = false, ROW_SCALE = false, CHUNK_SCALE = false;
    static constexpr int CHUNK_BYTES = 16, SCALE_SHIFT = 0;  // bytes a thread takes per step; chunks per scale = 1 << SCALE_SHIFT
    __host__ __device__ static inline uint32_t row_stride(int K) { return (uint32_t)K * (uint32_t)sizeof(T); }
    __host__ __device__ static inline uint32_t scale_off(int) { return 0; }
    __device__ static inline float dot(const uint4& w, uint32_t, const float (&x)[EPC], float a) {
        float f[EPC];
        Elem<T>::unpack(w, f);
#pragma unroll
        for (int e = 0; e < EPC; ++e) a = fmaf(f[e], x[e], a);
        return a;
    }
};
template <> struct Wfmt<Fp8Row> {
    static constexpr int EPC = 16;
    static constexpr bool QUANT = true, ROW_SCALE = true, CHUNK_SCALE = false;
    static constexpr int CHUNK_BYTES = 16, SCALE_SHIFT = 0;
    __host__ __device__ static inline uint32_t row_stride(int K) { return (uint32_t)K + 16u; }
    __host__ __device__ static inline uint32_t scale_off(int K) { return (uint32_t)K; }
    // Decoding is kept off the integer pipe (it saturates first when every byte is an
    // element): the hardware e4m3x2 -> f16x2 conversion, an exact widening to fp32, then
    // packed fp32 FMAs into four independent chains.
    __device__ static inline float dot(const uint4& w, uint32_t, const float (&x)[16], float a) {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t v = ws[q];
            const __half2 h01(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3));
            const __half2 h23(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3));
            ffma2(s0, __half22float2(h01), make_float2(x[4 * q + 0], x[4 * q + 1]));
            ffma2(s1, __half22float2(h23), make_float2(x[4 * q + 2], x[4 * q + 3]));
        }
        return a + ((s0.x + s0.y) + (s1.x + s1.y));
    }
};
template <> struct Wfmt<Int4G32> {
    static constexpr int EPC = 16;  // a thread takes half a group (8 bytes) per step, so that K = 4096 still fills 256 threads
    static constexpr bool QUANT = true, ROW_SCALE = false, CHUNK_SCALE = true;
    static constexpr int CHUNK_BYTES = 8, SCALE_SHIFT = 1;
    __host__ __device__ static inline uint32_t row_stride(int K) { return ((uint32_t)K / 2u + (uint32_t)K / 16u + 15u) & ~15u; }
    __host__ __device__ static inline uint32_t scale_off(int K) { return (uint32_t)K / 2u; }
    // Two nibbles at a time: masked into the mantissas of a pair of fp16 1024.0 they read
    // as 1024 + n; subtracting 1032 in fp16 is exact and leaves q = n - 8, which is widened
    // to fp32 for packed FMAs.  One logic op per pair (plus three shifts per word) on the
    // integer pipe; the rest runs on the floating-point pipes.
    __device__ static inline float dot(const uint4& w, uint32_t scale_bits, const float (&x)[16], float a) {
        const uint32_t ws[2] = {w.x, w.y};
        const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6408));  // 1032.0
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint32_t v = ws[q];
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // nibbles k and k + 4 of the word = elements 8q + 2k and 8q + 2k + 1
                const uint32_t bits = ((v >> (4 * k)) & 0x000F000Fu) | 0x64006400u;
                const float2 f = __half22float2(__hsub2(*reinterpret_cast<const __half2*>(&bits), bias));
                ffma2((k & 1) ? s1 : s0, f, make_float2(x[8 * q + 2 * k], x[8 * q + 2 * k + 1]));
            }
        }
        const float t = (s0.x + s0.y) + (s1.x + s1.y);
        return fmaf(t, __half2float(__ushort_as_half((unsigned short)scale_bits)), a);
    }
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

// ------------------------------------------------------------------ sm_100a async-copy plumbing
// mbarrier + 1-D bulk copy (the TMA engine without a tensor map) and programmatic
// dependent launch.  Every wait is bounded: on expiry the caller records an error
// code in DevState::error and leaves the kernel instead of spinning for ever.
__device__ inline uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ inline void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ inline void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ inline void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
constexpr int MBAR_WAIT_LIMIT = 1 << 22;  // try_wait suspends for a while per call: seconds in total
__device__ inline bool mbar_wait(uint32_t bar, uint32_t parity, int limit = MBAR_WAIT_LIMIT) {
    for (int i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completion counted on an mbarrier of the same CTA.  Local memory only, no multicast.
__device__ inline void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// The same copy tagged evict-first in L2: weights are read once per token and are far
// larger than L2, so they should not push out the few KB that are re-read all the
// time (activations, RoPE rows, page table, attention partials).
__device__ inline uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ inline void bulk_g2s_stream(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
// Fire-and-forget request to bring `bytes` (multiple of 16) at `src` into L2.
__device__ inline void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ inline uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// Programmatic dependent launch: let the next kernel of the stream start its
// (input-independent) prologue now; wait for the previous kernel's results.
__device__ inline void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ inline void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

enum { DEV_ERR_NONE = 0, DEV_ERR_FULL_WAIT = 1, DEV_ERR_EMPTY_WAIT = 2 };

// 16-byte streaming load of data another kernel of the same token wrote (KV rows):
// L2-only path (ld.global.cg): never served from L1, never non-coherent.  Under programmatic dependent
// launch kernels of one chain overlap, so nothing written during a token may be read
// through the non-coherent path or trusted in L1; activations use ld.global.cg.
__device__ inline uint4 ldg_stream_coherent(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p) : "memory");
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
