// Batched prefill for sm_100a: every linear of the prompt pass is one tensor-core GEMM
//   C[M tokens, N features] = A[M, K] (activations, 16-bit) * B[N, K]^T (weights as stored for the GEMVs)
// issued with tcgen05.mma, accumulators in tensor memory, operands staged by TMA.
// The same kernel also computes the attention of the prompt as two batched GEMMs per
// layer (scores = Q K^T over the paged cache, output = P V) with a row softmax between.
// Math follows the naive forward (full_model.rs:336-437, layer.rs:1287-1431) restricted to
// the prompt positions; K and V land in the decode layout (pages).  There is no batched
// prompt pass in the reference's Metal decoder: it feeds prompt tokens one at a time
// (inference.rs:650-670).
//
// One CTA = one 128 x BN output tile.  Warp 0: TMA producer (one thread).  Warp 1: owns the
// tensor-memory allocation and issues the MMAs (one thread).  Warps 2-5: epilogue, each
// reading the 32 accumulator lanes tcgen05.ld lets it see (lanes 32 * (warp % 4) ...).
// Shared memory: a ring of NST stages, each a [128][64] A tile and a [BN][64] B tile of
// 16-bit elements in the 128-byte-swizzled K-major layout TMA writes and the MMA reads.
// Every wait is bounded; on expiry the kernel records an error, skips its remaining
// work, still meets the final barrier and frees its tensor memory.
//
// Further down: pf_skinny_kernel, the same machinery with the operands swapped for at most 16
// activation rows (several samples decoding together), its epilogues, and the small kernels
// around both (embedding rows, RMSNorm to hi + lo 16-bit operands, softmax, V transpose).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace cd {

constexpr int PF_BM = 128, PF_BK = 64, PF_THREADS = 192;
enum { DEV_ERR_PF_FULL = 8, DEV_ERR_PF_EMPTY = 9, DEV_ERR_PF_ACCUM = 10 };

// SPLIT: the activation operand arrives as two 16-bit matrices hi + lo (lo = the rounding
// error of hi, itself rounded), both multiplied with the same weight tile into the same
// accumulator, so the product sees about 16 mantissa bits of the fp32 activation instead of 8.
template <int BN, bool SPLIT> struct PfTile {
    static constexpr uint32_t A_BYTES = PF_BM * PF_BK * 2, B_BYTES = BN * PF_BK * 2, STAGE = (SPLIT ? 2 : 1) * A_BYTES + B_BYTES;
    static constexpr int NST = (192 * 1024) / STAGE > 6 ? 6 : (192 * 1024) / STAGE;
    static constexpr size_t SMEM = (size_t)NST * STAGE + 1024 /* alignment slack */ + 256 /* barriers */;
};

struct PfGemm {
    int M, N, K;        // one problem per blockIdx.z
    int a_col_z;        // A column offset per z (a head's slice of q; 0 otherwise)
    int a_row_z;        // A row offset per z (a head's plane of P)
    int b_row_z;        // B row offset per z / b_zdiv (a kv head's rows of V^T)
    int b_zdiv;         // query heads per kv head
    int b_paged;        // 1: B is the K half of the paged cache through a 5-D map {d, token, kv head, k|v, page}
    int page_tokens;
    int causal;         // 1: tiles wholly above the diagonal are skipped; 2: the K loop stops at the diagonal
    int pos0;           // tokens already cached before this prompt chunk
    int* err;
    // FP8 linears: B holds the e4m3 values widened to 16 bits; output column n is multiplied by the
    // row scale stored behind row n of the quantised matrix (Wfmt<Fp8Row>), nullptr otherwise
    const unsigned char* qrows;
    uint32_t qstride, qscale_off;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ inline void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ inline void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ inline void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ inline void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ inline void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ inline void umma_commit(uint32_t bar) {  // arrives on bar once every MMA issued so far has finished
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ inline void tmem_ld32(uint32_t taddr, float (&v)[32]) {  // this lane's 32 consecutive accumulator columns
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte rows written by TMA with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart; the leading-dimension field is
// not used for this layout; descriptor version 1 (sm_100); swizzle mode 2 (128 B).
__device__ inline uint64_t umma_desc(uint32_t tile_smem) {
    uint64_t d = (uint64_t)((tile_smem & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// ------------------------------------------------------------------ epilogues: (z, row, first column, 32 values)
template <typename T16> __device__ inline T16 pf_cast(float v);
template <> __device__ inline __nv_bfloat16 pf_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ inline __half pf_cast<__half>(float v) { return __float2half_rn(v); }

struct PfEpiPartial {  // tensor parallel: this rank's partial product y, raw, for the all-reduce that follows
    float* y;
    int ld;
    __device__ void operator()(int, int row, int col, const float (&v)[32]) const {
        float4* p = reinterpret_cast<float4*>(y + (size_t)row * ld + col);
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
};

struct PfEpiResidual {  // x += alpha * y on the fp32 residual stream
    float* x;
    int ld;
    float alpha;
    __device__ void operator()(int, int row, int col, const float (&v)[32]) const {
        float4* p = reinterpret_cast<float4*>(x + (size_t)row * ld + col);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4 t = p[i];
            t.x += alpha * v[4 * i]; t.y += alpha * v[4 * i + 1]; t.z += alpha * v[4 * i + 2]; t.w += alpha * v[4 * i + 3];
            p[i] = t;
        }
    }
};

// value -> hi (+ lo when a second matrix is kept)
template <typename T16> __device__ inline void pf_store(T16* hi, T16* lo, size_t at, float v) {
    const T16 h = pf_cast<T16>(v);
    hi[at] = h;
    if (lo != nullptr) lo[at] = pf_cast<T16>(v - Elem<T16>::to_f32(h));
}

template <typename T16> struct PfEpiGate {  // columns (2j, 2j+1) = (w1, w3) column j: gate[j] = act(y1) * y3
    T16* gate;
    T16* gate_lo;
    int ld, act;
    __device__ void operator()(int, int row, int col, const float (&v)[32]) const {
        const size_t at = (size_t)row * ld + (col >> 1);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float y1 = v[2 * j], y3 = v[2 * j + 1];
            float a;
            if (act == 1) {
                const float l = fmaxf(y1, 0.5f * y1);
                a = l * l;
            } else {
                a = y1 / (1.0f + expf(-y1));
            }
            pf_store(gate, gate_lo, at + j, a * y3);
        }
    }
};

template <typename T16> struct PfEpiQKV {  // RoPE on q and k; q to a [M, Q] buffer, k and v into the pages
    T16* q;
    T16* q_lo;
    T16* kv_pool;
    const int* page_table;
    const float2* rope;
    int Q, KV, hd, kv_heads, page_tokens, pos0;
    __device__ void operator()(int, int row, int col, const float (&v)[32]) const {
        const int pos = pos0 + row;
        if (col < Q + KV) {
            float r[32];
            const float2* cs = rope + (size_t)pos * (hd >> 1) + ((col % hd) >> 1);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float2 c = cs[j];
                r[2 * j] = v[2 * j] * c.x - v[2 * j + 1] * c.y;
                r[2 * j + 1] = v[2 * j + 1] * c.x + v[2 * j] * c.y;
            }
            T16* dst;
            if (col < Q) {
#pragma unroll
                for (int j = 0; j < 32; ++j) pf_store(q, q_lo, (size_t)row * Q + col + j, r[j]);
                return;
            } else {
                const int ck = col - Q, head = ck / hd, d = ck % hd;
                const int page = page_table[pos / page_tokens], off = pos % page_tokens;
                dst = kv_pool + ((((size_t)page * 2 + 0) * kv_heads + head) * page_tokens + off) * hd + d;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[j] = pf_cast<T16>(r[j]);
        } else {
            const int cv = col - Q - KV, head = cv / hd, d = cv % hd;
            const int page = page_table[pos / page_tokens], off = pos % page_tokens;
            T16* dst = kv_pool + ((((size_t)page * 2 + 1) * kv_heads + head) * page_tokens + off) * hd + d;
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[j] = pf_cast<T16>(v[j]);
        }
    }
};

struct PfEpiScores {  // raw q.k into the fp32 score planes [heads][rows][ld]
    float* s;
    size_t plane;
    int ld;
    __device__ void operator()(int z, int row, int col, const float (&v)[32]) const {
        float4* p = reinterpret_cast<float4*>(s + (size_t)z * plane + (size_t)row * ld + col);
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
};

template <typename T16> struct PfEpiAttnOut {  // head z's output columns of the [M, Q] attention buffer
    T16* out;
    T16* out_lo;
    int ld, hd;
    __device__ void operator()(int z, int row, int col, const float (&v)[32]) const {
        const size_t at = (size_t)row * ld + z * hd + col;
#pragma unroll
        for (int j = 0; j < 32; ++j) pf_store(out, out_lo, at + j, v[j]);
    }
};

// ------------------------------------------------------------------ the GEMM
template <int BN, bool SPLIT, class Epi>
__global__ void __launch_bounds__(PF_THREADS, 1)
pf_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_a_lo, const __grid_constant__ CUtensorMap tma_b,
               PfGemm p, uint32_t idesc, Epi epi) {
    using TL = PfTile<BN, SPLIT>;
    constexpr uint32_t B_OFF = (SPLIT ? 2 : 1) * TL::A_BYTES;  // stage = A hi | A lo (SPLIT) | B
    constexpr int NST = TL::NST;
    extern __shared__ unsigned char pf_raw[];
    const int m0 = blockIdx.y * PF_BM, n0 = blockIdx.x * BN, z = blockIdx.z;
    if (p.causal == 1 && n0 > p.pos0 + m0 + PF_BM - 1) return;  // every key of this tile lies after every query of it
    int kmax = p.K;
    if (p.causal == 2) kmax = min(kmax, p.pos0 + m0 + PF_BM);    // P is zero beyond the diagonal
    const int nkb = (kmax + PF_BK - 1) / PF_BK;

    const uint32_t tiles = (smem_addr(pf_raw) + 1023u) & ~1023u;
    const uint32_t bars = tiles + NST * TL::STAGE;
    const uint32_t full0 = bars, empty0 = bars + 8u * NST, accum = bars + 16u * NST, slot = accum + 8u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, 1);
        }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(slot, BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(slot));
    bool failed = false;

    if (warp == 0) {
        if (lane == 0) {  // ---- TMA producer
            const int zb = z / p.b_zdiv;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % NST;
                if (kb >= NST && !mbar_wait(empty0 + 8u * s, ((kb / NST) - 1) & 1)) {
                    atomicExch(p.err, DEV_ERR_PF_EMPTY);
                    failed = true;
                    break;
                }
                const uint32_t a_dst = tiles + s * TL::STAGE, b_dst = a_dst + B_OFF;
                mbar_arrive_expect_tx(full0 + 8u * s, TL::STAGE);
                tma_load_2d(a_dst, &tma_a, z * p.a_col_z + kb * PF_BK, z * p.a_row_z + m0, full0 + 8u * s);
                if (SPLIT) tma_load_2d(a_dst + TL::A_BYTES, &tma_a_lo, z * p.a_col_z + kb * PF_BK, z * p.a_row_z + m0, full0 + 8u * s);
                if (p.b_paged) tma_load_5d(b_dst, &tma_b, kb * PF_BK, 0, zb, 0, n0 / p.page_tokens, full0 + 8u * s);
                else tma_load_2d(b_dst, &tma_b, kb * PF_BK, zb * p.b_row_z + n0, full0 + 8u * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- MMA issuer
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % NST;
                if (!mbar_wait(full0 + 8u * s, (kb / NST) & 1)) {
                    atomicExch(p.err, DEV_ERR_PF_FULL);
                    failed = true;
                    break;
                }
                tc_fence_after();
                const uint64_t adesc = umma_desc(tiles + s * TL::STAGE), bdesc = umma_desc(tiles + s * TL::STAGE + B_OFF);
                const uint64_t ldesc = umma_desc(tiles + s * TL::STAGE + TL::A_BYTES);
#pragma unroll
                for (int k = 0; k < PF_BK / 16; ++k) {  // 16 elements = 32 bytes further along K inside the swizzle span
                    umma_f16(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0);
                    if (SPLIT) umma_f16(tmem_base, ldesc + 2u * k, bdesc + 2u * k, idesc, 1u);
                }
                umma_commit(empty0 + 8u * s);  // the stage may be refilled once these MMAs have read it
            }
            if (!failed) umma_commit(accum);
        }
    } else {  // ---- epilogue warps
        const int lane_base = (warp & 3) * 32;
        const int row = m0 + lane_base + lane;
        if (nkb > 0 && !mbar_wait(accum, 0)) {
            atomicExch(p.err, DEV_ERR_PF_ACCUM);
            failed = true;
        }
        if (!failed) {
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                float v[32];
                if (nkb > 0) {
                    tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c * 32u, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                }
                if (p.qrows != nullptr && n0 + c * 32 < p.N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        v[i] *= *reinterpret_cast<const float*>(p.qrows + (size_t)(n0 + c * 32 + i) * p.qstride + p.qscale_off);
                }
                if (row < p.M && n0 + c * 32 < p.N) epi(z, row, n0 + c * 32, v);
            }
        }
    }
    if (__any_sync(0xffffffffu, failed)) {  // give copies that may still be in flight time to land before the CTA leaves
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, BN);
}

// ------------------------------------------------------------------ the GEMM for a handful of rows
// Multi-sample decode has at most 16 activation rows, so the operands swap roles: the weight
// tile [128 features][64] is the M-side operand (every staged byte is useful) and the
// activations are the N side, [NB rows][64] with rows 0-15 the hi parts and rows 16-31 the lo
// parts of the samples (NB = 16 without the lo parts).  D[feature lane][row column] in tensor
// memory; an epilogue thread owns one feature and adds column j + 16 to column j.  One CTA per
// 128 features, nine 20 KB stages: the kernel is a weight stream, bound by HBM.
constexpr int SK_ROWS = 16;  // samples per call at most
template <int NB> struct SkTile {
    static constexpr uint32_t A_BYTES = 128 * PF_BK * 2, B_BYTES = NB * PF_BK * 2, STAGE = A_BYTES + 2048 * ((B_BYTES + 2047) / 2048);
    static constexpr int NST = 5;  // two CTAs per SM: one streams while its neighbour starts up or drains
    static constexpr size_t SMEM = (size_t)NST * STAGE + 1024 + 256;
};

struct SkEpiPartial {  // this K slice's partial sums: part[slice][s][f] = y[s]
    float* part;
    int ld;
    __device__ void operator()(int f, bool valid, const float (&y)[SK_ROWS], int ns) const {
        if (!valid) return;
        float* p = part + (size_t)blockIdx.y * SK_ROWS * ld;
#pragma unroll
        for (int s = 0; s < SK_ROWS; ++s)
            if (s < ns) p[(size_t)s * ld + f] = y[s];
    }
};
struct SkEpiStore {  // out[s][f] = y[s]
    float* out;
    int ld;
    __device__ void operator()(int f, bool valid, const float (&y)[SK_ROWS], int ns) const {
        if (!valid) return;
#pragma unroll
        for (int s = 0; s < SK_ROWS; ++s)
            if (s < ns) out[(size_t)s * ld + f] = y[s];
    }
};
template <typename T16> struct SkEpiGate {  // features (2j, 2j+1) = (w1, w3) column j sit in neighbouring lanes
    T16* gate;
    T16* gate_lo;
    int ld, act;
    __device__ void operator()(int f, bool valid, const float (&y)[SK_ROWS], int ns) const {
#pragma unroll
        for (int s = 0; s < SK_ROWS; ++s) {
            if (s >= ns) break;  // uniform across the warp
            const float y3 = __shfl_xor_sync(0xffffffffu, y[s], 1);
            if (valid && !(f & 1)) {
                const float y1 = y[s];
                float a;
                if (act == 1) {
                    const float l = fmaxf(y1, 0.5f * y1);
                    a = l * l;
                } else {
                    a = y1 / (1.0f + expf(-y1));
                }
                pf_store(gate, gate_lo, (size_t)s * ld + (f >> 1), a * y3);
            }
        }
    }
};
template <typename T16> struct SkEpiQKV {  // RoPE pairs sit in neighbouring lanes; q fp32 per sample, k / v into the sample's page
    float* q;
    T16* kv_pool;
    const int* page_table;  // [samples][pages_per_seq]
    const float2* rope;
    const DevState* st;  // the samples' common position (read on the device: one captured graph serves every step)
    int Q, KV, hd, kv_heads, page_tokens, pages_per_seq;
    __device__ void operator()(int f, bool valid, const float (&y)[SK_ROWS], int ns) const {
        const int pos = __ldcg(&st->pos);
        const bool roped = f < Q + KV;
        float2 cs = make_float2(1.0f, 0.0f);
        if (valid && roped) cs = rope[(size_t)pos * (hd >> 1) + ((f % hd) >> 1)];
        const int kv01 = f < Q + KV ? 0 : 1;
        const int ck = f - Q - kv01 * KV, head = ck / hd, d = ck % hd;
#pragma unroll
        for (int s = 0; s < SK_ROWS; ++s) {
            if (s >= ns) break;  // uniform across the warp
            const float p = __shfl_xor_sync(0xffffffffu, y[s], 1);
            if (!valid) continue;
            float r = y[s];
            if (roped) r = (f & 1) ? y[s] * cs.x + p * cs.y : y[s] * cs.x - p * cs.y;
            if (f < Q) {
                q[(size_t)s * Q + f] = r;
            } else {
                const int page = page_table[(size_t)s * pages_per_seq + pos / page_tokens], off = pos % page_tokens;
                kv_pool[((((size_t)page * 2 + kv01) * kv_heads + head) * page_tokens + off) * hd + d] = pf_cast<T16>(r);
            }
        }
    }
};

template <int NB, class Epi>
__global__ void __launch_bounds__(PF_THREADS, 2)
pf_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x, int N, int K, int ns, uint32_t idesc, int* err, Epi epi) {
    using TL = SkTile<NB>;
    constexpr int NST = TL::NST;
    extern __shared__ unsigned char pf_raw[];
    const int n0 = blockIdx.x * 128;
    // blockIdx.y: which slice of K this CTA multiplies (a matrix with few rows is cut along K so that
    // enough CTAs stream it; the epilogue then stores a partial sum for the consumer to add up)
    const int nkb_all = (K + PF_BK - 1) / PF_BK, per = (nkb_all + (int)gridDim.y - 1) / (int)gridDim.y;
    const int kb_first = blockIdx.y * per, nkb = max(0, min(nkb_all, kb_first + per) - kb_first);
    const uint32_t tiles = (smem_addr(pf_raw) + 1023u) & ~1023u;
    const uint32_t bars = tiles + NST * TL::STAGE;
    const uint32_t full0 = bars, empty0 = bars + 8u * NST, accum = bars + 16u * NST, slot = accum + 8u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(full0 + 8u * s, 1);
            mbar_init(empty0 + 8u * s, 1);
        }
        mbar_init(accum, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(slot, 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(slot));
    bool failed = false;
    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % NST;
                if (kb >= NST && !mbar_wait(empty0 + 8u * s, ((kb / NST) - 1) & 1)) {
                    atomicExch(err, DEV_ERR_PF_EMPTY);
                    failed = true;
                    break;
                }
                const uint32_t a_dst = tiles + s * TL::STAGE;
                mbar_arrive_expect_tx(full0 + 8u * s, TL::A_BYTES + TL::B_BYTES);
                tma_load_2d(a_dst, &tma_w, (kb_first + kb) * PF_BK, n0, full0 + 8u * s);
                // Under programmatic dependent launch the first ring of weight tiles is requested before the
                // previous kernel has finished; the activations it produces are requested only after the wait.
                if (kb == min(NST, nkb) - 1) {
                    pdl_wait();
                    pdl_launch_dependents();
                    for (int k2 = 0; k2 <= kb; ++k2)
                        tma_load_2d(tiles + (k2 % NST) * TL::STAGE + TL::A_BYTES, &tma_x, (kb_first + k2) * PF_BK, 0, full0 + 8u * (k2 % NST));
                } else if (kb >= NST) {
                    tma_load_2d(a_dst + TL::A_BYTES, &tma_x, (kb_first + kb) * PF_BK, 0, full0 + 8u * s);
                }
            }
            if (nkb == 0) { pdl_wait(); pdl_launch_dependents(); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % NST;
                if (!mbar_wait(full0 + 8u * s, (kb / NST) & 1)) {
                    atomicExch(err, DEV_ERR_PF_FULL);
                    failed = true;
                    break;
                }
                tc_fence_after();
                const uint64_t adesc = umma_desc(tiles + s * TL::STAGE), bdesc = umma_desc(tiles + s * TL::STAGE + TL::A_BYTES);
#pragma unroll
                for (int k = 0; k < PF_BK / 16; ++k) umma_f16(tmem_base, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0);
                umma_commit(empty0 + 8u * s);
            }
            if (!failed) umma_commit(accum);
        }
    } else {
        const int lane_base = (warp & 3) * 32;
        const int f = n0 + lane_base + lane;
        pdl_wait();  // nothing is written before the previous kernel is complete
        if (nkb > 0 && !mbar_wait(accum, 0)) {
            atomicExch(err, DEV_ERR_PF_ACCUM);
            failed = true;
        }
        if (!failed) {
            tc_fence_after();
            float v[32];
            if (nkb > 0) {
                tmem_ld32(tmem_base + ((uint32_t)lane_base << 16), v);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.0f;
            }
            float y[SK_ROWS];
#pragma unroll
            for (int j = 0; j < SK_ROWS; ++j) y[j] = NB == 32 ? v[j] + v[j + 16] : v[j];
            epi(f, f < N, y, ns);
        }
    }
    if (__any_sync(0xffffffffu, failed)) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 32);
}

// FP8 rows (Wfmt<Fp8Row>: K e4m3 bytes, then the row scale) to a [N][K] 16-bit matrix of the unscaled
// e4m3 values, which both 16-bit types hold exactly; the scale is applied to the GEMM's output column.
template <typename T16>
__global__ void __launch_bounds__(256) pf_widen_fp8_kernel(const unsigned char* __restrict__ rows, uint32_t stride, T16* __restrict__ out, int N, int K) {
    const size_t total = (size_t)N * (K / 4);
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (size_t)gridDim.x * blockDim.x) {
        const size_t r = j / (K / 4);
        const int c = (int)(j % (K / 4)) * 4;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(rows + r * stride + c);
        const __half2 h01(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3));
        const __half2 h23(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3));
        const float2 a = __half22float2(h01), b = __half22float2(h23);
        T16* o = out + r * K + c;
        o[0] = pf_cast<T16>(a.x); o[1] = pf_cast<T16>(a.y); o[2] = pf_cast<T16>(b.x); o[3] = pf_cast<T16>(b.y);
    }
}

// ------------------------------------------------------------------ small batched kernels
// token rows of the embedding table into the fp32 residual stream (cpu/embedding.rs:8-16)
template <typename WT>
__global__ void pf_embed_kernel(const WT* __restrict__ embed, const uint32_t* __restrict__ ids, float* __restrict__ x, int D) {
    const WT* row = embed + (size_t)ids[blockIdx.x] * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)blockIdx.x * D + i] = Elem<WT>::to_f32(row[i]);
}

// the same with one token per sample, taken from the samples' device states
template <typename WT>
__global__ void pf_embed_samples_kernel(const WT* __restrict__ embed, DevState* __restrict__ st, float* __restrict__ x, int D, int vocab) {
    const WT* row = embed + (size_t)checked_token(st[blockIdx.x].token, vocab, &st[blockIdx.x].error) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)blockIdx.x * D + i] = Elem<WT>::to_f32(row[i]);
}

// fp32 values as a 16-bit hi (+ lo) GEMM operand
template <typename T16>
__global__ void pf_split_kernel(const float* __restrict__ in, T16* __restrict__ hi, T16* __restrict__ lo, size_t n) {
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) pf_store(hi, lo, i, in[i]);
}

// x * rsqrt(mean(x^2) + eps) * gamma per row (cpu/rmsnorm.rs:149-183), written as 16-bit GEMM input
template <typename T16>
__global__ void __launch_bounds__(256) pf_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma, T16* __restrict__ out,
                                                         T16* __restrict__ out_lo, int D) {
    __shared__ float red[32];
    pdl_launch_dependents();  // a following weight-streaming kernel may start fetching; it waits before it reads `out`
    const float* row = x + (size_t)blockIdx.x * D;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) ss += row[i] * row[i];
    const float inv = 1.0f / sqrtf(block_sum(ss, red) * (1.0f / (float)D) + RMS_EPS);
    for (int i = threadIdx.x; i < D; i += blockDim.x) pf_store(out, out_lo, (size_t)blockIdx.x * D + i, row[i] * inv * gamma[i]);
}

// The same after folding in a linear that was cut along K: x += alpha * (sum of the slices' partial
// sums, in slice order), written back, then normalised.  One CTA of up to 1024 threads per row.
template <typename T16>
__global__ void __launch_bounds__(1024) pf_reduce_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ part, int nslices, float alpha,
                                                                 const float* __restrict__ gamma, T16* __restrict__ out, T16* __restrict__ out_lo, int D) {
    __shared__ float red[32];
    pdl_launch_dependents();
    float* row = x + (size_t)blockIdx.x * D;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < nslices; ++k) acc += part[((size_t)k * SK_ROWS + blockIdx.x) * D + i];
        const float v = row[i] + alpha * acc;
        row[i] = v;
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) * (1.0f / (float)D) + RMS_EPS);
    for (int i = threadIdx.x; i < D; i += blockDim.x) pf_store(out, out_lo, (size_t)blockIdx.x * D + i, row[i] * inv * gamma[i]);
}

// V of the first ntok cached positions, transposed per kv head: vt[head][d][tok] (ld = ntok rounded up)
template <typename T16>
__global__ void __launch_bounds__(256) pf_transpose_v_kernel(const T16* __restrict__ kv_pool, const int* __restrict__ page_table, T16* __restrict__ vt,
                                                             int ntok, int ld, int kv_heads, int hd, int page_tokens) {
    __shared__ T16 tile[64][130];
    const int t0 = blockIdx.x * 64, head = blockIdx.y;
    for (int j = threadIdx.x; j < 64 * hd; j += blockDim.x) {
        const int t = j / hd, d = j % hd, tok = t0 + t;
        T16 val = pf_cast<T16>(0.0f);
        if (tok < ntok) {
            const int page = page_table[tok / page_tokens], off = tok % page_tokens;
            val = kv_pool[((((size_t)page * 2 + 1) * kv_heads + head) * page_tokens + off) * hd + d];
        }
        tile[t][d] = val;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < 64 * hd; j += blockDim.x) {
        const int d = j / 64, t = j % 64;
        if (t0 + t < ld) vt[((size_t)head * hd + d) * ld + t0 + t] = tile[t][d];
    }
}

// Causal softmax of one query row of one head: p = exp(s * scale - max) / sum over keys
// 0 .. pos0 + row (sdpa_fwd.rs:36-46, :325-354), written as 16-bit; the rest of the row up
// to where the P V product stops reading (the end of the row's 128-row tile) is zeroed.
template <typename T16>
__global__ void __launch_bounds__(256) pf_softmax_kernel(const float* __restrict__ s, T16* __restrict__ pmat, T16* __restrict__ pmat_lo, size_t plane,
                                                         int ld, int pos0, float scale) {
    __shared__ float red[32];
    const int row = blockIdx.x, z = blockIdx.y;
    const float* srow = s + (size_t)z * plane + (size_t)row * ld;
    const size_t prow = (size_t)z * plane + (size_t)row * ld;
    const int valid = pos0 + row + 1;
    const int upto = min(ld, pos0 + (row / PF_BM + 1) * PF_BM);
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < valid; i += blockDim.x) mx = fmaxf(mx, srow[i] * scale);
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < valid; i += blockDim.x) sum += expf(srow[i] * scale - mx);
    sum = block_sum(sum, red);
    const float inv = 1.0f / sum;
    for (int i = threadIdx.x; i < upto; i += blockDim.x) pf_store(pmat, pmat_lo, prow + i, i < valid ? expf(srow[i] * scale - mx) * inv : 0.0f);
}

// ---------------------------------------------------------------------- tensor parallel: all-reduce of a [rows, dim] partial product
// After the row-sharded Wo / W2 GEMM every rank holds a partial y_r in one of its two buffers of the link region.
// tp_pf_publish_kernel tells every peer so (a sequence number into the peer's flag row, after a system-scope
// fence); tp_pf_reduce_kernel waits (bounded) until all ranks have published `seq`, then x += alpha * sum_r y_r
// with the ranks' buffers read over NVLink and added in rank order, so every rank keeps a bit-identical residual
// stream.  Two buffers alternate: a rank overwrites a buffer only after it has seen every rank publish the
// all-reduce in between, i.e. after every rank finished reading it.
static __global__ void tp_pf_publish_kernel(TpLink tp, size_t flags_off, int buf, unsigned int seq) {
    __threadfence_system();
    if ((int)threadIdx.x < tp.world)
        st_release_sys(reinterpret_cast<unsigned int*>(tp.peers[threadIdx.x] + flags_off) + buf * tp.world + tp.rank, seq);
}

static __global__ void __launch_bounds__(256)
tp_pf_reduce_kernel(TpLink tp, size_t flags_off, size_t buf_off, int buf, unsigned int seq, float* __restrict__ x, int rows, size_t buf_rows,
                    float alpha, int* err) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < tp.world) {
        const unsigned int* f = reinterpret_cast<const unsigned int*>(tp.peers[tp.rank] + flags_off) + buf * tp.world + threadIdx.x;
        if (!tp_wait_flag(f, seq, tp.st, tp.wait_ns)) { atomicCAS(err, 0, DEV_ERR_TP_WAIT); s_ok = 0; }
    }
    __syncthreads();
    if (!s_ok) return;
    const size_t n4 = (size_t)rows * tp.dim / 4, off = buf_off + (size_t)buf * buf_rows * tp.dim * 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < tp.world; ++r) {  // rank order; L2-only loads: the buffers are rewritten every other all-reduce
            const float4 v = __ldcg(reinterpret_cast<const float4*>(tp.peers[r] + off) + i);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        float4 t = reinterpret_cast<float4*>(x)[i];
        t.x += alpha * a.x; t.y += alpha * a.y; t.z += alpha * a.z; t.w += alpha * a.w;
        reinterpret_cast<float4*>(x)[i] = t;
    }
}

}  // namespace cd
