// One persistent kernel per decoded token.
//
// The multi-kernel path pays a fixed 4-6 us at each of its 5 x nlayers kernel boundaries
// (drain, launch, ring refill) during which HBM idles.  Here one cooperative grid of one
// CTA per SM walks the whole token: its producer thread streams this CTA's share of EVERY
// weight matrix, layer after layer, through one shared-memory ring with 1-D bulk copies and
// never stops at an operator boundary, because weights do not depend on activations.  The
// eight consumer warps run the operators in order and meet the other CTAs at a grid barrier
// wherever the next operator needs the whole activation vector (five times per layer).
// While consumers sit in a barrier the ring keeps filling, so HBM stays busy; afterwards
// they drain shared memory several times faster than HBM can refill it and catch up.
//
// Phases of a layer (same arithmetic and epilogues as the stand-alone kernels):
//   1 RMSNorm + q|k|v GEMV + RoPE + KV append     | barrier
//   2 split-K flash-decode attention (two 128-thread teams per CTA take (head, slice)
//     items; the team that arrives last for a head merges its slices)              | barrier
//   3 Wo GEMV + scaled residual                    | barrier
//   4 RMSNorm + W1|W3 GEMV + gate                  | barrier
//   5 W2 GEMV + scaled residual                    | barrier
// then the final RMSNorm + LM head into the logits buffer; the per-block head reductions
// and samplers run as the small kernels they already are.
//
// Every wait (mbarrier, grid barrier) is bounded: on expiry the CTA records an error in
// DevState::error, stops working and leaves, and so does every other CTA when its own
// wait runs out.
#pragma once
#include "kernels.cuh"

namespace cd {

struct MegaLayer {
    const void *wqkv, *wo, *w13, *w2;
    const float *gamma1, *gamma2;
    void* kv;
};

struct MegaParams {
    const MegaLayer* layers;  // device array [nlayers]
    const void* embed;
    const void* lm_head;
    const float* gamma_final;
    float *x_a, *x_b, *q, *attn, *gate, *logits, *norm_final;
    float *part_acc, *part_ml;
    unsigned int* counters;            // [heads]
    unsigned long long* grid_counter;  // monotonic arrival counter of the grid barrier
    DevState* st;
    const int* page_table;
    const float2* rope;
    int dim, hidden, heads, kv_heads, hd, nlayers, vocab, q_dim, kv_dim, gqa, page_tokens, nsplit, activation;
    float alpha, attn_scale;
    int nstages;
    uint32_t stage_cap;   // bytes per ring stage
    int rows_cap;         // rows a CTA may own in any phase
    int input_embed;      // 1: x = embed[st->token]; 0: x already in x_a
    int want_logits;
    uint32_t lookahead_bytes;   // per CTA distance of the L2 look-ahead (0 = off)
    int npages;                 // page-table entries of the sequence
    unsigned long long* trace;  // optional [2][1 + 10 * nlayers + 1] globaltimer stamps of CTA 0 and the last CTA
};

constexpr int GRID_SPIN_LIMIT = 1 << 22;
// Two groups of eight consumer warps take alternate ring stages: a stage's latency chain
// (shared-memory loads, FMA chain, shuffle reduction) is long, and only with two stages
// in progress do the consumers drain the ring clearly faster than HBM fills it, which is
// what lets them catch up after every barrier.
constexpr int MEGA_GROUPS = 2;
constexpr int MEGA_CONSUMERS = MEGA_GROUPS * GEMV_CONSUMERS;
constexpr int MEGA_THREADS = MEGA_CONSUMERS + 32;
constexpr int MEGA_TEAMS = MEGA_CONSUMERS / 128;

__device__ inline void mega_bar() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ inline void group_bar(int grp) { asm volatile("bar.sync %0, 256;" ::"r"(4 + grp) : "memory"); }
__device__ inline float group_sum(float v, float* red, int grp) {
    const int lane = threadIdx.x & 31, warp = (threadIdx.x & 255) >> 5;
    v = warp_sum(v);
    group_bar(grp);
    if (lane == 0) red[warp] = v;
    group_bar(grp);
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < GEMV_CONSUMERS / 32; ++i) t += red[i];
    return t;
}

struct Ring {
    uint32_t base, full0, empty0, stage_cap;
    int nstages;
    int g;  // stages used so far (producer and consumers count the same sequence)
};

// rows [r0, r1) of an [N, K] matrix owned by this CTA
__device__ inline void cta_rows(int N, int unit, int& r0, int& r1) {
    const int nunits = N / unit;
    r0 = (int)((long long)blockIdx.x * nunits / gridDim.x) * unit;
    r1 = (int)((long long)(blockIdx.x + 1) * nunits / gridDim.x) * unit;
}

// ---- L2 look-ahead: a second cursor over this CTA's weight sequence (q|k|v, Wo, W1|W3, W2 of
// each layer, wrapping to layer 0 for the next token) that stays a fixed distance in front of
// the bulk copies and asks L2 for those bytes.  The ring alone holds ~3 us of HBM traffic;
// attention and the grid barriers keep consumers away from it for longer, and with the
// look-ahead HBM keeps streaming into L2 meanwhile, from where the ring refills faster.
struct LookAhead {
    const MegaParams* p;
    uint32_t rb_d, rb_h;
    int l, seg;
    size_t off;
    __device__ inline void segment(const char*& base, size_t& bytes) const {
        const MegaLayer& L = p->layers[l];
        int r0, r1;
        uint32_t rb = rb_d;
        const void* w;
        if (seg == 0) { cta_rows(p->q_dim + 2 * p->kv_dim, 2, r0, r1); w = L.wqkv; }
        else if (seg == 1) { cta_rows(p->dim, 1, r0, r1); w = L.wo; }
        else if (seg == 2) { cta_rows(2 * p->hidden, 2, r0, r1); w = L.w13; }
        else { cta_rows(p->dim, 1, r0, r1); w = L.w2; rb = rb_h; }
        base = reinterpret_cast<const char*>(w) + (size_t)r0 * rb;
        bytes = (size_t)(r1 - r0) * rb;
    }
    __device__ inline void advance(size_t n) {
        int empty = 0;  // a CTA that owns no rows anywhere must not loop for ever
        while (n > 0 && empty <= 4 * p->nlayers) {
            const char* base;
            size_t bytes;
            segment(base, bytes);
            const size_t take = min(n, bytes - off);
            empty = take == 0 ? empty + 1 : 0;
            for (size_t o = 0; o < take; o += 32768) bulk_prefetch_l2(base + off + o, (uint32_t)min((size_t)32768, take - o));
            off += take;
            n -= take;
            if (off >= bytes) {
                off = 0;
                if (++seg == 4) { seg = 0; if (++l == p->nlayers) l = 0; }
            }
        }
    }
};

// ---- producer side: queue one matrix's rows for this CTA
template <int R>
__device__ inline bool produce_segment(Ring& ring, const void* W, uint32_t row_bytes, int N, int unit, uint64_t policy, int* err,
                                       LookAhead* ahead) {
    int r0, r1;
    cta_rows(N, unit, r0, r1);
    const char* Wb = reinterpret_cast<const char*>(W) + (size_t)r0 * row_bytes;
    const int ngroups = (r1 - r0 + R - 1) / R;
    for (int g = 0; g < ngroups; ++g, ++ring.g) {
        const int s = ring.g % ring.nstages;
        const uint32_t full = ring.full0 + 8u * s, empty = ring.empty0 + 8u * s;
        if (ring.g >= ring.nstages && !mbar_wait(empty, ((ring.g / ring.nstages) - 1) & 1)) {
            atomicExch(err, DEV_ERR_EMPTY_WAIT);
            return false;
        }
        const int rows = min(R, (r1 - r0) - g * R);
        const uint32_t bytes = (uint32_t)rows * row_bytes;
        mbar_arrive_expect_tx(full, bytes);
        bulk_g2s_stream(ring.base + (uint32_t)s * ring.stage_cap, Wb + (size_t)g * R * row_bytes, bytes, full, policy);
        if (ahead != nullptr) ahead->advance(bytes);
    }
    return true;
}

// ---- consumer side: one GEMV phase.  x comes from `x` (fp32, L2-only loads) or, when
// `embed_row` is given, from a row of the embedding table in storage form.
template <typename WT, int NITER, int R, int UNIT, bool NORM, class Epi>
__device__ inline bool consume_gemv(Ring& ring, const float* x, const WT* embed_row, float* x_copy, const float* gamma,
                                    float* norm_out, int N, int K, float* partial, float* red, int* err, int* abort_flag,
                                    const Epi& epi) {
    constexpr int EPC = Elem<WT>::EPC;
    constexpr int NW = GEMV_CONSUMERS / 32;
    const int grp = threadIdx.x >> 8, tid = threadIdx.x & 255, lane = tid & 31, warp = tid >> 5;
    const int nchunks = K / EPC;
    const uint32_t row_bytes = (uint32_t)K * sizeof(WT);
    int r0, r1;
    cta_rows(N, UNIT, r0, r1);
    const int ngroups = (r1 - r0 + R - 1) / R;
    red += grp * 32;

    float xr[NITER][EPC];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NITER; ++i) {
        const int c = tid + i * GEMV_CONSUMERS;
        if (embed_row != nullptr) {
            if (c < nchunks) {
                const uint4 w = ldg_stream(reinterpret_cast<const char*>(embed_row) + (size_t)c * 16);
                Elem<WT>::unpack(w, xr[i]);
                if (x_copy != nullptr && blockIdx.x == 0 && grp == 0) {
#pragma unroll
                    for (int e = 0; e < EPC; e += 4)
                        *reinterpret_cast<float4*>(x_copy + (size_t)c * EPC + e) = make_float4(xr[i][e], xr[i][e + 1], xr[i][e + 2], xr[i][e + 3]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < EPC; ++e) xr[i][e] = 0.0f;
            }
#pragma unroll
            for (int e = 0; e < EPC; ++e) ss += xr[i][e] * xr[i][e];
        } else {
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < nchunks) v = __ldcg(reinterpret_cast<const float4*>(x + (size_t)c * EPC + e));
                xr[i][e] = v.x; xr[i][e + 1] = v.y; xr[i][e + 2] = v.z; xr[i][e + 3] = v.w;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
    }
    if (NORM) {
        const float tot = group_sum(ss, red, grp);
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
                    if (norm_out != nullptr && blockIdx.x == 0 && grp == 0)
                        *reinterpret_cast<float4*>(norm_out + (size_t)c * EPC + e) =
                            make_float4(xr[i][e], xr[i][e + 1], xr[i][e + 2], xr[i][e + 3]);
                }
            }
        }
    }

    // Ring slots are owned by groups for the whole kernel: group = (global stage number) & 1,
    // and the ring has an even number of slots, so the successive uses of one slot are all
    // consumed, in order, by the same group.  (A parity wait can only tell adjacent phases of
    // an mbarrier apart; a group that skipped another group's use of a slot could mistake
    // an old phase for the one it wants.)
    for (int g = (grp - ring.g) & 1; g < ngroups; g += MEGA_GROUPS) {
        const int rg = ring.g + g;
        const int s = rg % ring.nstages;
        if (!mbar_wait(ring.full0 + 8u * s, (rg / ring.nstages) & 1)) {
            atomicExch(err, DEV_ERR_FULL_WAIT);
            *abort_flag = 1;  // every consumer still meets at the barrier below, then all leave together
            break;
        }
        const uint32_t base = ring.base + (uint32_t)s * ring.stage_cap;
        uint4 w[R][NITER];
#pragma unroll
        for (int j = 0; j < R; ++j)
#pragma unroll
            for (int i = 0; i < NITER; ++i) {
                const int c = tid + i * GEMV_CONSUMERS;
                w[j][i] = (c < nchunks) ? lds128(base + (uint32_t)j * row_bytes + (uint32_t)c * 16u) : make_uint4(0, 0, 0, 0);
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(ring.empty0 + 8u * s);
        float acc[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < NITER; ++i) {
                float f[EPC];
                Elem<WT>::unpack(w[j][i], f);
#pragma unroll
                for (int e = 0; e < EPC; ++e) a = fmaf(f[e], xr[i][e], a);
            }
            acc[j] = a;
        }
        int rr;
        const float tot = warp_reduce_rows<R>(acc, lane, rr);
        const int row = g * R + rr;
        if ((lane & (32 / R - 1)) == 0 && row < r1 - r0) partial[row * NW + warp] = tot;
    }
    ring.g += ngroups;
    mega_bar();
    if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return false;
    const int u0 = r0 / UNIT, nu = (r1 - r0) / UNIT;
    for (int u = threadIdx.x; u < nu; u += MEGA_CONSUMERS) {
        float y[UNIT];
#pragma unroll
        for (int k = 0; k < UNIT; ++k) {
            float sacc = 0.0f;
#pragma unroll
            for (int wi = 0; wi < NW; ++wi) sacc += partial[(u * UNIT + k) * NW + wi];
            y[k] = sacc;
        }
        epi(u0 + u, y);
    }
    return true;
}

// ---- grid barrier for the consumer threads of all CTAs (arrival k of this launch)
__device__ inline bool grid_barrier(unsigned long long* counter, unsigned long long target, int* err, int* abort_flag) {
    mega_bar();  // every consumer's global writes of the phase are issued
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1ull);
        bool ok = false;
        for (int i = 0; i < GRID_SPIN_LIMIT; ++i) {
            if (*reinterpret_cast<volatile unsigned long long*>(counter) >= target) { ok = true; break; }
            __nanosleep(40);
        }
        if (!ok) {
            atomicExch(err, 3);
            *abort_flag = 1;
        }
        __threadfence();
    }
    mega_bar();
    return *reinterpret_cast<volatile int*>(abort_flag) == 0;
}

__device__ inline void team_bar(int team) { asm volatile("bar.sync %0, 128;" ::"r"(8 + team) : "memory"); }

// ---- one (head, slice) item of the attention phase, run by a 128-thread team
template <typename KT, int HD>
__device__ inline void attention_item(const MegaParams& p, const KT* kv_pool, int h, int s, int attn_len, int per, int nactive,
                                      int team, int tt, float* accs, float* gm, float* gl, int* flag, const int* pt) {
    constexpr int EPC = Elem<KT>::EPC;
    constexpr int LPT = HD / EPC;
    constexpr int NG = 128 / LPT;
    constexpr int UNR = 8;
    constexpr float NEG = -3.402823466e+38f;
    const int g = tt / LPT, l = tt % LPT;
    const int kvh = h / p.gqa;
    const int nsplit = p.nsplit;
    const size_t head_stride = (size_t)p.page_tokens * HD;
    const size_t page_stride = (size_t)2 * p.kv_heads * head_stride;
    const int t0 = s * per, t1 = min(attn_len, t0 + per);

    float qf[EPC];
#pragma unroll
    for (int e = 0; e < EPC; e += 4) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.q + (size_t)h * HD + l * EPC + e));
        qf[e] = v.x; qf[e + 1] = v.y; qf[e + 2] = v.z; qf[e + 3] = v.w;
    }
    float m = NEG, lsum = 0.0f;
    float acc[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) acc[e] = 0.0f;
    for (int tb = t0; tb < t1; tb += NG * UNR) {
        uint4 kw[UNR], vw[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int t = tb + g + u * NG;
            if (t < t1) {
                const int page = pt[t / p.page_tokens], off = t % p.page_tokens;
                const KT* kp = kv_pool + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)off * HD + l * EPC;
                kw[u] = ldg_stream_coherent(kp);
                vw[u] = ldg_stream_coherent(kp + (size_t)p.kv_heads * head_stride);
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
            sc[u] = (tb + g + u * NG < t1) ? d * p.attn_scale : NEG;
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
                    const float pr = expf(sc[u] - mnew);
                    lsum += pr;
                    float f[EPC];
                    Elem<KT>::unpack(vw[u], f);
#pragma unroll
                    for (int e = 0; e < EPC; ++e) acc[e] = fmaf(pr, f[e], acc[e]);
                }
            }
            m = mnew;
        }
    }
#pragma unroll
    for (int e = 0; e < EPC; ++e) accs[g * HD + l * EPC + e] = acc[e];
    if (l == 0) { gm[g] = m; gl[g] = lsum; }
    team_bar(team);
    const size_t slot = (size_t)h * nsplit + s;
    if (tt < HD) {
        float M = NEG;
#pragma unroll
        for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, gm[gg]);
        float L = 0.0f, a = 0.0f;
#pragma unroll
        for (int gg = 0; gg < NG; ++gg) {
            if (gl[gg] > 0.0f) {
                const float wgt = expf(gm[gg] - M);
                L += gl[gg] * wgt;
                a += accs[gg * HD + tt] * wgt;
            }
        }
        p.part_acc[slot * HD + tt] = a;
        if (tt == 0) {
            p.part_ml[slot * 2 + 0] = M;
            p.part_ml[slot * 2 + 1] = L;
        }
    }
    __threadfence();
    team_bar(team);
    if (tt == 0) {
        const unsigned prev = atomicAdd(&p.counters[h], 1u);
        *flag = (prev == (unsigned)nactive - 1u);
    }
    team_bar(team);
    if (*flag) {  // last team for this head: merge the nactive slices (slices >= nactive are empty)
        __threadfence();
        float* wsl = accs;
        float* lsl = accs + 64;
        float ms = NEG, ls = 0.0f;
        if (tt < nactive) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((size_t)h * nsplit + tt) * 2));
            ms = ml.x;
            ls = ml.y;
        }
        float M = ls > 0.0f ? ms : NEG;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        if ((tt & 31) == 0 && tt < 64) gl[tt >> 5] = M;
        team_bar(team);
        M = fmaxf(gl[0], gl[1]);
        if (tt < nactive) {
            const float wgt = ls > 0.0f ? expf(ms - M) : 0.0f;
            wsl[tt] = wgt;
            lsl[tt] = ls * wgt;
        }
        team_bar(team);
        if (tt < HD) {
            float L = 0.0f, o = 0.0f;
            const float* pa = p.part_acc + (size_t)h * nsplit * HD + tt;
#pragma unroll 8
            for (int ss2 = 0; ss2 < nactive; ++ss2) {
                L += lsl[ss2];
                o += __ldcg(pa + (size_t)ss2 * HD) * wsl[ss2];
            }
            p.attn[(size_t)h * HD + tt] = L > 0.0f ? o / L : 0.0f;
        }
        if (tt == 0) p.counters[h] = 0u;
    }
    team_bar(team);  // accs / gm / gl are free for the team's next item
}

template <typename KT>
__device__ inline void attention_phase(const MegaParams& p, const void* kv, float* attn_smem, int* flags, const int* pt, int attn_len) {
    const int tid = threadIdx.x, team = tid >> 7, tt = tid & 127;  // MEGA_TEAMS teams of 128 threads
    // one (head, slice) item per team where possible: slices need not be whole pages
    const int teams = gridDim.x * MEGA_TEAMS;
    const int max_slices = max(1, min(p.nsplit, teams / p.heads));
    const int want = min(max_slices, (attn_len + 15) / 16);
    const int per = (attn_len + want - 1) / want;
    const int nactive = (attn_len + per - 1) / per;  // slices that hold at least one position
    const int nitems = p.heads * nactive;
    float* accs = attn_smem + team * (128 * 8 + 64);
    float* gm = accs + 128 * 8;
    float* gl = gm + 32;
    for (int item = blockIdx.x * MEGA_TEAMS + team; item < nitems; item += teams) {
        const int h = item / nactive, s = item % nactive;
        if (p.hd == 128) attention_item<KT, 128>(p, reinterpret_cast<const KT*>(kv), h, s, attn_len, per, nactive, team, tt, accs, gm, gl, flags + team, pt);
        else attention_item<KT, 64>(p, reinterpret_cast<const KT*>(kv), h, s, attn_len, per, nactive, team, tt, accs, gm, gl, flags + team, pt);
    }
}

template <typename WT, typename KT, int ND, int RD, int NH, int RH>
__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_mega_kernel(const MegaParams p) {
    constexpr int NW = GEMV_CONSUMERS / 32;
    extern __shared__ __align__(128) unsigned char smraw[];
    float* partial = reinterpret_cast<float*>(smraw + (size_t)p.nstages * p.stage_cap);  // [rows_cap][NW]
    float* red = partial + (size_t)p.rows_cap * NW;                                       // 32 per group
    float* attn_smem = red + 32 * MEGA_GROUPS;                                            // per team 1024 + 64
    int* flags = reinterpret_cast<int*>(attn_smem + MEGA_TEAMS * (128 * 8 + 64));         // [0..3] team flags, [4] abort
    int* pt_s = flags + 8;                                                                // page table copy
    uint64_t* bars = reinterpret_cast<uint64_t*>(pt_s + ((p.npages + 3) & ~3));
    Ring ring;
    ring.base = smem_addr(smraw);
    ring.full0 = smem_addr(bars);
    ring.empty0 = ring.full0 + 8u * p.nstages;
    ring.stage_cap = p.stage_cap;
    ring.nstages = p.nstages;
    ring.g = 0;
    int* err = &p.st->error;
    const int tid = threadIdx.x, warp = tid >> 5;
    const uint32_t rb_d = (uint32_t)p.dim * sizeof(WT), rb_h = (uint32_t)p.hidden * sizeof(WT);

    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(ring.full0 + 8u * s, 1);
            mbar_init(ring.empty0 + 8u * s, NW);
        }
        mbar_fence_init();
        for (int i = 0; i < 8; ++i) flags[i] = 0;
    }
    for (int i = tid; i < p.npages; i += MEGA_THREADS) pt_s[i] = p.page_table[i];
    __syncthreads();

    if (warp == MEGA_CONSUMERS / 32) {  // ---- producer: the whole token's weights for this CTA, in operator order
        if ((tid & 31) == 0) {
            const uint64_t policy = l2_evict_first_policy();
            LookAhead la{&p, rb_d, rb_h, 0, 0, 0};
            LookAhead* ahead = p.lookahead_bytes > 0 ? &la : nullptr;
            // the previous token's kernel already asked for the first lookahead_bytes: start behind them
            if (ahead) {
                size_t skip = p.lookahead_bytes;
                for (int guard = 0; skip > 0 && guard < 8 * p.nlayers + 8; ++guard) {
                    const char* base; size_t bytes;
                    la.segment(base, bytes);
                    const size_t take = min(skip, bytes - la.off);
                    la.off += take; skip -= take;
                    if (la.off >= bytes) { la.off = 0; if (++la.seg == 4) { la.seg = 0; if (++la.l == p.nlayers) la.l = 0; } }
                }
            }
            bool ok = true;
            for (int l = 0; l < p.nlayers && ok; ++l) {
                const MegaLayer& L = p.layers[l];
                ok = produce_segment<RD>(ring, L.wqkv, rb_d, p.q_dim + 2 * p.kv_dim, 2, policy, err, ahead) &&
                     produce_segment<RD>(ring, L.wo, rb_d, p.dim, 1, policy, err, ahead) &&
                     produce_segment<RD>(ring, L.w13, rb_d, 2 * p.hidden, 2, policy, err, ahead) &&
                     produce_segment<RH>(ring, L.w2, rb_h, p.dim, 1, policy, err, ahead);
            }
            if (ok && p.want_logits) produce_segment<RD>(ring, p.lm_head, rb_d, p.vocab, 1, policy, err, nullptr);
        }
        return;
    }

    // ---- consumers
    const unsigned long long nbar = 5ull * (unsigned long long)p.nlayers;
    const unsigned long long epoch = __ldcg(&p.st->epoch);  // launches completed so far; stable until the last barrier
    unsigned long long arrivals = epoch * nbar;  // barriers completed by earlier launches
    auto barrier = [&]() {
        arrivals += 1;
        return grid_barrier(p.grid_counter, arrivals * gridDim.x, err, flags + 4);
    };
    unsigned long long* tr = nullptr;
    if (p.trace != nullptr && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
        tr = p.trace + (blockIdx.x == 0 ? 0 : 1) * (size_t)(10 * p.nlayers + 2);
    auto stamp = [&]() {
        if (tr != nullptr) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            *tr++ = t;
        }
    };
    stamp();
    const int attn_len = __ldcg(&p.st->pos) + 1;
    const WT* embed_row = nullptr;
    if (p.input_embed) embed_row = reinterpret_cast<const WT*>(p.embed) + (size_t)__ldcg(&p.st->token) * p.dim;
    bool ok = true;
    for (int l = 0; l < p.nlayers && ok; ++l) {
        const MegaLayer L = p.layers[l];
        EpiQKV<KT> eq{p.q, reinterpret_cast<KT*>(L.kv), p.page_table, p.st, p.rope, p.q_dim, p.kv_dim, p.hd, p.kv_heads, p.page_tokens};
        ok = consume_gemv<WT, ND, RD, 2, true>(ring, p.x_a, l == 0 ? embed_row : nullptr, p.x_a, L.gamma1, nullptr,
                                               p.q_dim + 2 * p.kv_dim, p.dim, partial, red, err, flags + 4, eq);
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        attention_phase<KT>(p, L.kv, attn_smem, flags, pt_s, attn_len);
        stamp();
        if (!(ok = barrier())) break;
        stamp();
        ok = consume_gemv<WT, ND, RD, 1, false>(ring, p.attn, nullptr, nullptr, nullptr, nullptr, p.dim, p.q_dim, partial, red, err,
                                                flags + 4, EpiResidual{p.x_a, p.x_b, p.alpha});
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        ok = consume_gemv<WT, ND, RD, 2, true>(ring, p.x_b, nullptr, nullptr, L.gamma2, nullptr, 2 * p.hidden, p.dim, partial, red, err,
                                               flags + 4, EpiGate{p.gate, p.activation});
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        ok = consume_gemv<WT, NH, RH, 1, false>(ring, p.gate, nullptr, nullptr, nullptr, nullptr, p.dim, p.hidden, partial, red, err,
                                                flags + 4, EpiResidual{p.x_b, p.x_a, p.alpha});
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
    }
    if (ok && p.want_logits)
        ok = consume_gemv<WT, ND, RD, 1, true>(ring, p.x_a, nullptr, nullptr, p.gamma_final, p.norm_final, p.vocab, p.dim, partial, red,
                                               err, flags + 4, EpiStore{p.logits});
    stamp();
    if (ok && tid == 0 && blockIdx.x == 0) p.st->epoch = epoch + 1;  // every CTA read it before its first barrier
    if (!ok) {
        // leave only once copies that may still be in flight towards this CTA have landed (bounded)
        for (int s = 0; s < p.nstages; ++s) mbar_wait(ring.full0 + 8u * s, (ring.g / ring.nstages) & 1);
    }
}

}  // namespace cd
