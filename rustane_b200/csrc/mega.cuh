// One persistent kernel per decoded token.
//
// The multi-kernel path pays a fixed 4-6 us at each of its 5 x nlayers kernel boundaries
// (drain, launch, ring refill) during which HBM idles.  Here one cooperative grid of one
// CTA per SM walks the whole token.  Its producer thread streams, layer after layer and
// through one shared-memory ring of 1-D bulk copies, everything this CTA will read from
// HBM in the order it will need it: its rows of the q|k|v matrix, the K/V tiles of the
// cached positions its attention work covers, its rows of Wo, W1|W3 and W2 - and never
// stops at an operator boundary, because none of that depends on this token's activations
// (the one K/V row that does, the current position's, is read straight from global memory
// by the consumers instead).  Sixteen consumer warps run the operators in order and meet
// the other CTAs at a grid barrier wherever the next operator needs a whole activation
// vector (five times per layer).  While consumers sit in a barrier the ring keeps filling,
// so HBM stays busy; afterwards they drain shared memory several times faster than HBM can
// refill it and catch up.
//
// Phases of a layer (same arithmetic and epilogues as the stand-alone kernels):
//   1 RMSNorm + q|k|v GEMV + RoPE + KV append                                        | barrier
//   2 attention: every kv head belongs to a few CTAs, each of which takes a contiguous
//     run of tiles of cached positions out of the ring (already resident: they were
//     requested while phase 1 ran), keeps a running softmax per team of four warps,
//     merges its teams in shared memory and stores ONE partial (max, sum, weighted V)
//     per q head                                                                      | barrier
//   3 every CTA merges the few partials of every head (fixed order: deterministic, no
//     atomics, nobody waits for a "last arriver"), then Wo GEMV + scaled residual       | barrier
//   4 RMSNorm + W1|W3 GEMV + gate                                                     | barrier
//   5 W2 GEMV + scaled residual                                                       | barrier
// then the final RMSNorm + LM head into the logits buffer; the per-block head reductions
// and samplers run as the small kernels they already are.
//
// Tensor parallel (TpLink::world > 1): every rank runs this kernel on its shard (its heads, its FFN columns,
// its LM-head rows).  The Wo and W2 phases push their partial vectors into every rank's inbox from the
// epilogue, and the phase that follows takes its input from the inbox - it polls (bounded by time) until
// all ranks' words are there and adds them in rank order - so the exchange needs no grid barrier of its
// own: barriers 3 and 5 become CTA-local, three grid barriers per layer remain.
//
// Every wait (mbarrier, grid barrier) is bounded: on expiry the CTA records an error in
// DevState::error, stops working and leaves, and so does every other CTA when its own
// wait runs out.  No reference counterpart (the reference encodes 15 dispatches per layer,
// lib.rs:513-634).
#pragma once
#include "kernels.cuh"

namespace cd {

struct MegaLayer {
    const void *wqkv, *wo, *w13, *w2;
    const float *gamma1, *gamma2;
    void* kv;
};

constexpr int MEGA_MAX_PARTS = 64;  // partial attention results per head the buffers hold
constexpr int MEGA_CPH_CAP = 8;     // CTAs that share a kv head: every CTA merges that many partials per head before Wo
constexpr int MEGA_MAX_GQA = 2;     // q heads per kv head the attention phase keeps in registers

struct MegaParams {
    const MegaLayer* layers;  // device array [nlayers]
    const void* embed;
    const void* lm_head;
    const float* gamma_final;
    float *x_a, *x_b, *q, *gate, *logits, *norm_final;
    float *part_acc, *part_ml;         // [heads][MEGA_MAX_PARTS][hd], [heads][MEGA_MAX_PARTS][2]
    unsigned long long* grid_counter;  // monotonic arrival counter of the grid barrier
    DevState* st;
    const int* page_table;
    const float2* rope;
    int dim, hidden, heads, kv_heads, hd, nlayers, vocab, q_dim, kv_dim, gqa, page_tokens, activation;
    int embed_rows;       // rows of the embedding table (vocab above is the LM-head rows this rank holds)
    float alpha, attn_scale;
    int nstages;
    uint32_t stage_cap;   // bytes per ring stage
    int rows_cap;         // rows a CTA may own in any phase
    int input_embed;      // 1: x = embed[st->token]; 0: x already in x_a
    int want_logits;
    int npages;                 // page-table entries of the sequence
    int tile_tokens;            // cached positions per attention tile (divides page_tokens; a K tile fits one ring stage)
    unsigned long long wait_ns; // bound of a grid-barrier wait
    unsigned long long* trace;  // optional [2][1 + 10 * nlayers + 1] globaltimer stamps of CTA 0 and the last CTA
    TpLink tp;                  // tensor parallel (world > 1): the dimensions above are this rank's shard
    int xs_dim;                 // floats of the CTA's vector scratch: q_dim, and dim when inputs are gathered from the ranks' inboxes
};

// Wo / W2 epilogue: x_out = res + alpha y on one GPU; tensor parallel, the rank's partial y goes to every rank's
// inbox instead (EpiPush) and the phase that consumes it adds the residual.
__device__ __noinline__ void push_partial(const TpLink& tp, int ar_out, int unit, float y) {
    const unsigned int seq = __ldcg(&tp.st->ar_base) + (unsigned int)ar_out;
    const size_t at = ((size_t)(seq % 3u) * tp.world + tp.rank) * tp.dim + unit;
    const float v = tp_sanitize(y);
    for (int r = 0; r < tp.world; ++r) reinterpret_cast<float*>(tp.peers[r])[at] = v;
}
struct EpiPushPartial {  // Wo / W2 under tensor parallelism: the rank's partial row to every rank's inbox as all-reduce ar_out
    const TpLink* tp;
    int ar_out;
    __device__ void operator()(int unit, const float (&y)[1]) const { push_partial(*tp, ar_out, unit, y[0]); }
};

// Two groups of eight consumer warps take alternate ring stages: a stage's latency chain
// (shared-memory loads, FMA chain, shuffle reduction) is long, and only with two stages
// in progress do the consumers drain the ring clearly faster than HBM fills it, which is
// what lets them catch up after every barrier.
constexpr int MEGA_GROUPS = 2;
constexpr int MEGA_CONSUMERS = MEGA_GROUPS * GEMV_CONSUMERS;
constexpr int MEGA_THREADS = MEGA_CONSUMERS + 32;  // + the producer's warp (one working thread)
constexpr int MEGA_TEAMS = MEGA_CONSUMERS / 128;
constexpr int MEGA_TEAM_SMEM = 128 * 8 + 64;  // floats per team: lane-group accumulators, then (max, sum) pairs
// floats of shared memory the attention phase needs: the teams' scratch (which the merged attention vector
// of the following phase reuses), then the teams' partials
__host__ __device__ inline size_t mega_attn_scratch_floats(int q_dim) {
    return (size_t)MEGA_TEAMS * MEGA_TEAM_SMEM > (size_t)q_dim ? (size_t)MEGA_TEAMS * MEGA_TEAM_SMEM : (size_t)q_dim;
}
__host__ __device__ inline size_t mega_attn_smem_floats(int q_dim) {
    return mega_attn_scratch_floats(q_dim) + (size_t)MEGA_TEAMS * MEGA_MAX_GQA * (128 + 2);
}

__device__ inline void mega_bar() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ inline void group_bar(int grp) { asm volatile("bar.sync %0, 256;" ::"r"(4 + grp) : "memory"); }
__device__ inline void team_bar(int team) { asm volatile("bar.sync %0, 128;" ::"r"(8 + team) : "memory"); }
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
// mbarrier wait that gives up after budget_ns, or at once when the CTA's abort flag is up: the waits of a CTA that is
// leaving (its ring may never be filled or drained again) must not each run for the seconds mbar_wait allows
__device__ inline bool mbar_wait_or_abort(uint32_t bar, uint32_t parity, const int* abort_flag, unsigned long long budget_ns) {
    unsigned long long t0 = 0;
    for (int i = 0;; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (abort_flag != nullptr && *reinterpret_cast<const volatile int*>(abort_flag) != 0) return false;
        if ((i & 15) == 15) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > budget_ns) return false;
        }
    }
}
__device__ inline void mbar_arrive_n(uint32_t bar, uint32_t n) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(n) : "memory");
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

// ---- who computes which part of the attention
// A kv head belongs to `cph` consecutive CTAs (as many as fit, at most one per tile and at most
// MEGA_MAX_PARTS); CTA j of them takes tiles [j * ntiles / cph, (j + 1) * ntiles / cph) and
// produces partial j of every q head of that kv head.  With more kv heads than CTAs each CTA
// walks heads blockIdx.x, blockIdx.x + gridDim.x, ... on its own (cph = 1).
struct AttnPlan {
    int cph;          // CTAs (= partials) per kv head
    int first, step;  // this CTA's kv heads: first, first + step, ... (first < 0: none)
    int part;         // this CTA's partial index within its head
};
__device__ inline AttnPlan attn_plan(int kv_heads, int ntiles) {
    AttnPlan a;
    const int G = gridDim.x, c = blockIdx.x;
    if (kv_heads <= G) {
        a.cph = max(1, min(min(G / kv_heads, ntiles), MEGA_CPH_CAP));
        a.first = c < kv_heads * a.cph ? c / a.cph : -1;
        a.step = kv_heads;  // one head only
        a.part = c % a.cph;
    } else {
        a.cph = 1;
        a.first = c;
        a.step = G;
        a.part = 0;
    }
    return a;
}
__device__ inline void attn_tiles(const AttnPlan& a, int ntiles, int& t0, int& t1) {
    t0 = (int)((long long)a.part * ntiles / a.cph);
    t1 = (int)((long long)(a.part + 1) * ntiles / a.cph);
}

// ---- the token's stream: everything this CTA reads from HBM for one token, stage by stage, in the
// order the consumers use it.  f(src, bytes, is_kv) is called once per ring stage; false stops the walk.
template <int R, class F>
__device__ inline bool walk_rows(const void* W, uint32_t row_bytes, int N, int unit, F& f) {
    int r0, r1;
    cta_rows(N, unit, r0, r1);
    const char* Wb = reinterpret_cast<const char*>(W) + (size_t)r0 * row_bytes;
    const int ngroups = (r1 - r0 + R - 1) / R;
    for (int g = 0; g < ngroups; ++g) {
        const int rows = min(R, (r1 - r0) - g * R);
        if (!f(Wb + (size_t)g * R * row_bytes, (uint32_t)rows * row_bytes, false)) return false;
    }
    return true;
}
// the K and V tiles of this CTA's attention work, one stage each, K before V
template <class F>
__device__ inline bool walk_attention(const MegaParams& p, const char* kv, const int* pt, int attn_len, uint32_t kes, F& f) {
    const int T = p.tile_tokens, ntiles = (attn_len + T - 1) / T;
    const AttnPlan plan = attn_plan(p.kv_heads, ntiles);
    if (plan.first < 0) return true;
    int t0, t1;
    attn_tiles(plan, ntiles, t0, t1);
    const size_t head_bytes = (size_t)p.page_tokens * p.hd * kes, page_bytes = (size_t)2 * p.kv_heads * head_bytes;
    const uint32_t bytes = (uint32_t)T * p.hd * kes;
    // (one thread walks this: its dependent integer arithmetic is part of the pace of the phase, so page and offset
    // advance by increments instead of a division per tile)
    const int tpp = p.page_tokens / T;  // tiles per page
    const size_t v_off = (size_t)p.kv_heads * head_bytes;
    for (int h = plan.first; h < p.kv_heads; h += plan.step) {
        int pg = t0 / tpp, sub = t0 % tpp;
        const char* hb = kv + (size_t)h * head_bytes;
        for (int t = t0; t < t1; ++t) {
            const char* k = hb + (size_t)pt[pg] * page_bytes + (size_t)sub * bytes;
            if (!f(k, bytes, true) || !f(k + v_off, bytes, true)) return false;
            if (++sub == tpp) { sub = 0; ++pg; }
        }
    }
    return true;
}
template <int RD, int RH, class F>
__device__ inline bool walk_token_stream(const MegaParams& p, const int* pt, int attn_len, uint32_t rb_d, uint32_t rb_q, uint32_t rb_h, uint32_t kes, F& f) {
    for (int l = 0; l < p.nlayers; ++l) {
        const MegaLayer& L = p.layers[l];
        if (!(walk_rows<RD>(L.wqkv, rb_d, p.q_dim + 2 * p.kv_dim, 2, f) &&
              walk_attention(p, reinterpret_cast<const char*>(L.kv), pt, attn_len, kes, f) &&
              walk_rows<RD>(L.wo, rb_q, p.dim, 1, f) &&
              walk_rows<RD>(L.w13, rb_d, 2 * p.hidden, 2, f) &&
              walk_rows<RH>(L.w2, rb_h, p.dim, 1, f)))
            return false;
    }
    if (p.want_logits) return walk_rows<RD>(p.lm_head, rb_d, p.vocab, 1, f);
    return true;
}

// ---- tensor parallel: the CTA's input vector x = res + alpha * (sum over the ranks, in rank order, of all-reduce
// in_reduce), gathered from this rank's inbox into shared memory (xg), every thread a few float4 positions; both
// consumer groups then take their slices from there, CTA 0 keeps the vector in x_out.  Out of line: one copy for
// all phases, and none of it in the instruction stream of a single-GPU token.
__device__ __noinline__ void gather_input(const TpLink& tin, int K, float* xg, int* err, int* abort_flag) {
    const unsigned int seq = __ldcg(&tin.st->ar_base) + (unsigned int)tin.in_reduce;
    float* base = reinterpret_cast<float*>(tin.peers[tin.rank]);
    const float* inbox = base + (size_t)(seq % 3u) * tin.world * tin.dim;
    // re-arm the slot two all-reduces ahead (nobody reads or writes it now), split over the CTAs
    uint4* rearm = reinterpret_cast<uint4*>(base + (size_t)((seq + 2u) % 3u) * tin.world * tin.dim);
    const int n4 = tin.world * tin.dim / 4;
    for (int j = blockIdx.x * MEGA_CONSUMERS + threadIdx.x; j < n4; j += gridDim.x * MEGA_CONSUMERS)
        rearm[j] = make_uint4(TP_SENTINEL, TP_SENTINEL, TP_SENTINEL, TP_SENTINEL);
    for (int q4 = threadIdx.x; q4 < K / 4; q4 += MEGA_CONSUMERS) {
        float4 a;  // summed in fixed rank order: identical on every rank
        if (!tp_gather4(inbox, tin.world, tin.dim, (size_t)q4 * 4, a, tin.st, tin.wait_ns)) {
            atomicCAS(err, 0, DEV_ERR_TP_WAIT);
            *abort_flag = 1;
        }
        const float4 r4 = __ldcg(reinterpret_cast<const float4*>(tin.res + (size_t)q4 * 4));
        const float4 v = make_float4(r4.x + tin.alpha * a.x, r4.y + tin.alpha * a.y, r4.z + tin.alpha * a.z, r4.w + tin.alpha * a.w);
        *reinterpret_cast<float4*>(xg + (size_t)q4 * 4) = v;
        if (blockIdx.x == 0) *reinterpret_cast<float4*>(tin.x_out + (size_t)q4 * 4) = v;
    }
    mega_bar();
}

// ---- tensor parallel, first layer: the token's input vector (the embedding row of st->token, which CTA 0 also
// stores as fp32 in x_a, or x_a itself) into shared memory, so that every phase of such a kernel reads its input there
template <typename WT>
__device__ __noinline__ void stage_first_input(const MegaParams& p, float* xs) {
    constexpr int EPC = Elem<WT>::EPC;
    if (p.input_embed) {
        const WT* row = reinterpret_cast<const WT*>(p.embed) + (size_t)checked_token(__ldcg(&p.st->token), p.embed_rows, &p.st->error) * p.dim;
        for (int c = threadIdx.x; c < p.dim / EPC; c += MEGA_CONSUMERS) {
            float f[EPC];
            Elem<WT>::unpack(ldg_stream(reinterpret_cast<const char*>(row) + (size_t)c * 16), f);
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                const float4 v = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
                *reinterpret_cast<float4*>(xs + (size_t)c * EPC + e) = v;
                if (blockIdx.x == 0) *reinterpret_cast<float4*>(p.x_a + (size_t)c * EPC + e) = v;
            }
        }
    } else {
        for (int q4 = threadIdx.x; q4 < p.dim / 4; q4 += MEGA_CONSUMERS)
            *reinterpret_cast<float4*>(xs + (size_t)q4 * 4) = __ldcg(reinterpret_cast<const float4*>(p.x_a + (size_t)q4 * 4));
    }
    mega_bar();
}

// ---- consumer side: one GEMV phase.  The input vector comes from `x` (fp32, L2-only loads), from
// `x_smem` (this CTA's shared memory) or, when `embed_row` is given, from a row of the embedding
// table in storage form.
template <typename WT, int NITER, int R, int UNIT, bool NORM, class Epi>
__device__ inline bool consume_gemv(Ring& ring, const float* x, const float* x_smem, const WT* embed_row, float* x_copy, const float* gamma,
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
    float gm[NORM ? NITER : 1][NORM ? EPC : 1];  // gamma, requested together with x: one memory latency for both
    if (NORM) {
#pragma unroll
        for (int i = 0; i < NITER; ++i) {
            const int c = tid + i * GEMV_CONSUMERS;
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                const float4 g = c < nchunks ? *reinterpret_cast<const float4*>(gamma + (size_t)c * EPC + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                gm[NORM ? i : 0][NORM ? e : 0] = g.x; gm[NORM ? i : 0][NORM ? e + 1 : 0] = g.y;
                gm[NORM ? i : 0][NORM ? e + 2 : 0] = g.z; gm[NORM ? i : 0][NORM ? e + 3 : 0] = g.w;
            }
        }
    }
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
                if (c < nchunks) {
                    if (x_smem != nullptr) v = *reinterpret_cast<const float4*>(x_smem + (size_t)c * EPC + e);
                    else v = __ldcg(reinterpret_cast<const float4*>(x + (size_t)c * EPC + e));
                }
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
                    xr[i][e] = xr[i][e] * inv * gm[NORM ? i : 0][NORM ? e : 0];
                    xr[i][e + 1] = xr[i][e + 1] * inv * gm[NORM ? i : 0][NORM ? e + 1 : 0];
                    xr[i][e + 2] = xr[i][e + 2] * inv * gm[NORM ? i : 0][NORM ? e + 2 : 0];
                    xr[i][e + 3] = xr[i][e + 3] * inv * gm[NORM ? i : 0][NORM ? e + 3 : 0];
                    if (norm_out != nullptr && blockIdx.x == 0 && grp == 0)
                        *reinterpret_cast<float4*>(norm_out + (size_t)c * EPC + e) =
                            make_float4(xr[i][e], xr[i][e + 1], xr[i][e + 2], xr[i][e + 3]);
                }
            }
        }
    }

    // Ring slots are owned by groups for the whole GEMV phase: group = (global stage number) & 1,
    // and the ring has an even number of slots, so the successive uses of one slot are all
    // consumed, in order, by the same group.  (A parity wait can only tell adjacent phases of
    // an mbarrier apart; a group that skipped another group's use of a slot could mistake
    // an old phase for the one it wants.)
    for (int g = (grp - ring.g) & 1; g < ngroups; g += MEGA_GROUPS) {
        const int rg = ring.g + g;
        const int s = rg % ring.nstages;
        if (!mbar_wait(ring.full0 + 8u * s, (rg / ring.nstages) & 1)) {
            atomicCAS(err, 0, DEV_ERR_FULL_WAIT);
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
        if (lane == 0) mbar_arrive_n(ring.empty0 + 8u * s, 2);  // a stage expects 16 arrivals: eight warps of one group, twice each
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

// ---- grid barrier for the consumer threads of all CTAs (arrival k of this launch).  One thread
// per CTA adds to a monotonic counter with release semantics (a reduction, not an atomic with a
// result: no round trip) and polls it with acquire loads until all CTAs of this arrival are in;
// the wait is bounded by time.
__device__ inline bool grid_barrier(unsigned long long* counter, unsigned long long target, unsigned long long wait_ns, int* err, int* abort_flag) {
    mega_bar();  // every consumer's global writes of the phase are issued
    if (threadIdx.x == 0) {
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(counter), "l"(1ull) : "memory");
        bool ok = false;
        unsigned long long t0 = 0;
        for (int i = 0;; ++i) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(counter) : "memory");
            if (v >= target) { ok = true; break; }
            if ((i & 63) == 63) {
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > wait_ns) break;
            }
        }
        if (!ok) {
            atomicCAS(err, 0, 3);
            *abort_flag = 1;
        }
    }
    mega_bar();
    return *reinterpret_cast<volatile int*>(abort_flag) == 0;
}

// ---- attention phase (sdpa_causal, lib.rs:1426-1489, for the tiles of this CTA).  All sixteen warps
// work on every tile: team k (four warps) takes positions [k T / 4, (k + 1) T / 4) of it; LPT lanes hold one
// cached position's row as 16-byte chunks, 128 / LPT positions side by side, UNR deep, with a running
// (max, sum, weighted V) per lane group and q head.  A warp copies its rows of a tile to registers,
// releases the two ring slots (every warp arrives once on each) and computes while the next tile lands;
// nothing but the ring's barriers orders the warps until the merge at the end.
template <typename KT, int GQA>
__device__ inline bool attention_phase(Ring& ring, const MegaParams& p, const void* kv_pool, float* attn_smem, int* abort_flag, const int* pt,
                                       int attn_len, int* err) {
    constexpr int EPC = Elem<KT>::EPC;
    constexpr int UNR = 2;
    constexpr float NEG = -3.402823466e+38f;
    const int tid = threadIdx.x, team = tid >> 7, tt = tid & 127, lane = tid & 31;
    const int HD = p.hd, LPT = HD / EPC, NG = 128 / LPT;
    const int g = tt / LPT, l = tt % LPT;
    const int T = p.tile_tokens, ntiles = (attn_len + T - 1) / T, pos = attn_len - 1;
    constexpr int gqa = GQA;  // q heads per kv head: a template parameter so that one head's state costs no registers when there is one
    const AttnPlan plan = attn_plan(p.kv_heads, ntiles);
    const uint32_t row_bytes = (uint32_t)HD * sizeof(KT);
    const size_t head_stride = (size_t)p.page_tokens * HD, page_stride = (size_t)2 * p.kv_heads * head_stride;
    const KT* pool = reinterpret_cast<const KT*>(kv_pool);
    float* accs = attn_smem + team * MEGA_TEAM_SMEM;  // [NG][HD] lane-group accumulators of this team
    float* gm = accs + 128 * 8;                        // [NG] max, then [NG] sum
    float* gl = gm + 32;
    // per team and q head: (acc[HD], max, sum) for the merge across teams
    float* tparts = attn_smem + mega_attn_scratch_floats(p.xs_dim);  // [MEGA_TEAMS][MEGA_MAX_GQA][128 + 2]
    bool ok = true;
    if (plan.first >= 0) {
        int t0, t1;
        attn_tiles(plan, ntiles, t0, t1);
        const int ncta_tiles = t1 - t0;
        for (int h = plan.first; h < p.kv_heads && ok; h += plan.step) {
            float qf[GQA][EPC], acc[GQA][EPC], m[GQA], lsum[GQA];
#pragma unroll
            for (int qi = 0; qi < GQA; ++qi) {
                m[qi] = NEG;
                lsum[qi] = 0.0f;
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[qi][e] = 0.0f;
#pragma unroll
                for (int e = 0; e < EPC; e += 4) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(p.q + (size_t)(h * gqa + qi) * HD + l * EPC + e));
                    qf[qi][e] = v.x; qf[qi][e + 1] = v.y; qf[qi][e + 2] = v.z; qf[qi][e + 3] = v.w;
                }
            }
            const int TQ = max(1, T / MEGA_TEAMS);  // positions of a tile per team
            for (int idx = 0; idx < ncta_tiles; ++idx) {
                if (!ok) break;  // this warp only: the others learn it from the abort flag behind the barrier below
                const int tile = t0 + idx;
                const int sk = ring.g + 2 * idx, sv = sk + 1;
                const int slot_k = sk % ring.nstages, slot_v = sv % ring.nstages;
                if (!mbar_wait(ring.full0 + 8u * slot_k, (sk / ring.nstages) & 1) || !mbar_wait(ring.full0 + 8u * slot_v, (sv / ring.nstages) & 1)) {
                    atomicCAS(err, 0, DEV_ERR_FULL_WAIT);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t kbase = ring.base + (uint32_t)slot_k * ring.stage_cap, vbase = ring.base + (uint32_t)slot_v * ring.stage_cap;
                for (int tb = 0; tb < TQ; tb += NG * UNR) {  // bounds are uniform across the warp (shuffles inside)
                    uint4 kw[UNR], vw[UNR];
                    bool live[UNR];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int tq = tb + g + u * NG, ti = team * TQ + tq, tok = tile * T + ti;
                        kw[u] = make_uint4(0, 0, 0, 0);
                        vw[u] = make_uint4(0, 0, 0, 0);
                        live[u] = tq < TQ && ti < T && tok < attn_len;
                        if (live[u]) {
                            if (tok == pos) {  // this token's own row was written after the tile was requested: read it from global memory
                                const int page = pt[tok / p.page_tokens], off = tok % p.page_tokens;
                                const KT* kp = pool + (size_t)page * page_stride + (size_t)h * head_stride + (size_t)off * HD + l * EPC;
                                kw[u] = ldg_stream_coherent(kp);
                                vw[u] = ldg_stream_coherent(kp + (size_t)p.kv_heads * head_stride);
                            } else {
                                kw[u] = lds128(kbase + (uint32_t)ti * row_bytes + (uint32_t)l * 16u);
                                vw[u] = lds128(vbase + (uint32_t)ti * row_bytes + (uint32_t)l * 16u);
                            }
                        }
                    }
                    if (tb + NG * UNR >= TQ) {  // the warp's last rows of the tile are in registers: the slots may be refilled
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(ring.empty0 + 8u * slot_k);
                            mbar_arrive(ring.empty0 + 8u * slot_v);
                        }
                    }
#pragma unroll
                    for (int qi = 0; qi < GQA; ++qi) {
                        float sc[UNR];
                        float mnew = m[qi];
#pragma unroll
                        for (int u = 0; u < UNR; ++u) {
                            float f[EPC];
                            Elem<KT>::unpack(kw[u], f);
                            float d = 0.0f;
#pragma unroll
                            for (int e = 0; e < EPC; ++e) d = fmaf(qf[qi][e], f[e], d);
                            for (int o = LPT / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                            sc[u] = live[u] ? d * p.attn_scale : NEG;
                            mnew = fmaxf(mnew, sc[u]);
                        }
                        if (mnew > NEG) {
                            const float corr = expf(m[qi] - mnew);
                            lsum[qi] *= corr;
#pragma unroll
                            for (int e = 0; e < EPC; ++e) acc[qi][e] *= corr;
#pragma unroll
                            for (int u = 0; u < UNR; ++u) {
                                if (live[u]) {
                                    const float pr = expf(sc[u] - mnew);
                                    lsum[qi] += pr;
                                    float f[EPC];
                                    Elem<KT>::unpack(vw[u], f);
#pragma unroll
                                    for (int e = 0; e < EPC; ++e) acc[qi][e] = fmaf(pr, f[e], acc[qi][e]);
                                }
                            }
                            m[qi] = mnew;
                        }
                    }
                }
            }
            mega_bar();  // every warp is through its tiles (or has given up)
            if (*reinterpret_cast<volatile int*>(abort_flag) != 0) ok = false;
            ring.g += 2 * ncta_tiles;
            if (!ok) break;
            // ---- merge: lane groups of a team, then the teams; team 0 stores this CTA's partial of every q head
#pragma unroll
            for (int qi = 0; qi < GQA; ++qi) {  // unrolled: a run-time index would put the per-head state in local memory
#pragma unroll
                for (int e = 0; e < EPC; ++e) accs[g * HD + l * EPC + e] = acc[qi][e];
                if (l == 0) { gm[g] = m[qi]; gl[g] = lsum[qi]; }
                team_bar(team);
                float* mine = tparts + ((size_t)team * MEGA_MAX_GQA + qi) * (128 + 2);
                if (tt < HD) {
                    float M = NEG;
                    for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, gm[gg]);
                    float L = 0.0f, a = 0.0f;
                    for (int gg = 0; gg < NG; ++gg) {
                        if (gl[gg] > 0.0f) {
                            const float wgt = expf(gm[gg] - M);
                            L += gl[gg] * wgt;
                            a += accs[gg * HD + tt] * wgt;
                        }
                    }
                    mine[tt] = a;
                    if (tt == 0) { mine[128] = M; mine[129] = L; }
                }
                team_bar(team);
            }
            mega_bar();
            if (team == 0) {
                for (int qi = 0; qi < gqa; ++qi) {
                    if (tt < HD) {
                        float M = NEG;
#pragma unroll
                        for (int k = 0; k < MEGA_TEAMS; ++k) {
                            const float* tp = tparts + ((size_t)k * MEGA_MAX_GQA + qi) * (128 + 2);
                            if (tp[129] > 0.0f) M = fmaxf(M, tp[128]);
                        }
                        float L = 0.0f, a = 0.0f;
#pragma unroll
                        for (int k = 0; k < MEGA_TEAMS; ++k) {
                            const float* tp = tparts + ((size_t)k * MEGA_MAX_GQA + qi) * (128 + 2);
                            if (tp[129] > 0.0f) {
                                const float wgt = expf(tp[128] - M);
                                L += tp[129] * wgt;
                                a += tp[tt] * wgt;
                            }
                        }
                        const size_t slot = (size_t)(h * gqa + qi) * MEGA_MAX_PARTS + plan.part;
                        p.part_acc[slot * HD + tt] = a;
                        if (tt == 0) {
                            p.part_ml[slot * 2 + 0] = M;
                            p.part_ml[slot * 2 + 1] = L;
                        }
                    }
                }
            }
            mega_bar();  // the teams' partials are free for the next head
        }
    }
    return ok && *reinterpret_cast<volatile int*>(abort_flag) == 0;
}

// ---- after the barrier behind the attention phase: every CTA merges the partials of every head
// (fixed order) into the attention vector, in its own shared memory
__device__ inline void merge_attention(const MegaParams& p, float* xs, int attn_len) {
    constexpr float NEG = -3.402823466e+38f;
    const int HD = p.hd, T = p.tile_tokens, ntiles = (attn_len + T - 1) / T;
    const int cph = attn_plan(p.kv_heads, ntiles).cph;
    for (int c = threadIdx.x; c < p.q_dim / 4; c += MEGA_CONSUMERS) {  // four consecutive dimensions of one head
        const int hq = (c * 4) / HD, d = (c * 4) % HD;
        const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + (size_t)hq * MEGA_MAX_PARTS;
        const float* pa = p.part_acc + (size_t)hq * MEGA_MAX_PARTS * HD + d;
        // one pass with a running maximum, so that the loads of all partials are independent of each other
        float M = NEG, L = 0.0f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int k = 0; k < cph; ++k) {
            const float2 v = __ldcg(ml + k);
            const float4 a = __ldcg(reinterpret_cast<const float4*>(pa + (size_t)k * HD));
            if (v.y > 0.0f) {
                const float Mn = fmaxf(M, v.x);
                const float corr = expf(M - Mn), wgt = expf(v.x - Mn);
                L = L * corr + v.y * wgt;
                o.x = o.x * corr + a.x * wgt; o.y = o.y * corr + a.y * wgt; o.z = o.z * corr + a.z * wgt; o.w = o.w * corr + a.w * wgt;
                M = Mn;
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        *reinterpret_cast<float4*>(xs + (size_t)c * 4) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    }
    mega_bar();
}

// TPAR: the tensor-parallel form (a kernel of its own, so that none of it weighs on the single-GPU token)
template <typename WT, typename KT, int ND, int RD, int NH, int RH, bool TPAR>
__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_mega_kernel(const MegaParams p) {
    constexpr int NW = GEMV_CONSUMERS / 32;
    extern __shared__ __align__(128) unsigned char smraw[];
    float* partial = reinterpret_cast<float*>(smraw + (size_t)p.nstages * p.stage_cap);  // [rows_cap][NW]
    float* red = partial + (size_t)p.rows_cap * NW;                                       // 32 per group
    float* attn_smem = red + 32 * MEGA_GROUPS;                                            // see mega_attn_smem_floats
    float* xs = attn_smem;                                                                // [xs_dim] merged attention vector / gathered input, over the teams' scratch
    int* flags = reinterpret_cast<int*>(attn_smem + mega_attn_smem_floats(p.xs_dim));      // [4] abort
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
            mbar_init(ring.empty0 + 8u * s, 2 * NW);  // the GEMV group's eight warps twice, or all sixteen warps of the attention phase
        }
        mbar_fence_init();
        for (int i = 0; i < 8; ++i) flags[i] = 0;
    }
    for (int i = tid; i < p.npages; i += MEGA_THREADS) pt_s[i] = p.page_table[i];
    __syncthreads();
    const int attn_len = __ldcg(&p.st->pos) + 1;  // written by the previous token's last kernel

    if (warp == MEGA_CONSUMERS / 32) {  // ---- producer: fills the ring, stage after stage, as slots come free
        if ((tid & 31) == 0) {
            const uint64_t policy = l2_evict_first_policy();
            uint64_t kv_policy;
            asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(kv_policy));
            int slot = 0;        // ring.g % nstages and ring.g / nstages, kept by increments (no division per stage)
            uint32_t turns = 0;
            uint32_t dst = ring.base, full = ring.full0, empty = ring.empty0;
            const unsigned long long producer_budget = p.wait_ns + 2000000000ull;
            auto put = [&](const char* src, uint32_t bytes, bool is_kv) {
                // (a consumer that gave up raises the CTA's abort flag: the slot will not come free, and that is no error of its own)
                if (turns > 0 && !mbar_wait_or_abort(empty, (turns - 1) & 1u, flags + 4, producer_budget)) {
                    if (*reinterpret_cast<volatile int*>(flags + 4) == 0) atomicCAS(err, 0, DEV_ERR_EMPTY_WAIT);
                    return false;
                }
                mbar_arrive_expect_tx(full, bytes);
                if (is_kv) bulk_g2s_stream(dst, src, bytes, full, kv_policy);  // cached positions are read again by the next token: no evict-first
                else bulk_g2s_stream(dst, src, bytes, full, policy);
                ring.g += 1;
                if (++slot == ring.nstages) { slot = 0; turns += 1; dst = ring.base; full = ring.full0; empty = ring.empty0; }
                else { dst += ring.stage_cap; full += 8u; empty += 8u; }
                return true;
            };
            walk_token_stream<RD, RH>(p, pt_s, attn_len, rb_d, (uint32_t)p.q_dim * (uint32_t)sizeof(WT), rb_h, (uint32_t)sizeof(KT), put);
        }
        return;
    }
    // ---- consumers
    const unsigned long long nbar = (TPAR ? 3ull : 5ull) * (unsigned long long)p.nlayers;
    const unsigned long long epoch = __ldcg(&p.st->epoch);  // launches completed so far; stable until the last barrier
    unsigned long long arrivals = epoch * nbar;  // barriers completed by earlier launches
    auto barrier = [&]() {
        arrivals += 1;
        return grid_barrier(p.grid_counter, arrivals * gridDim.x, p.wait_ns, err, flags + 4);
    };
    // behind a phase whose output travels through the ranks' inboxes the consumer's poll is the synchronisation: the CTA
    // only has to be done with its own shared memory
    auto exchange = [&]() {
        if constexpr (!TPAR) return barrier();
        mega_bar();
        return *reinterpret_cast<volatile int*>(flags + 4) == 0;
    };
    unsigned long long* tr = nullptr;
    if (p.trace != nullptr && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
        tr = p.trace + (blockIdx.x == 0 ? 0 : 1) * (size_t)(10 * p.nlayers + 2);
    auto stamp = [&]() {
        if (tr != nullptr) *tr++ = global_ns();
    };
    stamp();
    const WT* embed_row = nullptr;
    if (!TPAR && p.input_embed) embed_row = reinterpret_cast<const WT*>(p.embed) + (size_t)checked_token(__ldcg(&p.st->token), p.embed_rows, err) * p.dim;
    TpLink tin = p.tp;  // tensor parallel: the all-reduced input of a phase, x = res + alpha * sum
    tin.alpha = p.alpha;
    bool ok = true;
    for (int l = 0; l < p.nlayers && ok; ++l) {
        const MegaLayer L = p.layers[l];
        EpiQKV<KT> eq{p.q, reinterpret_cast<KT*>(L.kv), p.page_table, p.st, p.rope, p.q_dim, p.kv_dim, p.hd, p.kv_heads, p.page_tokens};
        if constexpr (TPAR) {
            // layers after the first: x = x2 + alpha * sum(W2 partials of the layer before), kept in x_a
            if (l == 0) stage_first_input<WT>(p, xs);
            else { tin.in_reduce = 2 * l; tin.res = p.x_b; tin.x_out = p.x_a; gather_input(tin, p.dim, xs, err, flags + 4); }
            ok = consume_gemv<WT, ND, RD, 2, true>(ring, nullptr, xs, nullptr, nullptr, L.gamma1, nullptr, p.q_dim + 2 * p.kv_dim, p.dim, partial,
                                                   red, err, flags + 4, eq);
        } else {
            ok = consume_gemv<WT, ND, RD, 2, true>(ring, p.x_a, nullptr, l == 0 ? embed_row : nullptr, p.x_a, L.gamma1, nullptr,
                                                   p.q_dim + 2 * p.kv_dim, p.dim, partial, red, err, flags + 4, eq);
        }
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        ok = p.gqa == 1 ? attention_phase<KT, 1>(ring, p, L.kv, attn_smem, flags + 4, pt_s, attn_len, err)
                        : attention_phase<KT, 2>(ring, p, L.kv, attn_smem, flags + 4, pt_s, attn_len, err);
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        merge_attention(p, xs, attn_len);
        if constexpr (TPAR)
            ok = consume_gemv<WT, ND, RD, 1, false>(ring, nullptr, xs, nullptr, nullptr, nullptr, nullptr, p.dim, p.q_dim, partial, red, err,
                                                    flags + 4, EpiPushPartial{&p.tp, 2 * l + 1});
        else
            ok = consume_gemv<WT, ND, RD, 1, false>(ring, nullptr, xs, nullptr, nullptr, nullptr, nullptr, p.dim, p.q_dim, partial, red, err,
                                                    flags + 4, EpiResidual{p.x_a, p.x_b, p.alpha});
        stamp();
        if (!ok || !(ok = exchange())) break;
        stamp();
        if constexpr (TPAR) {  // x2 = x + alpha * sum(Wo partials), kept in x_b
            tin.in_reduce = 2 * l + 1; tin.res = p.x_a; tin.x_out = p.x_b;
            gather_input(tin, p.dim, xs, err, flags + 4);
            ok = consume_gemv<WT, ND, RD, 2, true>(ring, nullptr, xs, nullptr, nullptr, L.gamma2, nullptr, 2 * p.hidden, p.dim, partial, red, err,
                                                   flags + 4, EpiGate{p.gate, p.activation});
        } else {
            ok = consume_gemv<WT, ND, RD, 2, true>(ring, p.x_b, nullptr, nullptr, nullptr, L.gamma2, nullptr, 2 * p.hidden, p.dim, partial, red, err,
                                                   flags + 4, EpiGate{p.gate, p.activation});
        }
        stamp();
        if (!ok || !(ok = barrier())) break;
        stamp();
        if constexpr (TPAR)
            ok = consume_gemv<WT, NH, RH, 1, false>(ring, p.gate, nullptr, nullptr, nullptr, nullptr, nullptr, p.dim, p.hidden, partial, red, err,
                                                    flags + 4, EpiPushPartial{&p.tp, 2 * l + 2});
        else
            ok = consume_gemv<WT, NH, RH, 1, false>(ring, p.gate, nullptr, nullptr, nullptr, nullptr, nullptr, p.dim, p.hidden, partial, red, err,
                                                    flags + 4, EpiResidual{p.x_b, p.x_a, p.alpha});
        stamp();
        if (!ok || !(ok = exchange())) break;
        stamp();
    }
    if (ok && p.want_logits) {
        if constexpr (TPAR) {
            tin.in_reduce = 2 * p.nlayers; tin.res = p.x_b; tin.x_out = p.x_a;
            gather_input(tin, p.dim, xs, err, flags + 4);
            ok = consume_gemv<WT, ND, RD, 1, true>(ring, nullptr, xs, nullptr, nullptr, p.gamma_final, p.norm_final, p.vocab, p.dim, partial, red,
                                                   err, flags + 4, EpiStore{p.logits});
        } else {
            ok = consume_gemv<WT, ND, RD, 1, true>(ring, p.x_a, nullptr, nullptr, nullptr, p.gamma_final, p.norm_final, p.vocab, p.dim, partial, red,
                                                   err, flags + 4, EpiStore{p.logits});
        }
    }
    stamp();
    if (ok && tid == 0 && blockIdx.x == 0) p.st->epoch = epoch + 1;  // every CTA read it before its first barrier
    if (!ok) {
        // leave only once copies that may still be in flight towards this CTA have landed: a copy lands within
        // microseconds, and a slot nobody filled never completes, so the wait for each is short
        for (int s = 0; s < p.nstages; ++s) mbar_wait_or_abort(ring.full0 + 8u * s, (ring.g / ring.nstages) & 1, nullptr, 200000ull);
    }
}

}  // namespace cd
