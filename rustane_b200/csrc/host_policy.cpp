// Host-side policy and samplers of the token loop: backend selection, the LCG, the
// CPU samplers that run on read-back logits / candidates, and the top-k merge.
// No device work: these entry points are usable without a GPU.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <numeric>
#include <vector>

#include "../../include/cuda_decode.h"

namespace {
constexpr size_t AUTO_PARAM_THRESHOLD = 20000000;  // AUTO_METAL_PARAM_THRESHOLD, inference.rs:9
const float NEG_INF = -std::numeric_limits<float>::infinity();

// Rust's Iterator::max_by keeps the last of several equal maxima (inference.rs:776-781).
size_t argmax_keep_last(const float* x, size_t n) {
    size_t best = 0;
    for (size_t i = 1; i < n; ++i)
        if (x[i] >= x[best]) best = i;
    return best;
}

// softmax draw shared by the three samplers: sum of exp((z - max)/T) in index order,
// then inverse CDF by repeated subtraction (inference.rs:806-820, :841-848, :909-916).
template <class Get> long draw_index(size_t n, float t, uint64_t* rng, Get z, bool* degenerate) {
    float mx = NEG_INF;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, z(i));
    float sum = 0.0f;
    for (size_t i = 0; i < n; ++i) sum += std::exp((z(i) - mx) / t);
    *degenerate = !std::isfinite(sum) || sum <= 0.0f;
    if (*degenerate) return -1;
    float draw = cd_lcg_next_f32(rng) * sum;
    for (size_t i = 0; i < n; ++i) {
        draw -= std::exp((z(i) - mx) / t);
        if (draw <= 0.0f) return (long)i;
    }
    return n ? (long)n - 1 : 0;
}
}  // namespace

extern "C" {

size_t cd_param_count(const cd_config* c) {
    const size_t per_layer = 4 * (size_t)c->dim * c->dim + 3 * (size_t)c->dim * c->hidden;
    return (size_t)c->nlayers * per_layer + (size_t)c->vocab * c->dim + (size_t)c->dim * (2 * (size_t)c->nlayers + 1);
}

int cd_tp_shard_plan(const cd_config* cfg, int world, int rank, cd_config* local, int32_t* vocab_first, int32_t* vocab_rows) {
    if (!cfg || !local || !vocab_first || !vocab_rows) return CD_ERR_INVALID;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CD_ERR_INVALID;
    if (cfg->heads % world || cfg->kv_heads % world || cfg->hidden % (8 * world)) return CD_ERR_UNSUPPORTED;
    *local = *cfg;
    local->heads /= world; local->kv_heads /= world; local->hidden /= world; local->q_dim /= world; local->kv_dim /= world;
    const int nblk = (cfg->vocab + CD_HEAD_BLOCK - 1) / CD_HEAD_BLOCK, per = (nblk + world - 1) / world;
    *vocab_first = std::min(cfg->vocab, rank * per * CD_HEAD_BLOCK);
    *vocab_rows = std::min(cfg->vocab - *vocab_first, per * CD_HEAD_BLOCK);
    return *vocab_rows > 0 ? CD_OK : CD_ERR_UNSUPPORTED;
}

int cd_moe_shard_plan(const cd_config* cfg, const cd_moe_config* moe, int world, int rank, int32_t* expert_first, int32_t* expert_count,
                      int32_t* shared_first, int32_t* shared_cols) {
    if (!cfg || !moe || !expert_first || !expert_count || !shared_first || !shared_cols) return CD_ERR_INVALID;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return CD_ERR_INVALID;
    if (moe->n_experts % world || (moe->n_shared * cfg->hidden) % (8 * world)) return CD_ERR_UNSUPPORTED;
    *expert_count = moe->n_experts / world;
    *expert_first = rank * *expert_count;
    *shared_cols = moe->n_shared * cfg->hidden / world;
    *shared_first = rank * *shared_cols;
    return CD_OK;
}

const char* cd_backend_name(int b) { return b == CD_BACKEND_AUTO ? "auto" : b == CD_BACKEND_NAIVE ? "naive" : b == CD_BACKEND_CUDA ? "cuda" : "?"; }

int cd_backend_parse(const char* raw) {
    if (!raw) return -1;
    if (!strcmp(raw, "auto")) return CD_BACKEND_AUTO;
    if (!strcmp(raw, "naive")) return CD_BACKEND_NAIVE;
    if (!strcmp(raw, "cuda")) return CD_BACKEND_CUDA;
    return -1;
}

const char* cd_mode_name(int mode) {
    return mode == CD_MODE_PREFILL_ONLY ? "prefill_only" : mode == CD_MODE_NAIVE_FULL_CONTEXT ? "naive_full_context"
         : mode == CD_MODE_KV_CACHE_CUDA ? "kv_cache_cuda" : "?";
}

int cd_select_decode_mode(const cd_config* cfg, int backend, size_t ctx, size_t steps, cd_selection* out) {
    if (!cfg || !out) return CD_ERR_INVALID;
    out->fallback_reason = nullptr;
    out->auto_reason = nullptr;
    if (steps == 0) { out->mode = CD_MODE_PREFILL_ONLY; return CD_OK; }
    const bool window_ok = steps > 1 && ctx + steps <= (size_t)cfg->seq;
    const bool too_long = ctx + steps > (size_t)cfg->seq && steps > 1;
    switch (backend) {
        case CD_BACKEND_NAIVE:
            out->mode = CD_MODE_NAIVE_FULL_CONTEXT;
            return CD_OK;
        case CD_BACKEND_CUDA:
            if (window_ok) { out->mode = CD_MODE_KV_CACHE_CUDA; return CD_OK; }
            out->mode = CD_MODE_NAIVE_FULL_CONTEXT;
            out->fallback_reason = steps <= 1 ? "single_step_prefers_naive" : "requested_length_exceeds_cfg_seq";
            return CD_OK;
        case CD_BACKEND_AUTO:
            if (!window_ok) {
                out->mode = CD_MODE_NAIVE_FULL_CONTEXT;
                if (too_long) out->fallback_reason = "requested_length_exceeds_cfg_seq";
                out->auto_reason = steps <= 1 ? "single_step_prefers_naive" : "window_not_metal_eligible";
            } else if (cd_param_count(cfg) >= AUTO_PARAM_THRESHOLD) {
                out->mode = CD_MODE_KV_CACHE_CUDA;
                out->auto_reason = "model_param_count_ge_threshold";
            } else {
                out->mode = CD_MODE_NAIVE_FULL_CONTEXT;
                out->auto_reason = "model_param_count_lt_threshold";
            }
            return CD_OK;
        default: return CD_ERR_INVALID;
    }
}

uint64_t cd_lcg_next_u64(uint64_t* s) {
    *s = *s * 6364136223846793005ull + 1442695040888963407ull;
    return *s;
}

float cd_lcg_next_f32(uint64_t* s) { return (float)(cd_lcg_next_u64(s) >> 40) / 16777216.0f; }

size_t cd_sample_softmax_index(const float* logits, size_t n, float t, uint64_t* rng) {
    bool degenerate;
    const long i = draw_index(n, t, rng, [&](size_t j) { return logits[j]; }, &degenerate);
    return degenerate ? argmax_keep_last(logits, n) : (size_t)i;
}

uint32_t cd_sample_next(const float* logits, size_t n, float t, size_t top_k, uint64_t* rng) {
    if (n == 0) return 0;
    if (t <= 0.0f || top_k == 1) return (uint32_t)argmax_keep_last(logits, n);
    if (top_k == 0 || top_k >= n) return (uint32_t)cd_sample_softmax_index(logits, n, t, rng);
    // Top-k by descending logit.  The reference sorts with sort_unstable_by, leaving the
    // order of equal logits unspecified; equal logits go to the lower index here.
    std::vector<uint32_t> order(n);
    std::iota(order.begin(), order.end(), 0u);
    std::partial_sort(order.begin(), order.begin() + top_k, order.end(), [&](uint32_t a, uint32_t b) {
        return logits[a] > logits[b] || (logits[a] == logits[b] && a < b);
    });
    bool degenerate;
    const long i = draw_index(top_k, t, rng, [&](size_t j) { return logits[order[j]]; }, &degenerate);
    return degenerate ? order[0] : order[(size_t)i];
}

uint32_t cd_sample_topk_candidates(const uint32_t* idxs, const float* logits, size_t n, float t, uint64_t* rng) {
    if (n == 0) return 0;
    if (t <= 0.0f || n == 1) return idxs[0];
    bool degenerate;
    const long i = draw_index(n, t, rng, [&](size_t j) { return logits[j]; }, &degenerate);
    return degenerate ? idxs[0] : idxs[(size_t)i];
}

size_t cd_sample_block_from_stats(const float* maxes, const float* sums, size_t n, uint64_t* rng) {
    if (n == 0) return 0;
    float gmax = NEG_INF;
    for (size_t b = 0; b < n; ++b)
        if (std::isfinite(maxes[b])) gmax = std::max(gmax, maxes[b]);
    if (!std::isfinite(gmax)) return 0;
    auto weight = [&](size_t b) {
        const bool ok = std::isfinite(maxes[b]) && std::isfinite(sums[b]) && sums[b] > 0.0f;
        return ok ? std::exp(maxes[b] - gmax) * sums[b] : 0.0f;
    };
    float total = 0.0f;
    for (size_t b = 0; b < n; ++b) total += weight(b);
    if (!std::isfinite(total) || total <= 0.0f) return 0;
    float draw = cd_lcg_next_f32(rng) * total;
    for (size_t b = 0; b < n; ++b) {
        draw -= weight(b);
        if (draw <= 0.0f) return b;
    }
    return n - 1;
}

size_t cd_merge_topk_candidates(const float* vals, const uint32_t* idxs, size_t n, size_t top_k, float* out_vals,
                                uint32_t* out_idxs) {
    std::fill(out_vals, out_vals + top_k, NEG_INF);
    std::fill(out_idxs, out_idxs + top_k, 0xffffffffu);
    for (size_t j = 0; j < n; ++j) {
        const float v = vals[j];
        const uint32_t id = idxs[j];
        if (id == 0xffffffffu || !std::isfinite(v)) continue;
        size_t slot = 0;
        while (slot < top_k && !(v > out_vals[slot] || (v == out_vals[slot] && id < out_idxs[slot]))) ++slot;
        if (slot == top_k) continue;
        std::copy_backward(out_vals + slot, out_vals + top_k - 1, out_vals + top_k);
        std::copy_backward(out_idxs + slot, out_idxs + top_k - 1, out_idxs + top_k);
        out_vals[slot] = v;
        out_idxs[slot] = id;
    }
    size_t filled = 0;
    while (filled < top_k && out_idxs[filled] != 0xffffffffu) ++filled;
    return filled;
}

}  // extern "C"
