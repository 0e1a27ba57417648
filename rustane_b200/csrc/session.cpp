// InferenceSession (crates/engine/src/inference.rs:105-451, :542-757) restated over the
// cuda_decode model.  The prompt is prefilled once; every sample of every request
// rewinds the KV cache to the prompt length instead of re-uploading it
// (the reference re-seeds from CPU caches per sample, decode.rs:73-89).  A request's
// prompt suffix is prefilled once per request, as one chunk into the pages behind the
// prompt (the reference feeds it token by token, once for the logits and again for
// every sample: inference.rs:563-565, :650-670); the samples then start behind it.
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/cuda_decode.h"

namespace {
using Clock = std::chrono::steady_clock;
double ms_since(Clock::time_point t0) { return std::chrono::duration<double, std::milli>(Clock::now() - t0).count(); }

struct Sample {
    uint64_t seed = 0;
    std::vector<uint32_t> generated, sampled;
    double decode_ms = 0;
};
}  // namespace

struct cd_session {
    cd_model* m = nullptr;
    cd_config cfg;
    std::vector<uint32_t> prompt_ids;
    size_t prompt_len = 0;
    float softcap = 0.f;
    double prefill_ms = 0;
    std::vector<float> prompt_logits;
    std::vector<uint32_t> cache_tokens;  // ids whose K/V currently sit in cache positions [0, n)
    std::vector<Sample> results;
    std::string err;
};

namespace {
thread_local std::string g_session_error;

int sfail(cd_session* s, int code, const std::string& msg) {
    if (s) s->err = msg;
    g_session_error = msg;
    return code;
}

int model_fail(cd_session* s, int rc) { return sfail(s, rc, cd_last_error(s->m)); }

// validate_token_ids, inference.rs:736-749
int validate_ids(cd_session* s, const cd_config& cfg, const uint32_t* ids, size_t n, const char* source) {
    for (size_t i = 0; i < n; ++i)
        if (ids[i] >= (uint32_t)cfg.vocab)
            return sfail(s, CD_ERR_TOKEN, std::string(source) + " token id " + std::to_string(ids[i]) + " at position " +
                                              std::to_string(i) + " exceeds model vocab " + std::to_string(cfg.vocab));
    return CD_OK;
}

// fill_input_window, inference.rs:751-757: the last <= seq tokens.
void window_of(const std::vector<uint32_t>& ids, size_t seq, const uint32_t** p, size_t* n) {
    const size_t start = ids.size() > seq ? ids.size() - seq : 0;
    *p = ids.data() + start;
    *n = ids.size() - start;
}

// Full forward over the window from an empty cache: what forward_logits_ws does for
// the naive path and for InferenceSession::new.
int full_forward(cd_session* s, const std::vector<uint32_t>& ids, float* logits) {
    const uint32_t* w;
    size_t n;
    window_of(ids, (size_t)s->cfg.seq, &w, &n);
    int rc = cd_set_len(s->m, 0);
    if (rc == CD_OK) rc = cd_prefill(s->m, w, n, s->softcap, logits);
    if (rc) return model_fail(s, rc);
    s->cache_tokens.assign(w, w + n);
    return CD_OK;
}

// Make cache positions [0, prompt_len) hold the base prompt again (a naive request may
// have replaced them with a shifted window).
int restore_base(cd_session* s) {
    const uint32_t* w;
    size_t n;
    window_of(s->prompt_ids, (size_t)s->cfg.seq, &w, &n);
    if (s->cache_tokens.size() >= n && std::equal(w, w + n, s->cache_tokens.begin())) return CD_OK;
    std::vector<float> scratch(s->cfg.vocab);
    return full_forward(s, s->prompt_ids, scratch.data());
}

struct Stream {
    cd_stream_cb cb;
    void* user;
};

int emit(cd_session* s, const Stream* st, Sample& r, uint32_t tok) {
    r.generated.push_back(tok);
    r.sampled.push_back(tok);
    if (st && st->cb && st->cb(tok, r.sampled.data(), r.sampled.size(), r.generated.data(), r.generated.size(), st->user))
        return sfail(s, CD_ERR_INVALID, "stream callback aborted the request");
    return CD_OK;
}

// run_cached_sample, inference.rs:542-648
int run_cached(cd_session* s, const std::vector<uint32_t>& eff_prompt, const std::vector<float>& prompt_logits,
               size_t nsuffix, const cd_request& req, uint64_t seed, const Stream* st, Sample* out) {
    Sample r;
    r.seed = seed;
    r.generated = eff_prompt;
    uint64_t rng = seed;
    // seed_from_forward_caches: rewind to the shared prefill; the request's suffix is already cached behind it
    const size_t base = s->prompt_len + nsuffix;
    int rc = cd_set_len(s->m, base);
    if (rc) return model_fail(s, rc);
    s->cache_tokens.resize(std::min(s->cache_tokens.size(), base));
    const auto t0 = Clock::now();
    const size_t steps = (size_t)req.steps;
    if (steps > 0) {
        const uint32_t first = cd_sample_next(prompt_logits.data(), prompt_logits.size(), req.temperature, (size_t)req.top_k, &rng);
        if ((rc = emit(s, st, r, first))) return rc;
        const size_t rest = steps - 1;
        std::vector<uint32_t> ids(rest);
        const bool greedy = req.temperature <= 0.0f || req.top_k == 1;
        const bool per_token = st && st->cb;  // a streaming caller wants each token as it is made
        if (rest > 0 && !per_token && (greedy || req.top_k <= CD_MAX_GPU_TOPK)) {
            if (greedy) rc = cd_decode_steps_greedy(s->m, first, rest, ids.data());
            else if (req.top_k > 0) rc = cd_decode_steps_topk(s->m, first, rest, (size_t)req.top_k, req.temperature, s->softcap, &rng, ids.data());
            else rc = cd_decode_steps_fullvocab(s->m, first, rest, req.temperature, s->softcap, &rng, ids.data());
            if (rc) return model_fail(s, rc);
            for (uint32_t t : ids)
                if ((rc = emit(s, nullptr, r, t))) return rc;
        } else {
            uint32_t cur = first;
            std::vector<float> logits;
            for (size_t i = 0; i < rest; ++i) {
                uint32_t next = 0;
                if (greedy) rc = cd_decode_steps_greedy(s->m, cur, 1, &next);
                else if (req.top_k > 0 && req.top_k <= CD_MAX_GPU_TOPK)
                    rc = cd_decode_steps_topk(s->m, cur, 1, (size_t)req.top_k, req.temperature, s->softcap, &rng, &next);
                else if (req.top_k == 0) rc = cd_decode_steps_fullvocab(s->m, cur, 1, req.temperature, s->softcap, &rng, &next);
                else {  // top_k > 32: full logits to the host sampler (inference.rs:626-638)
                    logits.resize(s->cfg.vocab);
                    rc = cd_decode_token_logits_from_id(s->m, cur, s->softcap, logits.data());
                    if (rc == CD_OK) next = cd_sample_next(logits.data(), logits.size(), req.temperature, (size_t)req.top_k, &rng);
                }
                if (rc) return model_fail(s, rc);
                if ((rc = emit(s, st, r, next))) return rc;
                cur = next;
            }
        }
        // every fed token is now cached: the first sampled one up to the one before last
        for (size_t i = 0; i + 1 < r.sampled.size(); ++i) s->cache_tokens.push_back(r.sampled[i]);
    }
    r.decode_ms = ms_since(t0);
    *out = std::move(r);
    return CD_OK;
}

// run_naive_sample, inference.rs:687-734
int run_naive(cd_session* s, const std::vector<uint32_t>& eff_prompt, const std::vector<float>& prompt_logits,
              const cd_request& req, uint64_t seed, const Stream* st, Sample* out) {
    Sample r;
    r.seed = seed;
    r.generated = eff_prompt;
    uint64_t rng = seed;
    int rc;
    if (req.steps > 0) {
        const uint32_t first = cd_sample_next(prompt_logits.data(), prompt_logits.size(), req.temperature, (size_t)req.top_k, &rng);
        if ((rc = emit(s, st, r, first))) return rc;
    }
    const auto t0 = Clock::now();
    std::vector<float> logits(s->cfg.vocab);
    for (int i = 1; i < req.steps; ++i) {
        if ((rc = full_forward(s, r.generated, logits.data()))) return rc;
        const uint32_t next = cd_sample_next(logits.data(), logits.size(), req.temperature, (size_t)req.top_k, &rng);
        if ((rc = emit(s, st, r, next))) return rc;
    }
    r.decode_ms = ms_since(t0);
    *out = std::move(r);
    return CD_OK;
}

int generate_impl(cd_session* s, const cd_request* req, const uint32_t* suffix, size_t nsuffix, const Stream* st, cd_batch_info* info) {
    if (!s || !req) return sfail(s, CD_ERR_INVALID, "null argument");
    if (st && req->samples != 1) return sfail(s, CD_ERR_INVALID, "streaming only supports samples=1");
    if (req->samples <= 0) return sfail(s, CD_ERR_INVALID, "samples must be >= 1");
    if (req->steps < 0) return sfail(s, CD_ERR_INVALID, "steps must be >= 0");
    int rc = validate_ids(s, s->cfg, suffix, nsuffix, "prompt suffix");
    if (rc) return rc;
    const size_t eff_len = std::min(s->prompt_len + nsuffix, (size_t)s->cfg.seq);
    cd_selection sel;
    cd_select_decode_mode(&s->cfg, req->decode_backend, eff_len, (size_t)req->steps, &sel);
    const bool use_kv = sel.mode == CD_MODE_KV_CACHE_CUDA;
    std::vector<uint32_t> eff_prompt = s->prompt_ids;
    eff_prompt.insert(eff_prompt.end(), suffix, suffix + nsuffix);

    double request_prefill_ms = 0;
    std::vector<float> prompt_logits = s->prompt_logits;
    if (use_kv && (rc = restore_base(s))) return rc;
    if (nsuffix > 0) {
        const auto t0 = Clock::now();
        if (use_kv) {  // prefill_prompt_suffix_cached, inference.rs:650-670, as one chunk behind the prompt
            if ((rc = cd_set_len(s->m, s->prompt_len))) return model_fail(s, rc);
            s->cache_tokens.resize(std::min(s->cache_tokens.size(), s->prompt_len));
            if ((rc = cd_prefill(s->m, suffix, nsuffix, s->softcap, prompt_logits.data()))) return model_fail(s, rc);
            s->cache_tokens.insert(s->cache_tokens.end(), suffix, suffix + nsuffix);
        } else {  // prefill_prompt_suffix_naive, :672-685
            if ((rc = full_forward(s, eff_prompt, prompt_logits.data()))) return rc;
        }
        request_prefill_ms = ms_since(t0);
    }

    s->results.clear();
    double total_decode = 0;
    // Several samples of a KV-cached request advance together, one token per step each, when the
    // model can (cd_decode_steps_samples); each keeps the seed, first-token rule and draws of the
    // sequential loop below.  CD_SAMPLES=sequential keeps the reference's one-after-the-other order.
    const char* smode = getenv("CD_SAMPLES");
    const bool greedy_req = req->temperature <= 0.0f || req->top_k == 1;
    bool batched_done = false;
    if (use_kv && !st && req->samples > 1 && req->samples <= 16 && req->steps > 1 && (greedy_req || req->top_k <= CD_MAX_GPU_TOPK) &&
        !(smode && !strcmp(smode, "sequential"))) {
        const auto t0 = Clock::now();
        if ((rc = cd_set_len(s->m, s->prompt_len + nsuffix))) return model_fail(s, rc);
        s->cache_tokens.resize(std::min(s->cache_tokens.size(), s->prompt_len + nsuffix));
        const size_t ns = (size_t)req->samples, rest = (size_t)req->steps - 1;
        std::vector<uint32_t> firsts(ns), ids(ns * rest);
        std::vector<uint64_t> rngs(ns);
        for (size_t i = 0; i < ns; ++i) {
            rngs[i] = req->seed + (uint64_t)i;
            firsts[i] = cd_sample_next(prompt_logits.data(), prompt_logits.size(), req->temperature, (size_t)req->top_k, &rngs[i]);
        }
        const int mode = greedy_req ? CD_SAMPLES_GREEDY : req->top_k > 0 ? CD_SAMPLES_TOPK : CD_SAMPLES_FULLVOCAB;
        rc = cd_decode_steps_samples(s->m, firsts.data(), ns, rest, mode, (size_t)std::max(req->top_k, 0), req->temperature, s->softcap, rngs.data(),
                                     ids.data());
        if (rc == CD_OK) {
            const double each = ms_since(t0) / (double)ns;
            for (size_t i = 0; i < ns; ++i) {
                Sample r;
                r.seed = req->seed + (uint64_t)i;
                r.generated = eff_prompt;
                r.generated.push_back(firsts[i]);
                r.sampled.push_back(firsts[i]);
                r.generated.insert(r.generated.end(), ids.begin() + i * rest, ids.begin() + (i + 1) * rest);
                r.sampled.insert(r.sampled.end(), ids.begin() + i * rest, ids.begin() + (i + 1) * rest);
                r.decode_ms = each;
                total_decode += each;
                s->results.push_back(std::move(r));
            }
            batched_done = true;
        } else if (rc != CD_ERR_UNSUPPORTED && rc != CD_ERR_CAPACITY) {
            return model_fail(s, rc);
        }
    }
    for (int i = 0; i < req->samples && !batched_done; ++i) {
        const uint64_t seed = req->seed + (uint64_t)i;  // wrapping_add, inference.rs:256
        Sample r;
        rc = use_kv ? run_cached(s, eff_prompt, prompt_logits, nsuffix, *req, seed, st, &r)
                    : run_naive(s, eff_prompt, prompt_logits, *req, seed, st, &r);
        if (rc) return rc;
        total_decode += r.decode_ms;
        s->results.push_back(std::move(r));
    }
    if (info) {
        info->selection = sel;
        info->base_prefill_ms = s->prefill_ms;
        info->request_prefill_ms = request_prefill_ms;
        info->prefill_ms = s->prefill_ms + request_prefill_ms;
        info->total_decode_ms = total_decode;
        info->avg_decode_ms = total_decode / (double)req->samples;
        info->total_ms = info->prefill_ms + total_decode;
        info->nresults = (int32_t)s->results.size();
    }
    return CD_OK;
}
}  // namespace

extern "C" {

int cd_session_create(cd_model* m, const uint32_t* prompt_ids, size_t n, float softcap, cd_session** out) {
    if (!m || !out) return sfail(nullptr, CD_ERR_INVALID, "null argument");
    *out = nullptr;
    if (!prompt_ids || n == 0) return sfail(nullptr, CD_ERR_INVALID, "prompt must contain at least one token");
    cd_session* s = new cd_session();
    s->m = m;
    cd_model_get_config(m, &s->cfg, nullptr, nullptr);
    int rc = validate_ids(s, s->cfg, prompt_ids, n, "prompt");
    if (rc) { delete s; return rc; }
    s->prompt_ids.assign(prompt_ids, prompt_ids + n);
    s->prompt_len = std::min(n, (size_t)s->cfg.seq);
    s->softcap = softcap;
    s->prompt_logits.resize(s->cfg.vocab);
    const auto t0 = Clock::now();
    rc = full_forward(s, s->prompt_ids, s->prompt_logits.data());
    s->prefill_ms = ms_since(t0);
    if (rc) { delete s; return rc; }
    *out = s;
    return CD_OK;
}

void cd_session_destroy(cd_session* s) { delete s; }
const char* cd_session_last_error(const cd_session* s) { return s ? s->err.c_str() : g_session_error.c_str(); }
size_t cd_session_prompt_len(const cd_session* s) { return s ? s->prompt_len : 0; }
double cd_session_prefill_ms(const cd_session* s) { return s ? s->prefill_ms : 0.0; }

int cd_session_prompt_logits(const cd_session* s, float* out, size_t cap) {
    if (!s || !out) return CD_ERR_INVALID;
    if (cap < s->prompt_logits.size()) return CD_ERR_CAPACITY;
    memcpy(out, s->prompt_logits.data(), s->prompt_logits.size() * 4);
    return CD_OK;
}

int cd_session_generate(cd_session* s, const cd_request* req, const uint32_t* suffix, size_t nsuffix, cd_batch_info* info) {
    return generate_impl(s, req, suffix, nsuffix, nullptr, info);
}

int cd_session_generate_stream(cd_session* s, const cd_request* req, const uint32_t* suffix, size_t nsuffix, cd_stream_cb cb,
                               void* user, cd_batch_info* info) {
    const Stream st{cb, user};
    return generate_impl(s, req, suffix, nsuffix, &st, info);
}

int cd_session_result(const cd_session* s, int i, cd_sample_result* out) {
    if (!s || !out || i < 0 || (size_t)i >= s->results.size()) return CD_ERR_INVALID;
    const Sample& r = s->results[i];
    out->seed = r.seed;
    out->generated_len = r.generated.size();
    out->sampled_len = r.sampled.size();
    out->decode_ms = r.decode_ms;
    return CD_OK;
}

int cd_session_result_tokens(const cd_session* s, int i, uint32_t* generated, size_t gcap, uint32_t* sampled, size_t scap) {
    if (!s || i < 0 || (size_t)i >= s->results.size()) return CD_ERR_INVALID;
    const Sample& r = s->results[i];
    if ((generated && gcap < r.generated.size()) || (sampled && scap < r.sampled.size())) return CD_ERR_CAPACITY;
    if (generated) memcpy(generated, r.generated.data(), r.generated.size() * 4);
    if (sampled) memcpy(sampled, r.sampled.data(), r.sampled.size() * 4);
    return CD_OK;
}

}  // extern "C"
