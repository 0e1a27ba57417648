// CPU oracle for the rustane token loop — test infrastructure only; see oracle.h.
// Every function cites the reference lines it restates.  All arithmetic is fp32
// with fp32 accumulation (the reference's CPU and Metal paths are fp32).
#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

namespace {

constexpr float RMS_EPS = 1e-5f;        // cpu/rmsnorm.rs:10, metal-decode/src/lib.rs:14
constexpr int BLOCK = 256;              // metal-decode/src/lib.rs:156 (argmax_threads)
constexpr int MAX_GPU_TOPK = 32;        // metal-decode/src/lib.rs:15
constexpr size_t AUTO_KV_PARAM_THRESHOLD = 20000000;  // inference.rs:9

// ---------------------------------------------------------------- element types
struct bf16_t { uint16_t v; };
typedef _Float16 f16_t;

inline float to_f(float x) { return x; }
inline float to_f(bf16_t x) {
    uint32_t u = (uint32_t)x.v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline float to_f(f16_t x) { return (float)x; }

inline uint16_t f32_to_bf16_bits(float f) {  // round to nearest even
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline void from_f(float f, float* o) { *o = f; }
inline void from_f(float f, bf16_t* o) { o->v = f32_to_bf16_bits(f); }
inline void from_f(float f, f16_t* o) { *o = (f16_t)f; }

inline size_t esize(int dtype) { return dtype == ORC_F32 ? 4 : 2; }

inline float round_to(float v, int dtype) {
    if (dtype == ORC_BF16) { bf16_t b; from_f(v, &b); return to_f(b); }
    if (dtype == ORC_F16) { f16_t h; from_f(v, &h); return to_f(h); }
    return v;
}

// ---------------------------------------------------------------- synthetic tensors
// Counter-based generator shared (as a specification) with the CUDA library:
// three SplitMix64 outputs per element, the twelve 16-bit fields summed
// (Irwin–Hall, variance 65536^2), centred and scaled.  Integer up to the final
// multiply, hence bit-identical on any IEEE machine.
constexpr uint64_t GOLDEN = 0x9E3779B97F4A7C15ull;
inline uint64_t mix64(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}
inline uint32_t sum16(uint64_t a) {
    return (uint32_t)(a & 0xffff) + (uint32_t)((a >> 16) & 0xffff) + (uint32_t)((a >> 32) & 0xffff) +
           (uint32_t)(a >> 48);
}
inline float synth_value(uint64_t key, uint64_t idx, float scale) {
    uint64_t base = key + 3 * idx * GOLDEN;
    uint32_t s = sum16(mix64(base + GOLDEN)) + sum16(mix64(base + 2 * GOLDEN)) +
                 sum16(mix64(base + 3 * GOLDEN));
    return (float)((int32_t)s - 393210) * scale;
}
inline uint64_t synth_key(uint64_t seed, uint64_t uid) { return mix64(seed ^ mix64(uid + GOLDEN)); }

// ---------------------------------------------------------------- model
struct Layer {
    std::vector<uint8_t> wq, wk, wv, wo, w1, w3, w2;  // reference layouts, storage dtype
    std::vector<float> gamma1, gamma2;
};

}  // namespace

struct orc_model {
    orc_config cfg;
    int kv_dtype = -1;  // what a cached K/V value is rounded to when a cache asks for rounding; -1: the library's default for cfg.dtype
    std::vector<uint8_t> embed, lm_head;
    std::vector<float> gamma_final;
    std::vector<Layer> layers;
};

struct orc_cache {
    const orc_model* m;
    int kv_round;
    size_t len;
    std::vector<std::vector<float>> k, v;  // per layer [seq, kv_dim] row-major (lib.rs:1027-1053)
    std::vector<float> norm;               // the last normalised hidden (ws.norm, lib.rs:997)
};

namespace {

// The reference's cache is fp32 (lib.rs:1027-1053); a cache created with kv_round = 1 restates the
// library's 16-bit cache instead: fp16 for every 16-bit model unless orc_model_set_kv_dtype says otherwise.
inline int kv_dtype_of(const orc_model* m) { return m->kv_dtype >= 0 ? m->kv_dtype : (m->cfg.dtype == ORC_F32 ? ORC_F32 : ORC_F16); }

template <class T> const T* as(const std::vector<uint8_t>& b) { return (const T*)b.data(); }

template <class T> void store_vec(std::vector<uint8_t>& dst, size_t n) { dst.resize(n * sizeof(T)); }

void fill_from_f32(std::vector<uint8_t>& dst, const float* src, size_t n, int dtype) {
    dst.resize(n * esize(dtype));
    if (dtype == ORC_F32) memcpy(dst.data(), src, n * 4);
    else if (dtype == ORC_BF16) { bf16_t* d = (bf16_t*)dst.data(); for (size_t i = 0; i < n; ++i) from_f(src[i], d + i); }
    else { f16_t* d = (f16_t*)dst.data(); for (size_t i = 0; i < n; ++i) from_f(src[i], d + i); }
}

float elem(const std::vector<uint8_t>& b, size_t i, int dtype) {
    if (dtype == ORC_F32) return as<float>(b)[i];
    if (dtype == ORC_BF16) return to_f(as<bf16_t>(b)[i]);
    return to_f(as<f16_t>(b)[i]);
}

void synth_fill(std::vector<uint8_t>& dst, size_t n, uint64_t seed, uint64_t uid, float std, int dtype) {
    dst.resize(n * esize(dtype));
    const uint64_t key = synth_key(seed, uid);
    const float scale = std / 65536.0f;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
        float v = synth_value(key, (uint64_t)i, scale);
        if (dtype == ORC_F32) ((float*)dst.data())[i] = v;
        else if (dtype == ORC_BF16) from_f(v, (bf16_t*)dst.data() + i);
        else from_f(v, (f16_t*)dst.data() + i);
    }
}

// ---------------------------------------------------------------- linear algebra
// y[o] = sum_i w[o*n + i] * x[i] for "out-major" matrices (embed / lm_head [V,D],
// w2 [D,H]).  Sixteen strided partial sums, then a fixed tree: deterministic.
template <class T> inline float dot(const T* w, const float* x, size_t n) {
    float acc[16] = {0};
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
        for (int l = 0; l < 16; ++l) acc[l] += to_f(w[i + l]) * x[i + l];
    for (int l = 0; i < n; ++i, ++l) acc[l] += to_f(w[i]) * x[i];
    for (int s = 8; s > 0; s >>= 1)
        for (int l = 0; l < s; ++l) acc[l] += acc[l + s];
    return acc[0];
}

// Y[t, o] = sum_i X[t, i] * W[i*out + o]  ("in-major" matrices: wq wk wv wo w1 w3,
// stored [in, out] row-major — sdpa_fwd.rs:124-169, lib.rs:1124-1188 transposeLeft).
// Accumulates over i in ascending order.
template <class T>
void matmul_in_major(const float* X, int T_, int in, const T* W, int out, float* Y) {
    const int OB = 512, TB = 16;
    const int nob = (out + OB - 1) / OB, ntb = (T_ + TB - 1) / TB;
#pragma omp parallel for collapse(2) schedule(static)
    for (int tb = 0; tb < ntb; ++tb)
        for (int ob = 0; ob < nob; ++ob) {
            const int t0 = tb * TB, t1 = std::min(T_, t0 + TB);
            const int o0 = ob * OB, o1 = std::min(out, o0 + OB);
            for (int t = t0; t < t1; ++t)
                for (int o = o0; o < o1; ++o) Y[(size_t)t * out + o] = 0.0f;
            for (int i = 0; i < in; ++i) {
                const T* wrow = W + (size_t)i * out;
                for (int t = t0; t < t1; ++t) {
                    const float xi = X[(size_t)t * in + i];
                    float* y = Y + (size_t)t * out;
                    for (int o = o0; o < o1; ++o) y[o] += xi * to_f(wrow[o]);
                }
            }
        }
}

// Y[t, o] = sum_i W[o*in + i] * X[t, i]
template <class T>
void matmul_out_major(const float* X, int T_, int in, const T* W, int out, float* Y) {
#pragma omp parallel for schedule(static)
    for (int o = 0; o < out; ++o)
        for (int t = 0; t < T_; ++t) Y[(size_t)t * out + o] = dot(W + (size_t)o * in, X + (size_t)t * in, in);
}

// cpu/rmsnorm.rs:149-183 per position: sum of squares, 1/sqrt(mean + eps), x*inv*gamma.
float rmsnorm_row(const float* x, const float* gamma, float* out, int n) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const float inv = 1.0f / std::sqrt(ss * (1.0f / (float)n) + RMS_EPS);
    for (int i = 0; i < n; ++i) out[i] = x[i] * inv * gamma[i];
    return inv;
}

// Interleaved-pair RoPE: sdpa_fwd.rs:18-33 (table), :258-293 (rotate = (-odd, even));
// same formula in the Metal kernel lib.rs:1392-1408.
void rope_row(float* x, int nheads, int hd, int pos) {
    for (int h = 0; h < nheads; ++h)
        for (int i = 0; i < hd / 2; ++i) {
            const float theta = (float)pos / std::pow(10000.0f, 2.0f * (float)i / (float)hd);
            const float c = std::cos(theta), s = std::sin(theta);
            float* p = x + h * hd + 2 * i;
            const float e = p[0], o = p[1];
            p[0] = e * c - o * s;
            p[1] = o * c + e * s;
        }
}

inline float act_gate(int activation, float x) {  // layer.rs:821-832, lib.rs:1504-1513
    if (activation == ORC_ACT_LEAKY_RELU_SQ) {
        const float l = std::max(x, 0.5f * x);
        return l * l;
    }
    const float sig = 1.0f / (1.0f + std::exp(-x));
    return x * sig;
}

inline float softcap_apply(float z, float c) { return c > 0.0f ? c * std::tanh(z / c) : z; }

// ---------------------------------------------------------------- naive_full_context
// full_model.rs:336-437 + layer.rs:1287-1431, activations held row-major [pos, D]
// (the reference keeps them channel-first; the arithmetic per position is the same).
template <class T>
int forward_impl(const orc_model* m, const uint32_t* tokens, int npos, float softcap, int kv_round,
                 const int* rows, int nrows, float* logits_rows, float* k_cf, float* v_cf,
                 float* x_prenorm_last) {
    const orc_config& c = m->cfg;
    const int D = c.dim, Q = c.q_dim, KV = c.kv_dim, H = c.hidden, V = c.vocab, hd = c.hd;
    if (npos <= 0 || npos > c.seq) return -1;
    for (int t = 0; t < npos; ++t)
        if (tokens[t] >= (uint32_t)V) return -2;
    const float alpha = 1.0f / std::sqrt(2.0f * (float)c.nlayers);  // layer.rs:1300
    const float scale = 1.0f / std::sqrt((float)hd);                // sdpa_fwd.rs:325-335

    std::vector<float> x((size_t)npos * D), xn((size_t)npos * D), x2((size_t)npos * D);
    std::vector<float> q((size_t)npos * Q), k((size_t)npos * KV), v((size_t)npos * KV);
    std::vector<float> attn((size_t)npos * Q), o((size_t)npos * D);
    std::vector<float> h1((size_t)npos * H), h3((size_t)npos * H), y((size_t)npos * D);

    // 1. embedding gather (cpu/embedding.rs:8-16)
    const T* emb = as<T>(m->embed);
    for (int t = 0; t < npos; ++t)
        for (int i = 0; i < D; ++i) x[(size_t)t * D + i] = to_f(emb[(size_t)tokens[t] * D + i]);

    for (int l = 0; l < c.nlayers; ++l) {
        const Layer& L = m->layers[l];
#pragma omp parallel for schedule(static)
        for (int t = 0; t < npos; ++t) rmsnorm_row(&x[(size_t)t * D], L.gamma1.data(), &xn[(size_t)t * D], D);
        matmul_in_major(xn.data(), npos, D, as<T>(L.wq), Q, q.data());
        matmul_in_major(xn.data(), npos, D, as<T>(L.wk), KV, k.data());
        matmul_in_major(xn.data(), npos, D, as<T>(L.wv), KV, v.data());
#pragma omp parallel for schedule(static)
        for (int t = 0; t < npos; ++t) {
            rope_row(&q[(size_t)t * Q], c.heads, hd, t);
            rope_row(&k[(size_t)t * KV], c.kv_heads, hd, t);
            if (kv_round)
                for (int i = 0; i < KV; ++i) {
                    k[(size_t)t * KV + i] = round_to(k[(size_t)t * KV + i], kv_dtype_of(m));
                    v[(size_t)t * KV + i] = round_to(v[(size_t)t * KV + i], kv_dtype_of(m));
                }
        }
        if (k_cf && v_cf)  // ForwardCache k_rope / v, channel-first [KV, seq] (layer.rs:57-58)
            for (int t = 0; t < npos; ++t)
                for (int i = 0; i < KV; ++i) {
                    k_cf[((size_t)l * KV + i) * c.seq + t] = k[(size_t)t * KV + i];
                    v_cf[((size_t)l * KV + i) * c.seq + t] = v[(size_t)t * KV + i];
                }
        // causal softmax attention with GQA head mapping kv = q_head / ratio (sdpa_fwd.rs:48-67, :325-354)
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
        for (int t = 0; t < npos; ++t)
            for (int h = 0; h < c.heads; ++h) {
                const int kvh = h / c.gqa_ratio;
                const float* qv = &q[(size_t)t * Q + h * hd];
                std::vector<float> s(t + 1);
                float mx = -std::numeric_limits<float>::infinity();
                for (int t2 = 0; t2 <= t; ++t2) {
                    const float* kr = &k[(size_t)t2 * KV + kvh * hd];
                    float d = 0.0f;
                    for (int i = 0; i < hd; ++i) d += qv[i] * kr[i];
                    s[t2] = d * scale;
                    mx = std::max(mx, s[t2]);
                }
                float sum = 0.0f;
                for (int t2 = 0; t2 <= t; ++t2) { s[t2] = std::exp(s[t2] - mx); sum += s[t2]; }
                const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
                float* out = &attn[(size_t)t * Q + h * hd];
                for (int i = 0; i < hd; ++i) out[i] = 0.0f;
                for (int t2 = 0; t2 <= t; ++t2) {
                    const float p = s[t2] * inv;
                    const float* vr = &v[(size_t)t2 * KV + kvh * hd];
                    for (int i = 0; i < hd; ++i) out[i] += p * vr[i];
                }
            }
        matmul_in_major(attn.data(), npos, Q, as<T>(L.wo), D, o.data());  // dyn_matmul.rs:400-434
#pragma omp parallel for schedule(static)
        for (int t = 0; t < npos; ++t) {
            for (int i = 0; i < D; ++i) x2[(size_t)t * D + i] = x[(size_t)t * D + i] + alpha * o[(size_t)t * D + i];  // layer.rs:1397
            rmsnorm_row(&x2[(size_t)t * D], L.gamma2.data(), &xn[(size_t)t * D], D);
        }
        matmul_in_major(xn.data(), npos, D, as<T>(L.w1), H, h1.data());  // ffn_fused.rs:114-150
        matmul_in_major(xn.data(), npos, D, as<T>(L.w3), H, h3.data());
#pragma omp parallel for schedule(static)
        for (long long j = 0; j < (long long)npos * H; ++j) h1[j] = act_gate(c.activation, h1[j]) * h3[j];
        matmul_out_major(h1.data(), npos, H, as<T>(L.w2), D, y.data());  // w2 is [D,H] (ffn_fused.rs:8, :153)
#pragma omp parallel for schedule(static)
        for (long long j = 0; j < (long long)npos * D; ++j) x[j] = x2[j] + alpha * y[j];  // ffn_fused.rs:186-197
    }

    if (x_prenorm_last) memcpy(x_prenorm_last, &x[(size_t)(npos - 1) * D], (size_t)D * 4);
    // final RMSNorm + LM head on the requested rows only (the reference computes every
    // row, full_model.rs:419-428, and reads one, inference.rs:142-144).
    const T* head = c.untied ? as<T>(m->lm_head) : emb;
    std::vector<float> xf(D);
    for (int r = 0; r < nrows; ++r) {
        const int t = rows[r];
        if (t < 0 || t >= npos) return -3;
        rmsnorm_row(&x[(size_t)t * D], m->gamma_final.data(), xf.data(), D);
        float* lg = logits_rows + (size_t)r * V;
#pragma omp parallel for schedule(static)
        for (int vv = 0; vv < V; ++vv) lg[vv] = softcap_apply(dot(head + (size_t)vv * D, xf.data(), D), softcap);
    }
    return 0;
}

// ---------------------------------------------------------------- KV-cached decode
// One decoder layer for one token at `slot`, attending slot+1 keys: lib.rs:513-634.
template <class T>
void cached_layer(orc_cache* cc, int l, const float* x_cur, float* x_next, int slot) {
    const orc_model* m = cc->m;
    const orc_config& c = m->cfg;
    const Layer& L = m->layers[l];
    const int D = c.dim, Q = c.q_dim, KV = c.kv_dim, H = c.hidden, hd = c.hd;
    const int attn_len = slot + 1;
    const float alpha = 1.0f / std::sqrt(2.0f * (float)c.nlayers);  // lib.rs:201
    const float scale = 1.0f / std::sqrt((float)hd);
    std::vector<float> norm(D), q(Q), k(KV), v(KV), attn(Q), o(D), h1(H), h3(H);

    rmsnorm_row(x_cur, L.gamma1.data(), norm.data(), D);              // rmsnorm_single :1354
    matmul_in_major(norm.data(), 1, D, as<T>(L.wq), Q, q.data());     // q_proj :532
    matmul_in_major(norm.data(), 1, D, as<T>(L.wk), KV, k.data());
    matmul_in_major(norm.data(), 1, D, as<T>(L.wv), KV, v.data());
    rope_row(q.data(), c.heads, hd, slot);                            // rope_inplace :1392
    rope_row(k.data(), c.kv_heads, hd, slot);
    float* kc = cc->k[l].data();
    float* vc = cc->v[l].data();
    for (int i = 0; i < KV; ++i) {                                    // append_kv :1410
        kc[(size_t)slot * KV + i] = cc->kv_round ? round_to(k[i], kv_dtype_of(cc->m)) : k[i];
        vc[(size_t)slot * KV + i] = cc->kv_round ? round_to(v[i], kv_dtype_of(cc->m)) : v[i];
    }
    // sdpa_causal :1426-1489 — scores, max, exp, normalise probs, weighted sum of V.
#pragma omp parallel for schedule(static)
    for (int h = 0; h < c.heads; ++h) {
        const int kvh = h / c.gqa_ratio;
        std::vector<float> s(attn_len);
        float mx = -3.402823466e+38f;
        for (int t = 0; t < attn_len; ++t) {
            float d = 0.0f;
            const float* kr = kc + (size_t)t * KV + kvh * hd;
            for (int i = 0; i < hd; ++i) d += q[h * hd + i] * kr[i];
            s[t] = d * scale;
            mx = std::max(mx, s[t]);
        }
        float sum = 0.0f;
        for (int t = 0; t < attn_len; ++t) { s[t] = std::exp(s[t] - mx); sum += s[t]; }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int t = 0; t < attn_len; ++t) s[t] *= inv;
        for (int i = 0; i < hd; ++i) {
            float acc = 0.0f;
            for (int t = 0; t < attn_len; ++t) acc += s[t] * vc[(size_t)t * KV + kvh * hd + i];
            attn[h * hd + i] = acc;
        }
    }
    matmul_in_major(attn.data(), 1, Q, as<T>(L.wo), D, o.data());     // wo_proj :578
    for (int i = 0; i < D; ++i) x_next[i] = x_cur[i] + alpha * o[i];  // residual_add :1491
    rmsnorm_row(x_next, L.gamma2.data(), norm.data(), D);
    matmul_in_major(norm.data(), 1, D, as<T>(L.w1), H, h1.data());    // w1/w3 :595-617
    matmul_in_major(norm.data(), 1, D, as<T>(L.w3), H, h3.data());
    for (int j = 0; j < H; ++j) h1[j] = act_gate(c.activation, h1[j]) * h3[j];  // silu_gate :1504
    matmul_out_major(h1.data(), 1, H, as<T>(L.w2), D, o.data());      // w2_proj: x_next += alpha*W2*gate :621
    for (int i = 0; i < D; ++i) x_next[i] = x_next[i] + alpha * o[i];
}

template <class T> int cached_layers(orc_cache* cc, const float* x_in, float* x_out) {
    const orc_config& c = cc->m->cfg;
    if (cc->len >= (size_t)c.seq) return -1;  // "metal decode only supports lengths within cfg.seq"
    std::vector<float> a(x_in, x_in + c.dim), b(c.dim);
    const int slot = (int)cc->len;
    for (int l = 0; l < c.nlayers; ++l) {
        cached_layer<T>(cc, l, a.data(), b.data(), slot);
        a.swap(b);
    }
    memcpy(x_out, a.data(), (size_t)c.dim * 4);
    cc->len += 1;
    return 0;
}

template <class T> void embed_row(const orc_model* m, uint32_t tok, float* out) {  // embed_lookup :1380
    const T* e = as<T>(m->embed);
    for (int i = 0; i < m->cfg.dim; ++i) out[i] = to_f(e[(size_t)tok * m->cfg.dim + i]);
}

// final RMSNorm into cache->norm, then raw (un-capped) logits for every vocab row.
template <class T> void head_logits(orc_cache* cc, const float* x, float* logits) {
    const orc_model* m = cc->m;
    const orc_config& c = m->cfg;
    cc->norm.resize(c.dim);
    rmsnorm_row(x, m->gamma_final.data(), cc->norm.data(), c.dim);
    const T* head = c.untied ? as<T>(m->lm_head) : as<T>(m->embed);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < c.vocab; ++r) logits[r] = dot(head + (size_t)r * c.dim, cc->norm.data(), c.dim);
}

#define DISPATCH(m, expr_f32, expr_f16, expr_bf16)                     \
    ((m)->cfg.dtype == ORC_F32 ? (expr_f32) : (m)->cfg.dtype == ORC_F16 ? (expr_f16) : (expr_bf16))

int layers_dispatch(orc_cache* c, const float* x_in, float* x_out) {
    return DISPATCH(c->m, cached_layers<float>(c, x_in, x_out), cached_layers<f16_t>(c, x_in, x_out),
                    cached_layers<bf16_t>(c, x_in, x_out));
}
void embed_dispatch(const orc_model* m, uint32_t tok, float* out) {
    if (m->cfg.dtype == ORC_F32) embed_row<float>(m, tok, out);
    else if (m->cfg.dtype == ORC_F16) embed_row<f16_t>(m, tok, out);
    else embed_row<bf16_t>(m, tok, out);
}
void head_dispatch(orc_cache* c, const float* x, float* logits) {
    if (c->m->cfg.dtype == ORC_F32) head_logits<float>(c, x, logits);
    else if (c->m->cfg.dtype == ORC_F16) head_logits<f16_t>(c, x, logits);
    else head_logits<bf16_t>(c, x, logits);
}

// (val, idx) "better" rule of every Metal reduction: larger value, ties to the lower index
// (lib.rs:1553, :1612, :1747).
inline bool better(float v, uint32_t i, float bv, uint32_t bi) { return v > bv || (v == bv && i < bi); }

// inference.rs:770-782: Rust's max_by keeps the LAST of equal maxima.
uint32_t argmax_last(const float* x, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i)
        if (!(x[i] < x[best])) best = i;  // total_cmp(x[i], x[best]) >= Equal (no NaN expected)
    return (uint32_t)best;
}

int tokens_ok(const orc_model* m, const uint32_t* ids, int n) {
    for (int i = 0; i < n; ++i)
        if (ids[i] >= (uint32_t)m->cfg.vocab) return 0;
    return 1;
}

}  // namespace

// =================================================================== C interface
extern "C" {

float orc_rmsnorm(const float* x, const float* gamma, float* out, int n) { return rmsnorm_row(x, gamma, out, n); }

void orc_embedding(const float* table, int dim, const uint32_t* ids, int n, float* out) {
    for (int s = 0; s < n; ++s) memcpy(out + (size_t)s * dim, table + (size_t)ids[s] * dim, (size_t)dim * 4);
}

// inference.rs:759-768
uint64_t orc_next_u64(uint64_t* s) {
    *s = *s * 6364136223846793005ull + 1442695040888963407ull;
    return *s;
}
float orc_next_f32(uint64_t* s) { return (float)(orc_next_u64(s) >> 40) / (float)(1ull << 24); }

// layer.rs:806-817 / full_model.rs:1513-1524
void orc_reference_random_vec(float* out, size_t n, float scale) {
    uint64_t seed = 42 + (uint64_t)n;
    for (size_t i = 0; i < n; ++i) {
        seed = seed * 6364136223846793005ull + 1442695040888963407ull;
        const float r = ((float)(uint32_t)(seed >> 32) / (float)0xffffffffu) * 2.0f - 1.0f;
        out[i] = r * scale;
    }
}

float orc_round_to(float v, int dtype) { return round_to(v, dtype); }

float orc_synth_value(uint64_t seed, uint64_t uid, uint64_t idx, float std) {
    return synth_value(synth_key(seed, uid), idx, std / 65536.0f);
}

void orc_synth_prompt(uint64_t seed, int vocab, uint32_t* ids, int n) {
    const uint64_t key = synth_key(seed, 0x70726f6d7074ull);
    for (int i = 0; i < n; ++i) ids[i] = (uint32_t)(mix64(key + (uint64_t)(i + 1) * GOLDEN) % (uint64_t)vocab);
}

size_t orc_param_count(const orc_config* c) {  // model.rs:182-187
    const size_t per_layer = 4 * (size_t)c->dim * c->dim + 3 * (size_t)c->dim * c->hidden;
    return (size_t)c->nlayers * per_layer + (size_t)c->vocab * c->dim + (size_t)c->dim * (2 * c->nlayers + 1);
}

static orc_model* model_alloc(const orc_config* cfg) {
    orc_model* m = new orc_model();
    m->cfg = *cfg;
    m->layers.resize(cfg->nlayers);
    m->gamma_final.assign(cfg->dim, 1.0f);
    for (auto& L : m->layers) { L.gamma1.assign(cfg->dim, 1.0f); L.gamma2.assign(cfg->dim, 1.0f); }
    return m;
}

// tensor uids of the synthetic-weight specification
static uint64_t uid_layer(int l, int which) { return 16 + (uint64_t)l * 16 + (uint64_t)which; }

orc_model* orc_model_synth(const orc_config* c, uint64_t seed, float std) {
    orc_model* m = model_alloc(c);
    const size_t D = c->dim, Q = c->q_dim, KV = c->kv_dim, H = c->hidden, V = c->vocab;
    synth_fill(m->embed, V * D, seed, 0, std, c->dtype);
    if (c->untied) synth_fill(m->lm_head, V * D, seed, 2, std, c->dtype);
    for (int l = 0; l < c->nlayers; ++l) {
        Layer& L = m->layers[l];
        synth_fill(L.wq, D * Q, seed, uid_layer(l, 0), std, c->dtype);
        synth_fill(L.wk, D * KV, seed, uid_layer(l, 1), std, c->dtype);
        synth_fill(L.wv, D * KV, seed, uid_layer(l, 2), std, c->dtype);
        synth_fill(L.wo, Q * D, seed, uid_layer(l, 3), std, c->dtype);
        synth_fill(L.w1, D * H, seed, uid_layer(l, 4), std, c->dtype);
        synth_fill(L.w3, D * H, seed, uid_layer(l, 5), std, c->dtype);
        synth_fill(L.w2, D * H, seed, uid_layer(l, 6), std, c->dtype);
    }
    return m;
}

// ---------------------------------------------------------------- quantised linears
// No reference definition exists (the reference stores fp32 only); the rules below are the
// specification both this file and the CUDA library follow.
//   FP8:  per output channel, scale = max|w| / 448 in fp32 (1 if the row is all zero),
//         q = e4m3(w / scale), round to nearest even, saturating at +-448; w^ = q * scale.
//   INT4: per group of 32 consecutive inputs of one output channel,
//         scale = fp16(max|w| / 7), q = clamp(rint(w / scale), -8, 7) (0 if scale is 0); w^ = q * scale.
static float e4m3_round(float v) {  // nearest representable e4m3 value (bias 7, 3 mantissa bits, max 448)
    if (!(std::fabs(v) < 448.0f)) return v < 0 ? -448.0f : 448.0f;
    if (v == 0.0f) return v;
    int e;
    std::frexp(v, &e);              // |v| = f * 2^e, f in [0.5, 1)
    int exp = e - 1;                // |v| in [2^exp, 2^(exp+1))
    if (exp < -6) exp = -6;         // denormals share the step of the smallest normal binade
    const float step = std::ldexp(1.0f, exp - 3);
    return std::nearbyint(v / step) * step;  // default rounding mode: ties to even; v / step is exact
}

extern "C" void orc_quant_dequant(float* w, int in, int out, int in_major, int mode) {
    auto at = [&](int o, int i) -> float& { return in_major ? w[(size_t)i * out + o] : w[(size_t)o * in + i]; };
#pragma omp parallel for schedule(static)
    for (int o = 0; o < out; ++o) {
        if (mode == ORC_QUANT_FP8) {
            float amax = 0.0f;
            for (int i = 0; i < in; ++i) amax = std::max(amax, std::fabs(at(o, i)));
            const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
            for (int i = 0; i < in; ++i) at(o, i) = e4m3_round(at(o, i) / scale) * scale;
        } else {
            for (int g = 0; g + 32 <= in; g += 32) {
                float amax = 0.0f;
                for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(at(o, g + i)));
                const float s = round_to(amax / 7.0f, ORC_F16);
                for (int i = 0; i < 32; ++i) {
                    float q = 0.0f;
                    if (s > 0.0f) q = std::min(std::max(std::nearbyint(at(o, g + i) / s), -8.0f), 7.0f);
                    at(o, g + i) = q * s;
                }
            }
        }
    }
}

// The model the CUDA library builds for CD_DTYPE_FP8_E4M3 / CD_DTYPE_INT4_G32 from the same
// seed: linears quantised and held as fp32 w^, embedding / LM head rounded to bf16, cached
// K and V rounded to fp16 (the library's default cache type).  cfg->dtype must be ORC_F32 (the container of the values).
extern "C" orc_model* orc_model_synth_quant(const orc_config* c, uint64_t seed, float std, int mode) {
    if (c->dtype != ORC_F32 || (mode != ORC_QUANT_FP8 && mode != ORC_QUANT_INT4)) return nullptr;
    orc_model* m = orc_model_synth(c, seed, std);
    m->kv_dtype = ORC_F16;
    auto round_bf16 = [](std::vector<uint8_t>& b) {
        float* p = (float*)b.data();
        const long long n = (long long)(b.size() / 4);
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < n; ++i) p[i] = round_to(p[i], ORC_BF16);
    };
    round_bf16(m->embed);
    if (c->untied) round_bf16(m->lm_head);
    for (auto& L : m->layers) {
        orc_quant_dequant((float*)L.wq.data(), c->dim, c->q_dim, 1, mode);
        orc_quant_dequant((float*)L.wk.data(), c->dim, c->kv_dim, 1, mode);
        orc_quant_dequant((float*)L.wv.data(), c->dim, c->kv_dim, 1, mode);
        orc_quant_dequant((float*)L.wo.data(), c->q_dim, c->dim, 1, mode);
        orc_quant_dequant((float*)L.w1.data(), c->dim, c->hidden, 1, mode);
        orc_quant_dequant((float*)L.w3.data(), c->dim, c->hidden, 1, mode);
        orc_quant_dequant((float*)L.w2.data(), c->hidden, c->dim, 0, mode);
    }
    return m;
}

// ModelWeights::random (full_model.rs:154-163) + LayerWeights::random (layer.rs:696-722)
orc_model* orc_model_reference_random(const orc_config* c) {
    orc_model* m = model_alloc(c);
    const size_t D = c->dim, Q = c->q_dim, KV = c->kv_dim, H = c->hidden, V = c->vocab;
    std::vector<float> tmp;
    auto rnd = [&](std::vector<uint8_t>& dst, size_t n, float scale) {
        tmp.resize(n);
        orc_reference_random_vec(tmp.data(), n, scale);
        fill_from_f32(dst, tmp.data(), n, c->dtype);
    };
    auto zero = [&](std::vector<uint8_t>& dst, size_t n) { dst.assign(n * esize(c->dtype), 0); };
    rnd(m->embed, V * D, 0.005f);
    if (c->untied) rnd(m->lm_head, V * D, 0.005f);
    const float sq = 1.0f / std::sqrt((float)D), sf = 1.0f / std::sqrt((float)H);
    for (auto& L : m->layers) {
        rnd(L.wq, D * Q, sq); rnd(L.wk, D * KV, sq); rnd(L.wv, D * KV, sq);
        zero(L.wo, Q * D);
        rnd(L.w1, D * H, sf); rnd(L.w3, D * H, sf);
        zero(L.w2, D * H);
    }
    return m;
}

void orc_model_free(orc_model* m) { delete m; }
void orc_model_get_config(const orc_model* m, orc_config* out) { *out = m->cfg; }

size_t orc_model_tensor(const orc_model* m, int layer, int which, float* out, size_t cap) {
    const std::vector<uint8_t>* b = nullptr;
    const std::vector<float>* f = nullptr;
    if (which == 0) b = &m->embed;
    else if (which == 1) f = &m->gamma_final;
    else if (which == 2) b = &m->lm_head;
    else {
        if (layer < 0 || layer >= m->cfg.nlayers) return 0;
        const Layer& L = m->layers[layer];
        switch (which) {
            case 10: b = &L.wq; break; case 11: b = &L.wk; break; case 12: b = &L.wv; break;
            case 13: b = &L.wo; break; case 14: b = &L.w1; break; case 15: b = &L.w3; break;
            case 16: b = &L.w2; break; case 17: f = &L.gamma1; break; case 18: f = &L.gamma2; break;
            default: return 0;
        }
    }
    if (f) {
        if (out && cap >= f->size()) memcpy(out, f->data(), f->size() * 4);
        return f->size();
    }
    const size_t n = b->size() / esize(m->cfg.dtype);
    if (out && cap >= n)
        for (size_t i = 0; i < n; ++i) out[i] = elem(*b, i, m->cfg.dtype);
    return n;
}

// ---- RSTK files: v1/v2 exactly as checkpoint.rs:25-209 reads them; v3 adds the
// fields the reference cannot express (explicit hidden/heads/kv_heads/hd, storage
// dtype, untied head).
static void put_u32(std::vector<uint8_t>& b, uint32_t v) { for (int i = 0; i < 4; ++i) b.push_back((uint8_t)(v >> (8 * i))); }

int orc_model_save(const orc_model* m, const char* path, int version) {
    const orc_config& c = m->cfg;
    if (version < 3 && (c.dtype != ORC_F32 || c.untied || c.hd != 128 || c.kv_heads != c.heads || c.heads * 128 != c.dim)) return -1;
    std::vector<uint8_t> hdr = {'R', 'S', 'T', 'K'};
    put_u32(hdr, version); put_u32(hdr, 0); put_u32(hdr, c.dim); put_u32(hdr, c.nlayers);
    put_u32(hdr, c.vocab); put_u32(hdr, c.seq);
    if (version >= 2) put_u32(hdr, c.activation);
    if (version >= 3) {
        put_u32(hdr, c.hidden); put_u32(hdr, c.heads); put_u32(hdr, c.kv_heads); put_u32(hdr, c.hd);
        put_u32(hdr, c.dtype); put_u32(hdr, c.untied ? 1u : 0u);
    }
    FILE* f = fopen(path, "wb");
    if (!f) return -2;
    auto w = [&](const void* p, size_t n) { return fwrite(p, 1, n, f) == n; };
    bool ok = w(hdr.data(), hdr.size()) && w(m->embed.data(), m->embed.size()) && w(m->gamma_final.data(), m->gamma_final.size() * 4);
    if (c.untied) ok = ok && w(m->lm_head.data(), m->lm_head.size());
    for (const Layer& L : m->layers)
        ok = ok && w(L.wq.data(), L.wq.size()) && w(L.wk.data(), L.wk.size()) && w(L.wv.data(), L.wv.size()) &&
             w(L.wo.data(), L.wo.size()) && w(L.w1.data(), L.w1.size()) && w(L.w3.data(), L.w3.size()) &&
             w(L.w2.data(), L.w2.size()) && w(L.gamma1.data(), L.gamma1.size() * 4) && w(L.gamma2.data(), L.gamma2.size() * 4);
    fclose(f);
    return ok ? 0 : -3;
}

orc_model* orc_model_load(const char* path, char* err, int errlen) {
    auto fail = [&](const std::string& s) -> orc_model* { if (err && errlen > 0) snprintf(err, errlen, "%s", s.c_str()); return nullptr; };
    FILE* f = fopen(path, "rb");
    if (!f) return fail("cannot open checkpoint");
    fseek(f, 0, SEEK_END);
    const size_t total = (size_t)ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> bytes(total);
    if (fread(bytes.data(), 1, total, f) != total) { fclose(f); return fail("short read"); }
    fclose(f);
    if (total < 4 + 6 * 4) return fail("checkpoint too small for header");
    if (memcmp(bytes.data(), "RSTK", 4) != 0) return fail("invalid checkpoint magic");
    size_t cur = 4;
    auto u32 = [&](uint32_t* v) { if (cur + 4 > total) return false; memcpy(v, &bytes[cur], 4); cur += 4; return true; };
    uint32_t version = 0, step, dim, nlayers, vocab, seq, act = 0;
    u32(&version);
    if (version < 1 || version > 3) return fail("unsupported checkpoint version " + std::to_string(version));
    if (version >= 2 && total < 4 + 7 * 4) return fail("checkpoint too small for v2 header");
    u32(&step); u32(&dim); u32(&nlayers); u32(&vocab); u32(&seq);
    if (version >= 2) { u32(&act); if (act > 1) return fail("unsupported checkpoint activation code " + std::to_string(act)); }
    if (dim == 0 || nlayers == 0 || vocab == 0 || seq == 0) return fail("checkpoint config contains zero dimension");
    orc_config c;
    memset(&c, 0, sizeof(c));
    c.dim = dim; c.nlayers = nlayers; c.vocab = vocab; c.seq = seq; c.activation = act;
    if (version <= 2) {
        if (dim % 128 != 0) return fail("checkpoint dim " + std::to_string(dim) + " is not divisible by 128");
        if ((total - cur) % 4 != 0) return fail("checkpoint payload is not aligned to f32 values");
        const size_t payload = (total - cur) / 4;
        const size_t fixed = (size_t)vocab * dim + dim, layer_fixed = 4 * (size_t)dim * dim + 2 * dim;
        if (payload < fixed + nlayers * layer_fixed) return fail("checkpoint payload too small for fixed-size tensors");
        const size_t hidden_total = payload - fixed - nlayers * layer_fixed, denom = (size_t)nlayers * 3 * dim;
        if (hidden_total % denom != 0) return fail("checkpoint payload does not imply an integer hidden size");
        if (hidden_total / denom == 0) return fail("checkpoint hidden size inferred as zero");
        c.hidden = (int)(hidden_total / denom);
        c.heads = c.kv_heads = dim / 128; c.hd = 128; c.dtype = ORC_F32; c.untied = 0;
    } else {
        uint32_t hidden, heads, kvh, hd, dtype, flags;
        if (!(u32(&hidden) && u32(&heads) && u32(&kvh) && u32(&hd) && u32(&dtype) && u32(&flags))) return fail("checkpoint too small for v3 header");
        if (!hidden || !heads || !kvh || !hd || heads % kvh || dtype > 2 || (flags & ~1u)) return fail("invalid v3 header fields");
        c.hidden = hidden; c.heads = heads; c.kv_heads = kvh; c.hd = hd; c.dtype = dtype; c.untied = flags & 1;
    }
    c.q_dim = c.heads * c.hd; c.kv_dim = c.kv_heads * c.hd; c.gqa_ratio = c.heads / c.kv_heads;
    orc_model* m = model_alloc(&c);
    const size_t es = esize(c.dtype);
    bool ok = true;
    auto mat = [&](std::vector<uint8_t>& dst, size_t n) { if (!ok || cur + n * es > total) { ok = false; return; } dst.assign(&bytes[cur], &bytes[cur] + n * es); cur += n * es; };
    auto vec = [&](std::vector<float>& dst, size_t n) { if (!ok || cur + n * 4 > total) { ok = false; return; } dst.resize(n); memcpy(dst.data(), &bytes[cur], n * 4); cur += n * 4; };
    const size_t D = c.dim, Q = c.q_dim, KV = c.kv_dim, H = c.hidden, V = c.vocab;
    mat(m->embed, V * D); vec(m->gamma_final, D);
    if (c.untied) mat(m->lm_head, V * D);
    for (Layer& L : m->layers) {
        mat(L.wq, D * Q); mat(L.wk, D * KV); mat(L.wv, D * KV); mat(L.wo, Q * D);
        mat(L.w1, D * H); mat(L.w3, D * H); mat(L.w2, D * H); vec(L.gamma1, D); vec(L.gamma2, D);
    }
    if (!ok) { delete m; return fail("unexpected EOF reading tensor"); }
    if (cur != total) { delete m; return fail("checkpoint had trailing bytes"); }
    return m;
}

int orc_forward_logits(const orc_model* m, const uint32_t* tokens, int npos, float softcap, int kv_round,
                       const int* rows, int nrows, float* logits_rows, float* k_cf, float* v_cf,
                       float* x_prenorm_last) {
    return DISPATCH(m,
                    forward_impl<float>(m, tokens, npos, softcap, kv_round, rows, nrows, logits_rows, k_cf, v_cf, x_prenorm_last),
                    forward_impl<f16_t>(m, tokens, npos, softcap, kv_round, rows, nrows, logits_rows, k_cf, v_cf, x_prenorm_last),
                    forward_impl<bf16_t>(m, tokens, npos, softcap, kv_round, rows, nrows, logits_rows, k_cf, v_cf, x_prenorm_last));
}

// ---- cached model: Model::new / set_len / seed (lib.rs:147-237)
void orc_model_set_kv_dtype(orc_model* m, int dtype) { m->kv_dtype = dtype; }

orc_cache* orc_cache_new(const orc_model* m, int kv_round) {
    orc_cache* c = new orc_cache();
    c->m = m; c->kv_round = kv_round; c->len = 0;
    c->k.assign(m->cfg.nlayers, std::vector<float>((size_t)m->cfg.seq * m->cfg.kv_dim, 0.0f));
    c->v = c->k;
    c->norm.assign(m->cfg.dim, 0.0f);
    return c;
}
void orc_cache_free(orc_cache* c) { delete c; }
size_t orc_cache_len(const orc_cache* c) { return c->len; }
void orc_cache_set_len(orc_cache* c, size_t len) { c->len = std::min(len, (size_t)c->m->cfg.seq); }

void orc_cache_seed_cf(orc_cache* c, int layer, size_t live_len, const float* k_cf, const float* v_cf) {
    const int seq = c->m->cfg.seq, KV = c->m->cfg.kv_dim;
    live_len = std::min(live_len, (size_t)seq);
    std::fill(c->k[layer].begin(), c->k[layer].end(), 0.0f);
    std::fill(c->v[layer].begin(), c->v[layer].end(), 0.0f);
    for (size_t pos = 0; pos < live_len; ++pos)
        for (int d = 0; d < KV; ++d) {
            const float kk = k_cf[(size_t)d * seq + pos], vv = v_cf[(size_t)d * seq + pos];
            c->k[layer][pos * KV + d] = c->kv_round ? round_to(kk, kv_dtype_of(c->m)) : kk;
            c->v[layer][pos * KV + d] = c->kv_round ? round_to(vv, kv_dtype_of(c->m)) : vv;
        }
}

int orc_decode_token(orc_cache* c, const float* x_in, float* x_out) { return layers_dispatch(c, x_in, x_out); }

int orc_decode_token_from_id(orc_cache* c, uint32_t tok, float* x_out) {
    if (tok >= (uint32_t)c->m->cfg.vocab) return -2;
    std::vector<float> x(c->m->cfg.dim);
    embed_dispatch(c->m, tok, x.data());
    return layers_dispatch(c, x.data(), x_out);
}

// DecodeContext::decode_next_logits (decode.rs:91-127)
int orc_decode_logits(orc_cache* c, uint32_t tok, float softcap, float* logits) {
    std::vector<float> x(c->m->cfg.dim);
    int rc = orc_decode_token_from_id(c, tok, x.data());
    if (rc) return rc;
    head_dispatch(c, x.data(), logits);
    if (softcap > 0.0f)
        for (int i = 0; i < c->m->cfg.vocab; ++i) logits[i] = softcap * std::tanh(logits[i] * (1.0f / softcap));
    return 0;
}

// logits_argmax_blocks + finalize (lib.rs:1515-1565, :1725-1760)
int orc_decode_argmax_from_id(orc_cache* c, uint32_t tok, uint32_t* out) {
    const int V = c->m->cfg.vocab;
    std::vector<float> x(c->m->cfg.dim), lg(V);
    int rc = orc_decode_token_from_id(c, tok, x.data());
    if (rc) return rc;
    head_dispatch(c, x.data(), lg.data());
    float bv = -std::numeric_limits<float>::infinity();
    uint32_t bi = 0xffffffffu;
    for (int i = 0; i < V; ++i)
        if (better(lg[i], (uint32_t)i, bv, bi)) { bv = lg[i]; bi = (uint32_t)i; }
    *out = bi;
    return 0;
}

// logits_topk_blocks (lib.rs:1567-1635): per 256-row block, k rounds of argmax-and-remove.
int orc_decode_topk_from_id(orc_cache* c, uint32_t tok, int k, float* vals, uint32_t* idxs) {
    const int V = c->m->cfg.vocab;
    if (k <= 0 || k > MAX_GPU_TOPK) return -4;
    std::vector<float> x(c->m->cfg.dim), lg(V);
    int rc = orc_decode_token_from_id(c, tok, x.data());
    if (rc) return rc;
    head_dispatch(c, x.data(), lg.data());
    const int nblocks = (V + BLOCK - 1) / BLOCK;
    const float NEG = -std::numeric_limits<float>::infinity();
    for (int b = 0; b < nblocks; ++b) {
        float cand[BLOCK];
        uint32_t cidx[BLOCK];
        for (int t = 0; t < BLOCK; ++t) {
            const int row = b * BLOCK + t;
            cand[t] = row < V ? lg[row] : NEG;
            cidx[t] = row < V ? (uint32_t)row : 0xffffffffu;
        }
        for (int r = 0; r < k; ++r) {
            float bv = cand[0];
            uint32_t bi = cidx[0];
            for (int t = 1; t < BLOCK; ++t)
                if (better(cand[t], cidx[t], bv, bi)) { bv = cand[t]; bi = cidx[t]; }
            vals[b * k + r] = bv;
            idxs[b * k + r] = bi;
            for (int t = 0; t < BLOCK; ++t)
                if (cidx[t] == bi) { cand[t] = NEG; cidx[t] = 0xffffffffu; }
        }
    }
    return nblocks * k;
}

// logits_block_stats (lib.rs:1637-1700)
int orc_decode_block_stats_from_id(orc_cache* c, uint32_t tok, float inv_t, float softcap, float* maxes, float* sums) {
    const int V = c->m->cfg.vocab;
    std::vector<float> x(c->m->cfg.dim), lg(V);
    int rc = orc_decode_token_from_id(c, tok, x.data());
    if (rc) return rc;
    head_dispatch(c, x.data(), lg.data());
    const int nblocks = (V + BLOCK - 1) / BLOCK;
    for (int b = 0; b < nblocks; ++b) {
        const int r0 = b * BLOCK, r1 = std::min(V, r0 + BLOCK);
        float mx = -std::numeric_limits<float>::infinity();
        std::vector<float> z(r1 - r0);
        for (int r = r0; r < r1; ++r) {
            z[r - r0] = softcap_apply(lg[r], softcap) * inv_t;
            mx = std::max(mx, z[r - r0]);
        }
        float s = 0.0f;
        for (float zz : z) s += std::exp(zz - mx);
        maxes[b] = mx;
        sums[b] = s;
    }
    return nblocks;
}

// logits_block_materialize (lib.rs:1702-1723): from the still-resident normalised hidden.
int orc_materialize_block(orc_cache* c, int block, float softcap, float* out) {
    const orc_config& cfg = c->m->cfg;
    const int nblocks = (cfg.vocab + BLOCK - 1) / BLOCK;
    if (block < 0 || block >= nblocks) return -5;
    const int valid = std::min(BLOCK, cfg.vocab - block * BLOCK);
    for (int t = 0; t < valid; ++t) {
        const size_t row = (size_t)block * BLOCK + t;
        const std::vector<uint8_t>& hb = cfg.untied ? c->m->lm_head : c->m->embed;
        float d;
        if (cfg.dtype == ORC_F32) d = dot(as<float>(hb) + row * cfg.dim, c->norm.data(), cfg.dim);
        else if (cfg.dtype == ORC_F16) d = dot(as<f16_t>(hb) + row * cfg.dim, c->norm.data(), cfg.dim);
        else d = dot(as<bf16_t>(hb) + row * cfg.dim, c->norm.data(), cfg.dim);
        out[t] = softcap_apply(d, softcap);
    }
    return valid;
}

// ---- samplers: inference.rs:770-921
int orc_sample_softmax_index(const float* logits, int n, float t, uint64_t* rng) {  // :893-917
    float mx = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < n; ++i) mx = std::max(mx, logits[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += std::exp((logits[i] - mx) / t);
    if (!std::isfinite(sum) || sum <= 0.0f) return (int)argmax_last(logits, n);
    float draw = orc_next_f32(rng) * sum;
    for (int i = 0; i < n; ++i) {
        draw -= std::exp((logits[i] - mx) / t);
        if (draw <= 0.0f) return i;
    }
    return n > 0 ? n - 1 : 0;
}

uint32_t orc_sample_next(const float* logits, int n, float t, int top_k, uint64_t* rng) {  // :770-821
    if (t <= 0.0f || top_k == 1) return argmax_last(logits, n);
    if (top_k == 0 || top_k >= n) return (uint32_t)orc_sample_softmax_index(logits, n, t, rng);
    // sort_unstable_by(descending logit): tie order is unspecified in the reference;
    // this restatement breaks ties towards the lower index.
    std::vector<int> idx(n);
    for (int i = 0; i < n; ++i) idx[i] = i;
    std::partial_sort(idx.begin(), idx.begin() + top_k, idx.end(), [&](int a, int b) {
        return logits[a] > logits[b] || (logits[a] == logits[b] && a < b);
    });
    idx.resize(top_k);
    float mx = -std::numeric_limits<float>::infinity();
    for (int i : idx) mx = std::max(mx, logits[i]);
    float sum = 0.0f;
    for (int i : idx) sum += std::exp((logits[i] - mx) / t);
    if (!std::isfinite(sum) || sum <= 0.0f) return (uint32_t)idx[0];
    float draw = orc_next_f32(rng) * sum;
    for (int i : idx) {
        draw -= std::exp((logits[i] - mx) / t);
        if (draw <= 0.0f) return (uint32_t)i;
    }
    return (uint32_t)idx.back();
}

uint32_t orc_sample_topk_candidates(const uint32_t* idxs, const float* logits, int n, float t, uint64_t* rng) {  // :823-849
    if (n == 0) return 0;
    if (t <= 0.0f || n == 1) return idxs[0];
    float mx = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < n; ++i) mx = std::max(mx, logits[i]);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += std::exp((logits[i] - mx) / t);
    if (!std::isfinite(sum) || sum <= 0.0f) return idxs[0];
    float draw = orc_next_f32(rng) * sum;
    for (int i = 0; i < n; ++i) {
        draw -= std::exp((logits[i] - mx) / t);
        if (draw <= 0.0f) return idxs[i];
    }
    return idxs[n - 1];
}

int orc_sample_block_from_stats(const float* maxes, const float* sums, int n, uint64_t* rng) {  // :851-891
    if (n == 0) return 0;
    float gmax = -std::numeric_limits<float>::infinity();
    for (int i = 0; i < n; ++i)
        if (std::isfinite(maxes[i])) gmax = std::max(gmax, maxes[i]);
    if (!std::isfinite(gmax)) return 0;
    auto weight = [&](int i) {
        return (std::isfinite(maxes[i]) && std::isfinite(sums[i]) && sums[i] > 0.0f) ? std::exp(maxes[i] - gmax) * sums[i] : 0.0f;
    };
    float total = 0.0f;
    for (int i = 0; i < n; ++i) total += weight(i);
    if (!std::isfinite(total) || total <= 0.0f) return 0;
    float draw = orc_next_f32(rng) * total;
    for (int i = 0; i < n; ++i) {
        draw -= weight(i);
        if (draw <= 0.0f) return i;
    }
    return n - 1;
}

// decode.rs:218-253
int orc_merge_topk(const float* vals, const uint32_t* idxs, int n, int top_k, float* out_vals, uint32_t* out_idxs) {
    for (int i = 0; i < top_k; ++i) { out_vals[i] = -std::numeric_limits<float>::infinity(); out_idxs[i] = 0xffffffffu; }
    for (int j = 0; j < n; ++j) {
        const float val = vals[j];
        const uint32_t idx = idxs[j];
        if (idx == 0xffffffffu || !std::isfinite(val)) continue;
        int at = -1;
        for (int s = 0; s < top_k; ++s)
            if (val > out_vals[s] || (val == out_vals[s] && idx < out_idxs[s])) { at = s; break; }
        if (at >= 0) {
            for (int i = top_k - 1; i > at; --i) { out_vals[i] = out_vals[i - 1]; out_idxs[i] = out_idxs[i - 1]; }
            out_vals[at] = val;
            out_idxs[at] = idx;
        }
    }
    for (int i = 0; i < top_k; ++i)
        if (out_idxs[i] == 0xffffffffu) return i;
    return top_k;
}

// inference.rs:458-528
int orc_select_decode_mode(const orc_config* cfg, int backend, int ctx_len, int steps, const char** fallback, const char** autor) {
    *fallback = nullptr; *autor = nullptr;
    if (steps == 0) return ORC_MODE_PREFILL_ONLY;
    const bool window_ok = steps > 1 && ctx_len + steps <= cfg->seq;
    if (backend == ORC_BACKEND_NAIVE) return ORC_MODE_NAIVE;
    if (backend == ORC_BACKEND_KV) {
        if (window_ok) return ORC_MODE_KV;
        *fallback = steps <= 1 ? "single_step_prefers_naive" : "requested_length_exceeds_cfg_seq";
        return ORC_MODE_NAIVE;
    }
    if (!window_ok) {
        if (ctx_len + steps > cfg->seq && steps > 1) *fallback = "requested_length_exceeds_cfg_seq";
        *autor = steps <= 1 ? "single_step_prefers_naive" : "window_not_metal_eligible";
        return ORC_MODE_NAIVE;
    }
    if (orc_param_count(cfg) >= AUTO_KV_PARAM_THRESHOLD) { *autor = "model_param_count_ge_threshold"; return ORC_MODE_KV; }
    *autor = "model_param_count_lt_threshold";
    return ORC_MODE_NAIVE;
}

// ---- a whole request: generate_with_suffix (inference.rs:183-319) over
// run_naive_sample (:687-734) / run_cached_sample (:542-648).
int orc_generate(const orc_model* m, const uint32_t* prompt, int nprompt, const uint32_t* suffix, int nsuffix,
                 const orc_request* req, float softcap, int kv_round, uint32_t* out_tokens, float* trace,
                 int* out_mode) {
    const orc_config& c = m->cfg;
    const int V = c.vocab, seq = c.seq;
    if (nprompt <= 0 || req->samples <= 0) return -1;
    if (!tokens_ok(m, prompt, nprompt) || !tokens_ok(m, suffix, nsuffix)) return -2;
    const int prompt_len = std::min(nprompt, seq);
    const int eff_len = std::min(prompt_len + nsuffix, seq);
    const char *fb, *ar;
    const int mode = orc_select_decode_mode(&c, req->backend, eff_len, req->steps, &fb, &ar);
    if (out_mode) *out_mode = mode;
    const bool use_kv = mode == ORC_MODE_KV;

    std::vector<uint32_t> eff(prompt, prompt + nprompt);
    eff.insert(eff.end(), suffix, suffix + nsuffix);

    // window = last <= seq tokens (fill_input_window, inference.rs:751-757)
    auto naive_logits = [&](const std::vector<uint32_t>& ids, float* out, float* kcf, float* vcf) {
        const size_t start = ids.size() > (size_t)seq ? ids.size() - seq : 0;
        const int n = (int)(ids.size() - start);
        const int row = n - 1;
        return orc_forward_logits(m, ids.data() + start, n, softcap, kv_round, &row, 1, out, kcf, vcf, nullptr);
    };

    // InferenceSession::new: prefill over the base prompt (inference.rs:124-161)
    std::vector<float> base_logits(V), kcf, vcf;
    if (use_kv) { kcf.assign((size_t)c.nlayers * c.kv_dim * seq, 0.0f); vcf = kcf; }
    std::vector<uint32_t> base(prompt, prompt + nprompt);
    int rc = naive_logits(base, base_logits.data(), use_kv ? kcf.data() : nullptr, use_kv ? vcf.data() : nullptr);
    if (rc) return rc;

    orc_cache* cc = use_kv ? orc_cache_new(m, kv_round) : nullptr;
    auto seed_cache = [&]() {
        orc_cache_set_len(cc, prompt_len);
        for (int l = 0; l < c.nlayers; ++l)
            orc_cache_seed_cf(cc, l, prompt_len, kcf.data() + (size_t)l * c.kv_dim * seq, vcf.data() + (size_t)l * c.kv_dim * seq);
    };

    std::vector<float> prompt_logits = base_logits, lg(V);
    if (nsuffix > 0) {
        if (use_kv) {  // prefill_prompt_suffix_cached :650-670
            seed_cache();
            for (int i = 0; i < nsuffix; ++i) orc_decode_logits(cc, suffix[i], softcap, prompt_logits.data());
        } else {
            naive_logits(eff, prompt_logits.data(), nullptr, nullptr);
        }
    }

    for (int s = 0; s < req->samples; ++s) {
        uint64_t rng = req->seed + (uint64_t)s;
        uint32_t* sampled = out_tokens + (size_t)s * req->steps;
        float* tr = (trace && s == 0) ? trace : nullptr;
        std::vector<uint32_t> generated = eff;
        if (use_kv) {
            seed_cache();
            for (int i = 0; i < nsuffix; ++i) orc_decode_logits(cc, suffix[i], softcap, lg.data());
        }
        if (req->steps > 0) {
            const uint32_t next = orc_sample_next(prompt_logits.data(), V, req->temperature, req->top_k, &rng);
            if (tr) memcpy(tr, prompt_logits.data(), (size_t)V * 4);
            generated.push_back(next);
            sampled[0] = next;
        }
        for (int st = 1; st < req->steps; ++st) {
            const uint32_t cur = sampled[st - 1];
            uint32_t next;
            if (!use_kv) {
                naive_logits(generated, lg.data(), nullptr, nullptr);
                if (tr) memcpy(tr + (size_t)st * V, lg.data(), (size_t)V * 4);
                next = orc_sample_next(lg.data(), V, req->temperature, req->top_k, &rng);
            } else if (req->temperature <= 0.0f || req->top_k == 1) {
                orc_decode_argmax_from_id(cc, cur, &next);
            } else if (req->top_k > 0 && req->top_k <= MAX_GPU_TOPK) {
                const int k = std::min(std::min(req->top_k, MAX_GPU_TOPK), V);
                const int nb = (V + BLOCK - 1) / BLOCK;
                std::vector<float> vals((size_t)nb * k), mv(k);
                std::vector<uint32_t> idxs((size_t)nb * k), mi(k);
                const int count = orc_decode_topk_from_id(cc, cur, k, vals.data(), idxs.data());
                const int ml = orc_merge_topk(vals.data(), idxs.data(), count, k, mv.data(), mi.data());
                if (softcap > 0.0f)
                    for (int i = 0; i < ml; ++i) mv[i] = softcap * std::tanh(mv[i] / softcap);
                next = orc_sample_topk_candidates(mi.data(), mv.data(), ml, req->temperature, &rng);
            } else if (req->top_k == 0) {
                const int nb = (V + BLOCK - 1) / BLOCK;
                std::vector<float> mx(nb), sm(nb), bl(BLOCK);
                const float inv_t = 1.0f / std::max(req->temperature, std::numeric_limits<float>::min());
                orc_decode_block_stats_from_id(cc, cur, inv_t, softcap, mx.data(), sm.data());
                const int b = orc_sample_block_from_stats(mx.data(), sm.data(), nb, &rng);
                const int valid = orc_materialize_block(cc, b, softcap, bl.data());
                next = (uint32_t)(b * BLOCK) + (uint32_t)orc_sample_softmax_index(bl.data(), valid, req->temperature, &rng);
            } else {
                orc_decode_logits(cc, cur, softcap, lg.data());
                if (tr) memcpy(tr + (size_t)st * V, lg.data(), (size_t)V * 4);
                next = orc_sample_next(lg.data(), V, req->temperature, req->top_k, &rng);
            }
            generated.push_back(next);
            sampled[st] = next;
        }
    }
    if (cc) orc_cache_free(cc);
    return 0;
}

}  // extern "C"
