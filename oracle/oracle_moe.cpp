// CPU oracle of the MoE + MLA decoder (BASELINE configuration 5) — test infrastructure only.
//
// The reference has no MoE, no MLA and no latent KV cache (repo-wide: no router, no expert, no
// latent code), so there is nothing to restate line by line: PARITY UNPINNED, the definitions
// below are the builder's, and the CUDA path is checked against this file only.  What is kept
// from the reference is everything the two models share: RMSNorm with eps 1e-5
// (cpu/rmsnorm.rs:149-183), interleaved-pair RoPE (sdpa_fwd.rs:18-33, :258-293), the DeepNet
// residual scale alpha = 1/sqrt(2 nlayers) on both branches (layer.rs:1300, :1397), SwiGLU
// (ffn_fused.rs:114-197), the tied or untied LM head (full_model.rs:416-428), fp32 arithmetic.
//
// Definitions (per layer; D = dim, H = heads, C = kv_latent, R = rope_dim, N = nope_dim, V = v_dim):
//   xn   = rmsnorm(x, gamma1)
//   q    = xn wq                    [H (N + R)]   per head: N no-position dims, then R RoPE dims
//   c    = rmsnorm(xn wdkv, gamma_kv)  [C]        the cached latent (normalised before caching)
//   kr   = rope(xn wkr, pos)        [R]           one RoPE key shared by all heads, cached
//   k_h(t) = c(t) wuk[:, h]  [N],   v_h(t) = c(t) wuv[:, h]  [V]
//   s_h(t) = (q_nope_h . k_h(t) + rope(q_rope_h, pos) . kr(t)) / sqrt(N + R),  t <= pos
//   o_h  = sum_t softmax_t(s_h)(t) v_h(t);   x2 = x + alpha (concat_h o_h) wo
//   x2n  = rmsnorm(x2, gamma2);  p = softmax(x2n wr) over all experts;  S = the top_k largest p
//          (ties to the lower expert index); the chosen weights are NOT renormalised
//   y    = sum_{e in S} p_e FFN_e(x2n) + FFN_shared(x2n),  FFN(u) = (silu(u w1) * (u w3)) w2^T
//          (the n_shared shared experts are one FFN of n_shared * hidden columns)
//   x    = x2 + alpha y
// Weights are synthetic: element i of tensor uid is orc_synth_value(seed, uid, i) rounded to the
// storage type, uid = 0x100000 + 1024 layer + local (see enum below), logical layouts [in, out]
// row-major except the w2 matrices, which are [out, in] as in the dense model (ffn_fused.rs:8).
// Routed experts are generated the first time the router picks them.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <vector>

#include "oracle.h"

namespace {

constexpr float RMS_EPS = 1e-5f;
enum { L_WQ = 0, L_WDKV, L_WKR, L_WUK, L_WUV, L_WO, L_WR, L_WS1, L_WS3, L_WS2, L_EXPERT0 = 16 };
inline uint64_t moe_uid(int layer, int local) { return 0x100000ull + (uint64_t)layer * 1024ull + (uint64_t)local; }

// A matrix held in "output-major" form: row o holds the K inputs of output o, values already
// rounded to the storage type.
struct Mat {
    int out = 0, in = 0;
    std::vector<float> w;
    std::vector<uint16_t> b;  // bf16 bit patterns instead of w (the routed experts of a bf16 model: half the host memory)
    const float* row(int o) const { return w.data() + (size_t)o * in; }
};

// logical [in, out] (in_major) or [out, in]; element (o, i) of the result
Mat synth_mat(uint64_t seed, uint64_t uid, float std, int dtype, int in, int out, bool in_major, bool compact = false) {
    Mat m;
    m.out = out; m.in = in;
    compact = compact && dtype == ORC_BF16;
    if (compact) m.b.resize((size_t)out * in);
    else m.w.resize((size_t)out * in);
#pragma omp parallel for schedule(static)
    for (long long o = 0; o < out; ++o)
        for (int i = 0; i < in; ++i) {
            const uint64_t idx = in_major ? (uint64_t)i * out + (uint64_t)o : (uint64_t)o * in + (uint64_t)i;
            const float v = orc_round_to(orc_synth_value(seed, uid, idx, std), dtype);
            if (compact) {
                uint32_t u;
                memcpy(&u, &v, 4);
                m.b[(size_t)o * in + i] = (uint16_t)(u >> 16);  // v is exactly a bf16 value
            } else {
                m.w[(size_t)o * in + i] = v;
            }
        }
    return m;
}

inline float dotf(const float* a, const float* b, int n) {
    float acc[8] = {0};
    int i = 0;
    for (; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; ++l) acc[l] += a[i + l] * b[i + l];
    for (int l = 0; i < n; ++i, ++l) acc[l] += a[i] * b[i];
    return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

inline float dotb(const uint16_t* a, const float* b, int n) {  // the same sum over bf16 bit patterns
    float acc[8] = {0};
    int i = 0;
    auto f = [](uint16_t h) { uint32_t u = (uint32_t)h << 16; float v; memcpy(&v, &u, 4); return v; };
    for (; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; ++l) acc[l] += f(a[i + l]) * b[i + l];
    for (int l = 0; i < n; ++i, ++l) acc[l] += f(a[i]) * b[i];
    return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}
inline float rowdot(const Mat& m, int o, const float* x) {
    return m.b.empty() ? dotf(m.w.data() + (size_t)o * m.in, x, m.in) : dotb(m.b.data() + (size_t)o * m.in, x, m.in);
}

void matvec(const Mat& m, const float* x, float* y) {
#pragma omp parallel for schedule(static)
    for (int o = 0; o < m.out; ++o) y[o] = rowdot(m, o, x);
}

void rmsnorm(const float* x, const float* g, float* out, int n) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += x[i] * x[i];
    const float inv = 1.0f / std::sqrt(ss * (1.0f / (float)n) + RMS_EPS);
    for (int i = 0; i < n; ++i) out[i] = x[i] * inv * g[i];
}

void rope(float* x, int n, int pos) {  // interleaved pairs, theta = pos / 10000^(2i/n)
    for (int i = 0; i < n / 2; ++i) {
        const float theta = (float)pos / std::pow(10000.0f, 2.0f * (float)i / (float)n);
        const float c = std::cos(theta), s = std::sin(theta);
        const float e = x[2 * i], o = x[2 * i + 1];
        x[2 * i] = e * c - o * s;
        x[2 * i + 1] = o * c + e * s;
    }
}

struct Expert { Mat w1, w3, w2; };

struct MoeLayer {
    Mat wq, wdkv, wkr, wuk, wuv, wo, wr;
    Expert shared;
    std::map<int, Expert> routed;  // generated on first use
    std::vector<float> g1, g2, gkv;
};

}  // namespace

struct orc_moe_model {
    orc_moe_config cfg;
    uint64_t seed;
    float std;
    Mat embed, head;  // head is empty when tied
    std::vector<float> gfinal;
    std::vector<MoeLayer> layers;
    // cache: per layer, per position: rounded latent row [C + R], and what the heads derive from it
    int kv_dtype;
    size_t len = 0;
    std::vector<std::vector<float>> lat, kn, vv;  // [seq][C+R], [seq][H N], [seq][H V]
    std::vector<int> last_experts;                 // layer-major top_k ids of the last step
};

namespace {
const Expert& routed_expert(orc_moe_model* m, int layer, int e) {
    MoeLayer& L = m->layers[layer];
    auto it = L.routed.find(e);
    if (it != L.routed.end()) return it->second;
    const orc_moe_config& c = m->cfg;
    Expert x;
    x.w1 = synth_mat(m->seed, moe_uid(layer, L_EXPERT0 + 3 * e + 0), m->std, c.dtype, c.dim, c.hidden, true, true);
    x.w3 = synth_mat(m->seed, moe_uid(layer, L_EXPERT0 + 3 * e + 1), m->std, c.dtype, c.dim, c.hidden, true, true);
    x.w2 = synth_mat(m->seed, moe_uid(layer, L_EXPERT0 + 3 * e + 2), m->std, c.dtype, c.hidden, c.dim, false, true);
    return L.routed.emplace(e, std::move(x)).first->second;
}

void ffn(const Expert& e, const float* x, float scale, float* y_acc, std::vector<float>& h1, std::vector<float>& h3) {
    h1.resize(e.w1.out); h3.resize(e.w3.out);
    matvec(e.w1, x, h1.data());
    matvec(e.w3, x, h3.data());
    for (int j = 0; j < e.w1.out; ++j) {
        const float a = h1[j];
        h1[j] = (a / (1.0f + std::exp(-a))) * h3[j];
    }
    const int D = e.w2.out;
#pragma omp parallel for schedule(static)
    for (int o = 0; o < D; ++o) y_acc[o] += scale * rowdot(e.w2, o, h1.data());
}
}  // namespace

extern "C" {

orc_moe_model* orc_moe_synth(const orc_moe_config* c, uint64_t seed, float std) {
    if (c->top_k > c->n_experts || c->top_k <= 0 || c->heads <= 0) return nullptr;
    orc_moe_model* m = new orc_moe_model();
    m->cfg = *c; m->seed = seed; m->std = std;
    m->kv_dtype = c->dtype == ORC_F32 ? ORC_F32 : ORC_F16;
    const int D = c->dim, H = c->heads, C = c->kv_latent, R = c->rope_dim, N = c->nope_dim, V = c->v_dim;
    m->embed = synth_mat(seed, 0, std, c->dtype, D, c->vocab, false);
    if (c->untied) m->head = synth_mat(seed, 2, std, c->dtype, D, c->vocab, false);
    m->gfinal.assign(D, 1.0f);
    m->layers.resize(c->nlayers);
    for (int l = 0; l < c->nlayers; ++l) {
        MoeLayer& L = m->layers[l];
        L.wq = synth_mat(seed, moe_uid(l, L_WQ), std, c->dtype, D, H * (N + R), true);
        L.wdkv = synth_mat(seed, moe_uid(l, L_WDKV), std, c->dtype, D, C, true);
        L.wkr = synth_mat(seed, moe_uid(l, L_WKR), std, c->dtype, D, R, true);
        L.wuk = synth_mat(seed, moe_uid(l, L_WUK), std, c->dtype, C, H * N, true);
        L.wuv = synth_mat(seed, moe_uid(l, L_WUV), std, c->dtype, C, H * V, true);
        L.wo = synth_mat(seed, moe_uid(l, L_WO), std, c->dtype, H * V, D, true);
        L.wr = synth_mat(seed, moe_uid(l, L_WR), std, c->dtype, D, c->n_experts, true);
        const int SH = c->n_shared * c->hidden;
        L.shared.w1 = synth_mat(seed, moe_uid(l, L_WS1), std, c->dtype, D, SH, true);
        L.shared.w3 = synth_mat(seed, moe_uid(l, L_WS3), std, c->dtype, D, SH, true);
        L.shared.w2 = synth_mat(seed, moe_uid(l, L_WS2), std, c->dtype, SH, D, false);
        L.g1.assign(D, 1.0f); L.g2.assign(D, 1.0f); L.gkv.assign(C, 1.0f);
    }
    m->lat.resize(c->nlayers); m->kn.resize(c->nlayers); m->vv.resize(c->nlayers);
    for (int l = 0; l < c->nlayers; ++l) {
        m->lat[l].assign((size_t)c->seq * (C + R), 0.0f);
        m->kn[l].assign((size_t)c->seq * H * N, 0.0f);
        m->vv[l].assign((size_t)c->seq * H * V, 0.0f);
    }
    m->last_experts.assign((size_t)c->nlayers * c->top_k, -1);
    return m;
}

void orc_moe_free(orc_moe_model* m) { delete m; }
size_t orc_moe_len(const orc_moe_model* m) { return m->len; }
void orc_moe_set_len(orc_moe_model* m, size_t len) { m->len = std::min(len, (size_t)m->cfg.seq); }
void orc_moe_set_kv_dtype(orc_moe_model* m, int dtype) { m->kv_dtype = dtype; }

// the experts the router chose in layer `layer` during the last step, best first
int orc_moe_last_experts(const orc_moe_model* m, int layer, int32_t* out) {
    for (int k = 0; k < m->cfg.top_k; ++k) out[k] = m->last_experts[(size_t)layer * m->cfg.top_k + k];
    return m->cfg.top_k;
}

// One token at position len: appends its latent to the cache, writes [vocab] logits; returns 0 or -1 (cache full)
int orc_moe_decode_logits(orc_moe_model* m, uint32_t tok, float* logits) {
    const orc_moe_config& c = m->cfg;
    if (m->len >= (size_t)c.seq || tok >= (uint32_t)c.vocab) return -1;
    const int D = c.dim, H = c.heads, C = c.kv_latent, R = c.rope_dim, N = c.nope_dim, V = c.v_dim, QH = N + R;
    const int pos = (int)m->len;
    const float alpha = 1.0f / std::sqrt(2.0f * (float)c.nlayers);
    const float scale = 1.0f / std::sqrt((float)QH);
    std::vector<float> x(m->embed.row((int)tok), m->embed.row((int)tok) + D), xn(D), q((size_t)H * QH), craw(C), cn(C + R), kr(R);
    std::vector<float> attn((size_t)H * V), o(D), x2(D), x2n(D), r(c.n_experts), y(D), h1, h3, sc(pos + 1);
    for (int l = 0; l < c.nlayers; ++l) {
        MoeLayer& L = m->layers[l];
        rmsnorm(x.data(), L.g1.data(), xn.data(), D);
        matvec(L.wq, xn.data(), q.data());
        matvec(L.wdkv, xn.data(), craw.data());
        matvec(L.wkr, xn.data(), kr.data());
        rmsnorm(craw.data(), L.gkv.data(), cn.data(), C);
        rope(kr.data(), R, pos);
        float* row = m->lat[l].data() + (size_t)pos * (C + R);
        for (int i = 0; i < C; ++i) row[i] = orc_round_to(cn[i], m->kv_dtype);
        for (int i = 0; i < R; ++i) row[C + i] = orc_round_to(kr[i], m->kv_dtype);
        // what the heads see of this position: k_h = c wuk[:, h], v_h = c wuv[:, h] from the ROUNDED latent
        matvec(L.wuk, row, m->kn[l].data() + (size_t)pos * H * N);   // wuk as [H N outputs][C inputs]
        matvec(L.wuv, row, m->vv[l].data() + (size_t)pos * H * V);
#pragma omp parallel for schedule(static)
        for (int h = 0; h < H; ++h) {
            float* qh = q.data() + (size_t)h * QH;
            rope(qh + N, R, pos);
            std::vector<float> s(pos + 1);
            float mx = -INFINITY;
            for (int t = 0; t <= pos; ++t) {
                const float* kt = m->kn[l].data() + ((size_t)t * H + h) * N;
                const float* krt = m->lat[l].data() + (size_t)t * (C + R) + C;
                s[t] = (dotf(qh, kt, N) + dotf(qh + N, krt, R)) * scale;
                mx = std::max(mx, s[t]);
            }
            float sum = 0.0f;
            for (int t = 0; t <= pos; ++t) { s[t] = std::exp(s[t] - mx); sum += s[t]; }
            float* out = attn.data() + (size_t)h * V;
            for (int d = 0; d < V; ++d) out[d] = 0.0f;
            for (int t = 0; t <= pos; ++t) {
                const float p = s[t] / sum;
                const float* vt = m->vv[l].data() + ((size_t)t * H + h) * V;
                for (int d = 0; d < V; ++d) out[d] += p * vt[d];
            }
        }
        matvec(L.wo, attn.data(), o.data());
        for (int i = 0; i < D; ++i) x2[i] = x[i] + alpha * o[i];
        rmsnorm(x2.data(), L.g2.data(), x2n.data(), D);
        matvec(L.wr, x2n.data(), r.data());
        float rmax = -INFINITY;
        for (int e = 0; e < c.n_experts; ++e) rmax = std::max(rmax, r[e]);
        float rsum = 0.0f;
        for (int e = 0; e < c.n_experts; ++e) { r[e] = std::exp(r[e] - rmax); rsum += r[e]; }
        for (int e = 0; e < c.n_experts; ++e) r[e] /= rsum;
        std::vector<int> order(c.n_experts);
        for (int e = 0; e < c.n_experts; ++e) order[e] = e;
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return r[a] > r[b]; });  // ties: lower index first
        for (int i = 0; i < D; ++i) y[i] = 0.0f;
        for (int k = 0; k < c.top_k; ++k) {
            const int e = order[k];
            m->last_experts[(size_t)l * c.top_k + k] = e;
            ffn(routed_expert(m, l, e), x2n.data(), r[e], y.data(), h1, h3);
        }
        ffn(L.shared, x2n.data(), 1.0f, y.data(), h1, h3);
        for (int i = 0; i < D; ++i) x[i] = x2[i] + alpha * y[i];
    }
    rmsnorm(x.data(), m->gfinal.data(), xn.data(), D);
    const Mat& head = c.untied ? m->head : m->embed;
    matvec(head, xn.data(), logits);
    m->len += 1;
    return 0;
}

}  // extern "C"
