/*
 * CPU oracle for the rustane autoregressive token loop — TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain fp32 restatement, on the host, of the two reference paths the
 * CUDA library must agree with:
 *   - `naive_full_context`: crates/engine/src/full_model.rs:336-437 driving
 *     crates/engine/src/layer.rs:1287-1431 (whose attention / Wo / FFN math is
 *     defined by kernels/sdpa_fwd.rs:69-404, kernels/dyn_matmul.rs:400-434 and
 *     kernels/ffn_fused.rs:21-203), and
 *   - the KV-cached single-token decode: crates/metal-decode/src/lib.rs:513-634
 *     (layer sequencing) and :1354-1760 (kernel bodies),
 * plus the samplers / LCG of crates/engine/src/inference.rs:759-921, the top-k
 * merge of crates/engine/src/decode.rs:218-253 and the backend policy of
 * inference.rs:458-528.
 *
 * PARITY UNPINNED for the transformer-layer math: the reference holds no golden
 * vectors for it (its attention/FFN run inside Apple's ANE and its tests check
 * shapes only).  What the reference does pin — RMSNorm and embedding known
 * answers, the RSTK round trip, the backend policy table, the merge/tie rules —
 * is replayed against this file by tests/test_oracle_pins.py.
 *
 * Nothing in the shipped library may include, link or call this code.
 */
#ifndef RUSTANE_ORACLE_H
#define RUSTANE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2 };
enum { ORC_QUANT_FP8 = 3, ORC_QUANT_INT4 = 4 }; /* same numbering as the library's dtype codes */
enum { ORC_ACT_SWIGLU = 0, ORC_ACT_LEAKY_RELU_SQ = 1 };
enum { ORC_BACKEND_AUTO = 0, ORC_BACKEND_NAIVE = 1, ORC_BACKEND_KV = 2 };
enum { ORC_MODE_PREFILL_ONLY = 0, ORC_MODE_NAIVE = 1, ORC_MODE_KV = 2 };

typedef struct orc_config {
    int32_t dim, hidden, heads, kv_heads, hd, seq, nlayers, vocab;
    int32_t q_dim, kv_dim, gqa_ratio;
    int32_t activation; /* ORC_ACT_* */
    int32_t dtype;      /* storage type of matrices (values are exactly representable) */
    int32_t untied;     /* 1: separate lm_head[V,D]; 0: logits use the embedding table */
} orc_config;

typedef struct orc_request {
    int32_t backend; /* ORC_BACKEND_* */
    int32_t steps;
    float temperature;
    int32_t top_k;
    int32_t samples;
    uint64_t seed;
} orc_request;

typedef struct orc_model orc_model;
typedef struct orc_cache orc_cache;

/* ---- small pinned primitives ---- */
float orc_rmsnorm(const float* x, const float* gamma, float* out, int n); /* returns rms_inv */
void orc_embedding(const float* table, int dim, const uint32_t* ids, int n, float* out);
uint64_t orc_next_u64(uint64_t* state);
float orc_next_f32(uint64_t* state);
void orc_reference_random_vec(float* out, size_t n, float scale);
float orc_round_to(float v, int dtype);

/* ---- deterministic synthetic tensors (spec shared with the library, restated here) ---- */
float orc_synth_value(uint64_t seed, uint64_t tensor_uid, uint64_t idx, float std);
void orc_synth_prompt(uint64_t seed, int vocab, uint32_t* ids, int n);

/* ---- models ---- */
orc_model* orc_model_synth(const orc_config* cfg, uint64_t seed, float std);
orc_model* orc_model_reference_random(const orc_config* cfg); /* ModelWeights::random */
/* quantise-dequantise a matrix in place; in_major: 1 = [in, out] (wq..w3), 0 = [out, in] (w2) */
void orc_quant_dequant(float* w, int in, int out, int in_major, int mode);
/* synthetic model with quantised linears (cfg->dtype must be ORC_F32; see oracle.cpp) */
orc_model* orc_model_synth_quant(const orc_config* cfg, uint64_t seed, float std, int mode);
orc_model* orc_model_load(const char* path, char* err, int errlen);
int orc_model_save(const orc_model* m, const char* path, int version);
void orc_model_free(orc_model* m);
void orc_model_get_config(const orc_model* m, orc_config* out);
/* what kv_round = 1 rounds cached keys and values to (ORC_F32 / F16 / BF16); default: fp32 for an
 * fp32 model, fp16 otherwise, which is the library's default cache type */
void orc_model_set_kv_dtype(orc_model* m, int dtype);
size_t orc_param_count(const orc_config* cfg);
/* tensor access for building the CUDA model from the same values.
 * which: 0 embed, 1 gamma_final, 2 lm_head, 10+ per layer: wq wk wv wo w1 w3 w2 gamma1 gamma2 */
size_t orc_model_tensor(const orc_model* m, int layer, int which, float* out, size_t cap);

/* ---- naive_full_context ---- */
/* tokens: npos ids (positions >= npos are never computed: causality makes the
 * first npos rows independent of the reference's zero padding).  logits_rows
 * receives nrows rows of [vocab]; k_cf / v_cf (optional) receive per layer a
 * channel-first [kv_dim, seq] block as the reference's ForwardCache holds it. */
int orc_forward_logits(const orc_model* m, const uint32_t* tokens, int npos, float softcap,
                       int kv_round, const int* rows, int nrows, float* logits_rows,
                       float* k_cf, float* v_cf, float* x_prenorm_last);

/* ---- KV-cached decode (restates the Metal model) ---- */
orc_cache* orc_cache_new(const orc_model* m, int kv_round);
void orc_cache_free(orc_cache* c);
size_t orc_cache_len(const orc_cache* c);
void orc_cache_set_len(orc_cache* c, size_t len);
void orc_cache_seed_cf(orc_cache* c, int layer, size_t live_len, const float* k_cf,
                       const float* v_cf);
int orc_decode_token(orc_cache* c, const float* x_in, float* x_out);
int orc_decode_token_from_id(orc_cache* c, uint32_t tok, float* x_out);
int orc_decode_logits(orc_cache* c, uint32_t tok, float softcap, float* logits);
int orc_decode_argmax_from_id(orc_cache* c, uint32_t tok, uint32_t* out);
int orc_decode_topk_from_id(orc_cache* c, uint32_t tok, int k, float* vals, uint32_t* idxs);
int orc_decode_block_stats_from_id(orc_cache* c, uint32_t tok, float inv_t, float softcap,
                                   float* maxes, float* sums);
int orc_materialize_block(orc_cache* c, int block, float softcap, float* out);

/* ---- samplers, merge, policy ---- */
uint32_t orc_sample_next(const float* logits, int n, float t, int top_k, uint64_t* rng);
uint32_t orc_sample_topk_candidates(const uint32_t* idxs, const float* logits, int n, float t,
                                    uint64_t* rng);
int orc_sample_block_from_stats(const float* maxes, const float* sums, int n, uint64_t* rng);
int orc_sample_softmax_index(const float* logits, int n, float t, uint64_t* rng);
int orc_merge_topk(const float* vals, const uint32_t* idxs, int n, int top_k, float* out_vals,
                   uint32_t* out_idxs);
/* reasons are returned as static strings or NULL */
int orc_select_decode_mode(const orc_config* cfg, int backend, int ctx_len, int steps,
                           const char** fallback_reason, const char** auto_reason);

/* ---- whole request (run_naive_sample / run_cached_sample) ----
 * out_tokens: samples * steps sampled ids; trace_logits (optional): for sample 0,
 * steps rows of [vocab] = the logits each token was drawn from (naive and the
 * full-logits cached paths only; rows stay untouched otherwise). */
int orc_generate(const orc_model* m, const uint32_t* prompt, int nprompt, const uint32_t* suffix,
                 int nsuffix, const orc_request* req, float softcap, int kv_round,
                 uint32_t* out_tokens, float* trace_logits, int* out_mode);

/* ---- MoE + MLA decoder (BASELINE configuration 5; oracle_moe.cpp).  No reference counterpart: the
 * definitions are the builder's and are written out at the top of oracle_moe.cpp.  PARITY UNPINNED. */
typedef struct orc_moe_config {
    int32_t dim, hidden, heads, seq, nlayers, vocab;
    int32_t n_experts, top_k, n_shared;         /* routed experts, experts per token, shared experts (each `hidden` columns) */
    int32_t kv_latent, rope_dim, nope_dim, v_dim; /* MLA: cached latent width, decoupled RoPE width, per-head no-position and value widths */
    int32_t dtype;                               /* ORC_F32 or ORC_BF16 */
    int32_t untied;
} orc_moe_config;
typedef struct orc_moe_model orc_moe_model;
orc_moe_model* orc_moe_synth(const orc_moe_config* cfg, uint64_t seed, float std);
void orc_moe_free(orc_moe_model* m);
size_t orc_moe_len(const orc_moe_model* m);
void orc_moe_set_len(orc_moe_model* m, size_t len);
void orc_moe_set_kv_dtype(orc_moe_model* m, int dtype);
int orc_moe_decode_logits(orc_moe_model* m, uint32_t tok, float* logits);
int orc_moe_last_experts(const orc_moe_model* m, int layer, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif
