/*
 * cuda_decode — C ABI of the B200 (sm_100a) token-loop backend for rustane.
 *
 * The entry points mirror, one for one, the public methods of
 * `metal_decode::Model` (crates/metal-decode/src/lib.rs:129-511), which is the
 * only interface `engine::decode::DecodeContext` (crates/engine/src/decode.rs:14-197)
 * calls; each declaration cites the method it replaces.  Additive entry points
 * (prefill, multi-step on-device loops, checkpoint / synthetic construction,
 * session and policy helpers) follow in their own sections.
 *
 * Conventions: plain pointers and sizes only; the caller owns every host
 * buffer; the model copies weights at construction and owns all device memory.
 * Every function returns CD_OK (0) or a negative cd_status — nothing panics or
 * aborts across this boundary (the reference asserts; a binding maps non-zero
 * to the same messages via cd_last_error).  A handle is not thread-safe, like
 * the reference's `&mut self`.  There is no CPU fallback: without a usable
 * CUDA device construction fails with CD_ERR_CUDA.
 */
#ifndef CUDA_DECODE_H
#define CUDA_DECODE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cd_status {
    CD_OK = 0,
    CD_ERR_INVALID = -1,   /* bad argument / shape (reference: assert!, or None from Model::new); also returned by an on-device
                            * loop whose arg-max had no winner (logits without a finite maximum): the id it stored is not a
                            * vocabulary row, the next step used row 0 instead of it, and the ids returned are not meaningful */
    CD_ERR_SEQ_FULL = -2,  /* "metal decode only supports lengths within cfg.seq" */
    CD_ERR_TOKEN = -3,     /* "token id must fit vocab for metal decode" */
    CD_ERR_CAPACITY = -4,  /* caller buffer too small */
    CD_ERR_CUDA = -5,      /* a CUDA call failed; text in cd_last_error */
    CD_ERR_IO = -6,        /* checkpoint file problems (io::Error in checkpoint.rs) */
    CD_ERR_DEVICE_WAIT = -7, /* a bounded device-side wait ran out (cd_last_error says which) */
    CD_ERR_UNSUPPORTED = -8
} cd_status;

enum { CD_DTYPE_F32 = 0, CD_DTYPE_F16 = 1, CD_DTYPE_BF16 = 2,
       /* quantised linears (no reference counterpart): the seven per-layer matrices are
          quantised when the model is built; embedding and LM head stay bf16, gammas fp32.
          FP8: e4m3 with one fp32 scale per output channel (max|row| / 448).  INT4: symmetric,
          groups of 32 along the input, values -8..7, fp16 scale (max|group| / 7).  Under tensor
          parallelism every rank quantises its shard with the scales of the unsharded matrix. */
       CD_DTYPE_FP8_E4M3 = 3, CD_DTYPE_INT4_G32 = 4 };
enum { CD_ACT_SWIGLU = 0, CD_ACT_LEAKY_RELU_SQ = 1 }; /* model.rs:4-24 checkpoint codes */
enum { CD_BACKEND_AUTO = 0, CD_BACKEND_NAIVE = 1, CD_BACKEND_CUDA = 2 }; /* inference.rs:11-35 */
enum { CD_MODE_PREFILL_ONLY = 0, CD_MODE_NAIVE_FULL_CONTEXT = 1, CD_MODE_KV_CACHE_CUDA = 2 }; /* :37-52 */

#define CD_MAX_GPU_TOPK 32 /* metal-decode/src/lib.rs:15 */
#define CD_HEAD_BLOCK 256  /* vocab rows per block: lib.rs:156, inference.rs:613 */

/* metal_decode::Config, lib.rs:22-35 (same fields, same meaning). */
typedef struct cd_config {
    int32_t dim, hidden, heads, kv_heads, hd, seq, nlayers, vocab;
    int32_t q_dim, kv_dim, gqa_ratio;
} cd_config;

/* metal_decode::LayerInit, lib.rs:37-47.  fp32 host tensors in the reference's
 * layouts: wq/wk/wv/w1/w3 are [in=dim, out] row-major, wo is [q_dim, dim],
 * w2 is [dim, hidden]. */
typedef struct cd_layer_init {
    const float *wq, *wk, *wv, *wo, *w1, *w3, *w2, *gamma1, *gamma2;
} cd_layer_init;

/* metal_decode::FinalHeadInit, lib.rs:49-52.  lm_head == NULL means the tied
 * head of the reference (logits use the embedding table). */
typedef struct cd_head_init {
    const float *gamma_final, *embed, *lm_head;
} cd_head_init;

/* KV-cache storage, independent of the weight storage.  AUTO: fp32 weights keep an fp32 cache (as the
 * reference's, lib.rs:1027-1053), fp16 weights an fp16 cache, and bf16 / FP8 / INT4 models an fp16
 * cache too: the same two bytes as bf16 with three more mantissa bits, and post-RoPE keys and
 * values are nowhere near fp16's range. */
enum { CD_KV_AUTO = 0, CD_KV_F32 = 1, CD_KV_F16 = 2, CD_KV_BF16 = 3 };

/* What the reference has no field for.  Zero-initialise for reference behaviour
 * (fp32 storage, SwiGLU, current device, single GPU). */
typedef struct cd_options {
    int32_t weight_dtype; /* CD_DTYPE_*: storage of the matrices (embedding / LM head are bf16 for the quantised kinds) */
    int32_t activation;   /* CD_ACT_* */
    int32_t device;       /* CUDA ordinal; -1 = current */
    int32_t page_tokens;  /* KV page size in tokens; 0 = 64 */
    int32_t max_samples;  /* sequences that may share a prefill; 0 = 1 */
    int32_t use_graph;    /* 1: replay one captured CUDA graph per token */
    int32_t kv_dtype;     /* CD_KV_* */
    int32_t tp_rank;      /* tensor parallelism: this process holds shard tp_rank ... */
    int32_t tp_world;     /* ... of a model split over tp_world GPUs (0 or 1 = single GPU) */
    int32_t wait_us;      /* bound, in microseconds, of every device-side wait on a peer GPU; 0 = 2,000,000 */
    /* Test-only knobs; leave zero.  test_flags bit 0: no programmatic dependent launch; bit 1: one kernel per
     * operator even where the one-kernel-per-token path applies; bit 2: keep phase time stamps of that path
     * (cd_debug_phase_trace); bit 3: on the kernel-per-operator path the first CTA of every streamed GEMV withholds
     * its last ring stage and its consumers wait for it only briefly, so the bounded wait runs out: every token call
     * of such a model returns CD_ERR_DEVICE_WAIT (the expiry path is exercised without a fault); test_ring_kb: shared
     * memory of a GEMV CTA. */
    int32_t test_flags;
    int32_t test_ring_kb;
} cd_options;

typedef struct cd_model cd_model;

/* ---------------------------------------------------------------- the reference's methods */

/* Model::new, lib.rs:147-207 (None -> CD_ERR_*). */
int cd_model_create(const cd_config* cfg, const cd_layer_init* layers, int nlayers,
                    const cd_head_init* head, const cd_options* opts, cd_model** out);
void cd_model_destroy(cd_model* m);
/* text of the last failure on this handle (NULL handle: last construction failure) */
const char* cd_last_error(const cd_model* m);

/* Model::len / Model::set_len (clamped to seq), lib.rs:209-215. */
int cd_len(const cd_model* m, size_t* len);
int cd_set_len(cd_model* m, size_t len);

/* Model::seed_layer_cache_from_channel_first, lib.rs:217-237: k_rope_cf and v_cf
 * are [kv_dim, seq] channel-first fp32; rows >= live_len are zeroed. */
int cd_seed_layer_cache_cf(cd_model* m, int layer, size_t live_len, const float* k_rope_cf,
                           const float* v_cf);

/* Model::decode_token, lib.rs:239-269: x_in -> layers -> x_out (both [dim]). */
int cd_decode_token(cd_model* m, const float* x_in, float* x_out);
/* Model::decode_token_from_id, lib.rs:271-304. */
int cd_decode_token_from_id(cd_model* m, uint32_t token, float* x_out);
/* Model::decode_token_argmax, lib.rs:306-338. */
int cd_decode_token_argmax(cd_model* m, const float* x_in, uint32_t* out_token);
/* Model::decode_token_argmax_from_id, lib.rs:340-375. */
int cd_decode_token_argmax_from_id(cd_model* m, uint32_t token, uint32_t* out_token);
/* Model::decode_token_topk_from_id, lib.rs:377-434: writes nblocks*top_k (val, idx)
 * pairs block-major; *count = nblocks*top_k. */
int cd_decode_token_topk_from_id(cd_model* m, uint32_t token, size_t top_k, float* out_vals,
                                 uint32_t* out_idxs, size_t cap, size_t* count);
/* Model::decode_token_block_stats_from_id, lib.rs:436-487. */
int cd_decode_token_block_stats_from_id(cd_model* m, uint32_t token, float inv_temperature,
                                        float softcap, float* out_maxes, float* out_sums,
                                        size_t cap, size_t* nblocks);
/* Model::materialize_current_logits_block, lib.rs:489-511 (does not advance len). */
int cd_materialize_current_logits_block(cd_model* m, size_t block_idx, float softcap,
                                        float* out_logits, size_t cap, size_t* valid);

/* ---------------------------------------------------------------- additive: construction */

/* Stream an RSTK checkpoint (v1/v2 as checkpoint.rs:25-209 reads them; v3 adds
 * hidden/heads/kv_heads/hd/dtype/untied) into HBM.  opts->weight_dtype < 0 keeps
 * the file's dtype.  cfg_out (optional) receives the parsed configuration. */
int cd_model_create_from_checkpoint(const char* path, const cd_options* opts, cd_config* cfg_out,
                                    cd_model** out);
/* Parse and validate a checkpoint header on the host (no GPU).  meta[4] receives
 * version, dtype, activation code, flags (bit0 untied head, bit1 quantised linears).  Errors carry the messages of
 * checkpoint.rs:30-155 in cd_last_error(NULL). */
int cd_checkpoint_info(const char* path, cd_config* cfg_out, int32_t* meta);
/* Seeded random-init weights generated directly in HBM (counter-based generator:
 * element i of tensor uid is a pure function of (seed, uid, i)); gammas are 1. */
int cd_model_create_synthetic(const cd_config* cfg, const cd_options* opts, uint64_t seed,
                              float std, int untied_head, cd_model** out);
/* host-side values of the same generator, for writing identical checkpoints */
float cd_synth_value(uint64_t seed, uint64_t tensor_uid, uint64_t idx, float std);
void cd_synth_prompt(uint64_t seed, int vocab, uint32_t* ids, int n);
/* Write a seeded checkpoint file (RSTK v3; v2 when the shape allows and version==2). */
int cd_write_synthetic_checkpoint(const char* path, const cd_config* cfg, int dtype, int activation,
                                  int untied_head, uint64_t seed, float std, int version);
/* Quantised checkpoints (no reference counterpart: the reference stores fp32 only, checkpoint.rs:25-209).
 * RSTK v3 with flags bit1 and dtype code CD_DTYPE_FP8_E4M3 / CD_DTYPE_INT4_G32 stores the seven linears of
 * every layer already quantised, as rows in GEMV orientation ([out][in]: wq, wk, wv rows of dim inputs, wo
 * rows of heads * hd inputs, w1, w3 rows of dim inputs, w2 rows of hidden inputs) in the row format the
 * kernels read - FP8: `in` E4M3 codes, the row's fp32 scale, 12 bytes of padding; INT4: in / 2 bytes of
 * nibbles, in / 32 fp16 group scales, padding to 16 bytes - the embedding and an untied head as bf16, the
 * gammas as fp32.  cd_model_create_from_checkpoint streams such a file into HBM without converting
 * anything (a tensor-parallel rank takes its rows, and of wo / w2 its columns with the whole row's scale);
 * cd_checkpoint_info reports flags bit1 in meta[3] (bit0: untied head).
 * cd_convert_checkpoint: read any RSTK file, quantise on `device` (-1: current), write the quantised file.
 * cd_model_save_quantised: the same from a live single-GPU dense model whose linears are quantised.
 * cd_model_get_linear_rows: this rank's rows of one linear (0 wq .. 6 w2) of a quantised model, as stored
 * on the device, for inspection and tests. */
int cd_convert_checkpoint(const char* src_path, const char* dst_path, int quant_dtype, int device);
int cd_model_save_quantised(cd_model* m, const char* path);
int cd_model_get_linear_rows(cd_model* m, int layer, int which, void* out, size_t cap);
int cd_model_get_config(const cd_model* m, cd_config* cfg, cd_options* opts, int* untied_head);

/* ---------------------------------------------------------------- additive: MoE + MLA decoder
 * A mixture-of-experts FFN behind multi-head latent attention.  No counterpart in the reference (it
 * has no router, no expert and no latent-cache code): the model is defined here.  Per layer, with
 * xn = rmsnorm(x, gamma1):
 *   q = xn wq (heads x (nope_dim + rope_dim));  c = rmsnorm(xn wdkv, gamma_kv) (kv_latent wide) and
 *   kr = rope(xn wkr) (rope_dim wide, shared by the heads) are what the cache keeps per position;
 *   k_h(t) = c(t) wuk[:, h], v_h(t) = c(t) wuv[:, h];  score_h(t) = (q_nope_h . k_h(t) +
 *   rope(q_rope_h) . kr(t)) / sqrt(nope_dim + rope_dim);  x2 = x + alpha (softmax-weighted v) wo;
 *   p = softmax(rmsnorm(x2, gamma2) wr) over all n_experts, the top_k largest (ties: lower index) are
 *   used with their p unchanged (no renormalisation);  x = x2 + alpha (sum p_e FFN_e + FFN_shared),
 *   FFN = SwiGLU of `hidden` columns per routed expert and n_shared * hidden for the shared one;
 *   alpha = 1/sqrt(2 nlayers), RoPE pairs and RMSNorm as in the dense model.
 * cd_config describes the common part: dim, hidden = one expert's columns, heads, kv_heads = 1,
 * hd = nope_dim + rope_dim, q_dim = heads * hd, kv_dim = kv_latent + rope_dim, gqa_ratio = heads.
 * Limits: heads <= 16, kv_latent <= 512; weights f32 / f16 / bf16.  Every call that takes a cd_model
 * works on the handle except cd_seed_layer_cache_cf and cd_decode_steps_samples (CD_ERR_UNSUPPORTED;
 * the session then runs the samples one after the other); the prompt goes one token at a time.
 * Expert parallel: opts->tp_world ranks each hold n_experts / tp_world routed experts and
 * 1 / tp_world of the shared FFN's columns; attention, router and LM head are replicated; the ranks'
 * partial FFN sums are combined by the push all-reduce of the tensor-parallel path (connect the
 * ranks with cd_tp_region_handle / cd_tp_connect as there). */
typedef struct cd_moe_config {
    int32_t n_experts, top_k, n_shared;
    int32_t kv_latent, rope_dim, nope_dim, v_dim;
} cd_moe_config;
int cd_moe_model_create_synthetic(const cd_config* cfg, const cd_moe_config* moe, const cd_options* opts, uint64_t seed,
                                  float std, int untied_head, cd_model** out);
/* What rank `rank` of `world` holds under expert parallelism (host only, no GPU): routed experts
 * expert_first .. + expert_count and columns shared_first .. + shared_cols of the shared FFN. */
int cd_moe_shard_plan(const cd_config* cfg, const cd_moe_config* moe, int world, int rank, int32_t* expert_first,
                      int32_t* expert_count, int32_t* shared_first, int32_t* shared_cols);
/* the experts the router chose in `layer` at the last decoded position, best first (top_k ids) */
int cd_moe_last_experts(cd_model* m, int layer, int32_t* out_ids, size_t cap);

/* ---------------------------------------------------------------- additive: tensor parallelism
 * One process per GPU.  Create each rank's model with opts->tp_world = world size (2, 4 or 8)
 * and opts->tp_rank = rank: it keeps heads/world attention heads, hidden/world FFN columns
 * and a contiguous range of LM-head rows; the residual stream is replicated.  Exchange the 64-byte
 * handles of cd_tp_region_handle between the ranks (any transport), pass all of them, in rank
 * order, to cd_tp_connect, and then drive every rank with the same calls.  The two [dim]
 * all-reduces per layer are push-based peer stores fused into the GEMV kernels.  Supported
 * on a tensor-parallel model: cd_prefill (without logits), cd_decode_token_argmax_from_id,
 * cd_decode_token_topk_from_id (every rank returns all ranks' per-block candidates, in block order),
 * cd_decode_steps_greedy, cd_decode_steps_topk (the ranks exchange their per-block candidates and draw the
 * same token), cd_decode_steps_fullvocab (the ranks exchange per-block (max, sum); the rank that owns the
 * chosen block draws the token); the rest return CD_ERR_UNSUPPORTED. */
/* What rank `rank` of `world` holds (host only, no GPU): the per-rank config and its LM-head rows. */
int cd_tp_shard_plan(const cd_config* cfg, int world, int rank, cd_config* local, int32_t* vocab_first,
                     int32_t* vocab_rows);
int cd_tp_region_handle(cd_model* m, void* out_handle, size_t cap);
int cd_tp_connect(cd_model* m, const void* handles, int world);
/* The same for ranks that live in ONE process (one host thread per GPU, peer access enabled by the
 * caller): the link regions are exchanged as device pointers instead of IPC handles. */
int cd_tp_region_ptr(cd_model* m, void** out_region);
int cd_tp_connect_ptrs(cd_model* m, void* const* regions, int world);
/* Every wait of a rank on its peers is bounded by cd_options.wait_us; when one runs out the call
 * returns CD_ERR_DEVICE_WAIT (later waits of the same call return at once), the cache length is
 * not advanced and the handle stays valid.  The ranks' exchange counters are then out of step:
 * destroy the models of all ranks and build them again before decoding further. */

/* ---------------------------------------------------------------- additive: token loop on device */

/* DecodeContext::decode_next_logits, decode.rs:91-127, with the final norm and the
 * LM head on the GPU: token -> [vocab] logits (softcap applied when > 0). */
int cd_decode_token_logits_from_id(cd_model* m, uint32_t token, float softcap, float* out_logits);

/* Prefill n prompt tokens starting at the current len; last_logits (optional,
 * [vocab]) receives the logits of the last prompt position — what
 * InferenceSession::new (inference.rs:124-161) keeps of its forward pass.  With n >= 8 on a
 * bf16 / fp16 / FP8 single-GPU model the tokens are processed together (tensor-core GEMMs,
 * K and V written into the decode pages); otherwise one at a time as
 * prefill_prompt_suffix_cached does (inference.rs:650-670).  The first batched call
 * allocates a workspace that grows with the longest prompt seen. */
int cd_prefill(cd_model* m, const uint32_t* ids, size_t n, float softcap, float* last_logits);

/* run_cached_sample's three hot loops (inference.rs:576-625) without a host round
 * trip per token: feed first_token, produce nsteps further tokens.  Only token
 * ids cross the boundary.  rng_state is the sample's LCG state (inference.rs:759),
 * updated in place. */
int cd_decode_steps_greedy(cd_model* m, uint32_t first_token, size_t nsteps, uint32_t* out_ids);
int cd_decode_steps_topk(cd_model* m, uint32_t first_token, size_t nsteps, size_t top_k,
                         float temperature, float softcap, uint64_t* rng_state, uint32_t* out_ids);
int cd_decode_steps_fullvocab(cd_model* m, uint32_t first_token, size_t nsteps, float temperature,
                              float softcap, uint64_t* rng_state, uint32_t* out_ids);

/* Several samples continuing the cached prompt together (`--samples N`; the reference runs them one
 * after the other, inference.rs:255-297, re-seeding the cache for each).  Sample s feeds
 * first_tokens[s] at position len and then draws nsteps tokens with its own LCG state
 * rng_states[s] exactly as cd_decode_steps_{greedy,topk,fullvocab} would for that sample alone;
 * all samples advance one token per step, so the weights are read once per step for all of them.
 * Prompt pages are shared, the page the prompt ends in is copied per sample.  out_ids is
 * [nsamples][nsteps]; rng_states (may be NULL for greedy) is updated; len is left at the prompt
 * length.  nsamples <= min(16, cd_options.max_samples); bf16 / fp16 single-GPU models. */
enum { CD_SAMPLES_GREEDY = 0, CD_SAMPLES_TOPK = 1, CD_SAMPLES_FULLVOCAB = 2 };
int cd_decode_steps_samples(cd_model* m, const uint32_t* first_tokens, size_t nsamples, size_t nsteps, int mode, size_t top_k,
                            float temperature, float softcap, uint64_t* rng_states, uint32_t* out_ids);

/* Measurement aid: run ONE greedy step with a CUDA event behind every kernel and
 * return device milliseconds and launch counts per kernel class:
 * 0 misc (state, embed), 1 qkv GEMV, 2 attention, 3 wo GEMV, 4 w1|w3 GEMV, 5 w2 GEMV,
 * 6 LM-head GEMV, 7 head reduction / sampler.  Advances len by one. */
int cd_profile_decode_step(cd_model* m, uint32_t token, float* ms_by_class, uint32_t* launches_by_class,
                           size_t nclasses);
/* Measurement aid for the one-kernel-per-token path: globaltimer stamps (ns) taken by the
 * first and the last CTA at every phase boundary of the most recent token; only when the
 * model was created with CD_TRACE=1 in the environment.  Layout: 2 x (1 + 10*nlayers + 1). */
int cd_debug_phase_trace(cd_model* m, unsigned long long* out, size_t cap, size_t* n);
/* device time of the last cd_decode_steps_* / cd_prefill call, from CUDA events */
int cd_last_device_ms(const cd_model* m, float* ms);
/* kernels launched by this handle so far (graph replays count their nodes) */
int cd_kernel_launches(const cd_model* m, uint64_t* n);

/* ---------------------------------------------------------------- additive: single operators */

/* sdpa_causal (metal-decode/src/lib.rs:1426-1489) for one query token on caller data,
 * through the split-K flash-decode kernel the model uses.  Host buffers: q [heads*hd]
 * fp32; k and v [attn_len, kv_heads*hd] row-major in `dtype`; out [heads*hd] fp32.
 * nsplit <= 0 picks the model's rule (one slice per 64-token page, at most 32).
 * Allocates and frees its device buffers and scratch on every call. */
int cd_flash_decode(int dtype, int heads, int kv_heads, int hd, size_t attn_len, int nsplit,
                    const float* q, const void* k, const void* v, float* out);

/* No counterpart in the reference.  cd_flash_decode for callers that must not allocate
 * device memory: an engine whose own arena already owns all of HBM, a latency-critical
 * thread that cannot take cudaMalloc's device-wide synchronisation, a plug-in host that
 * forbids driver allocations after start-up.  Inputs and outputs are DEVICE pointers the
 * caller owns: d_q [heads*hd] fp32; d_kv_pages in the cache layout
 * [page][2 (k,v)][kv_heads][page_tokens][hd] of `dtype`; d_page_table [ceil(attn_len /
 * page_tokens)] int32 (logical -> physical page); d_out [heads*hd] fp32.  The kernel's
 * scratch is a fixed array inside the library (about 1.1 MB, held by every GPU that loads
 * the library until exit), so the call makes no cudaMalloc / cudaFree / allocating library
 * call.  Limits: heads <= 64, slices <= 32, hd <= 128; beyond them CD_ERR_UNSUPPORTED.
 * The work is enqueued on `stream` (a cudaStream_t, NULL = default stream) and not
 * synchronised.  Every call shares the one scratch array: calls whose kernels overlap on
 * the GPU race and must be serialised by the caller.  The first call on a device resolves
 * the array's address; make it before any stream capture begins.  attn_len is limited to 2^24.
 * Failures of this call are reported through cd_last_error(NULL), which is per host thread. */
int cd_flash_decode_static(int dtype, int heads, int kv_heads, int hd, size_t attn_len, int nsplit,
                           int page_tokens, const float* d_q, const void* d_kv_pages,
                           const int* d_page_table, float* d_out, void* stream);

/* ---------------------------------------------------------------- additive: host policy / samplers
 * (no device work; usable without a GPU) */

typedef struct cd_request { /* GenerationRequest, inference.rs:61-82 */
    int32_t decode_backend; /* CD_BACKEND_* */
    int32_t steps;
    float temperature;
    int32_t top_k;
    int32_t samples;
    uint64_t seed;
} cd_request;

typedef struct cd_selection { /* DecodeSelection, inference.rs:54-59 */
    int32_t mode;
    const char* fallback_reason;
    const char* auto_reason;
} cd_selection;

size_t cd_param_count(const cd_config* cfg);                /* model.rs:182-187 */
int cd_select_decode_mode(const cd_config* cfg, int backend, size_t effective_context_len,
                          size_t steps, cd_selection* out);  /* inference.rs:458-528 */
const char* cd_backend_name(int backend);                    /* "auto" | "naive" | "cuda" */
int cd_backend_parse(const char* raw);                       /* -1 when unknown */
const char* cd_mode_name(int mode);
uint64_t cd_lcg_next_u64(uint64_t* state);                   /* inference.rs:759-764 */
float cd_lcg_next_f32(uint64_t* state);                      /* inference.rs:766-768 */
uint32_t cd_sample_next(const float* logits, size_t n, float temperature, size_t top_k,
                        uint64_t* rng);                      /* inference.rs:770-821 */
uint32_t cd_sample_topk_candidates(const uint32_t* idxs, const float* logits, size_t n,
                                   float temperature, uint64_t* rng); /* :823-849 */
size_t cd_sample_block_from_stats(const float* maxes, const float* sums, size_t n,
                                  uint64_t* rng);            /* :851-891 */
size_t cd_sample_softmax_index(const float* logits, size_t n, float temperature,
                               uint64_t* rng);               /* :893-917 */
size_t cd_merge_topk_candidates(const float* vals, const uint32_t* idxs, size_t n, size_t top_k,
                                float* out_vals, uint32_t* out_idxs); /* decode.rs:218-253 */

/* ---------------------------------------------------------------- additive: InferenceSession
 * inference.rs:105-451 restated over a cd_model. */

typedef struct cd_session cd_session;

typedef struct cd_sample_result { /* SampleResult, inference.rs:84-90 (token lists via getters) */
    uint64_t seed;
    size_t generated_len; /* prompt + new */
    size_t sampled_len;   /* new only */
    double decode_ms;
} cd_sample_result;

typedef struct cd_batch_info { /* GenerationBatch, inference.rs:92-103 */
    cd_selection selection;
    double base_prefill_ms, request_prefill_ms, prefill_ms;
    double total_decode_ms, avg_decode_ms, total_ms;
    int32_t nresults;
} cd_batch_info;

/* callback of generate_stream_with_suffix: (token, sampled, nsampled, generated, ngenerated, user);
 * a non-zero return aborts the request */
typedef int (*cd_stream_cb)(uint32_t, const uint32_t*, size_t, const uint32_t*, size_t, void*);

/* InferenceSession::new, inference.rs:124-161 (runs the prefill). */
int cd_session_create(cd_model* m, const uint32_t* prompt_ids, size_t n, float softcap,
                      cd_session** out);
void cd_session_destroy(cd_session* s);
const char* cd_session_last_error(const cd_session* s);
size_t cd_session_prompt_len(const cd_session* s);
double cd_session_prefill_ms(const cd_session* s);
int cd_session_prompt_logits(const cd_session* s, float* out, size_t cap);
/* generate / generate_with_suffix, inference.rs:179-319 */
int cd_session_generate(cd_session* s, const cd_request* req, const uint32_t* suffix, size_t nsuffix,
                        cd_batch_info* info);
/* generate_stream_with_suffix, inference.rs:321-451 (samples must be 1) */
int cd_session_generate_stream(cd_session* s, const cd_request* req, const uint32_t* suffix,
                               size_t nsuffix, cd_stream_cb cb, void* user, cd_batch_info* info);
/* results of the last generate call */
int cd_session_result(const cd_session* s, int sample, cd_sample_result* out);
int cd_session_result_tokens(const cd_session* s, int sample, uint32_t* generated, size_t gcap,
                             uint32_t* sampled, size_t scap);

#ifdef __cplusplus
}
#endif
#endif /* CUDA_DECODE_H */
