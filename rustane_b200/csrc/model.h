// Internal definition of cd_model, shared by the ABI translation units.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/cuda_decode.h"
#include "common.cuh"

struct cd_layer_dev {
    void* wqkv;   // [(q_dim + 2 kv_dim), dim]   rows: q | k | v
    void* wo;     // [dim, q_dim]
    void* w13;    // [2 hidden, dim]             rows 2j / 2j+1 = w1 / w3 column j
    void* w2;     // [dim, hidden]
    float* gamma1;
    float* gamma2;
    void* kv;     // this layer's pages: [num_pages][2][kv_heads][page_tokens][hd]
};

enum cd_head_mode { HEAD_NONE = 0, HEAD_LOGITS, HEAD_ARGMAX, HEAD_TOPK, HEAD_STATS,
                    LOOP_GREEDY, LOOP_TOPK, LOOP_FULLVOCAB };

struct cd_graph_key {
    int mode, k, input;
    float t, inv_t, softcap;
    bool operator<(const cd_graph_key& o) const {
        if (mode != o.mode) return mode < o.mode;
        if (k != o.k) return k < o.k;
        if (input != o.input) return input < o.input;
        if (t != o.t) return t < o.t;
        if (inv_t != o.inv_t) return inv_t < o.inv_t;
        return softcap < o.softcap;
    }
};

struct cd_graph_entry {
    cudaGraphExec_t exec;
    uint64_t nodes;
};

// tensor selectors of the builder (values 10.. follow the checkpoint order)
enum { T_EMBED = 0, T_GAMMA_FINAL = 1, T_LM_HEAD = 2,
       T_WQ = 10, T_WK, T_WV, T_WO, T_W1, T_W3, T_W2, T_GAMMA1, T_GAMMA2 };

// MoE + MLA decoder (cd_moe_model_create_synthetic): per-layer weights and the step's scratch
struct cd_moe_layer_dev {
    void* wqa;     // [(heads (nope + rope) + latent + rope) rows][dim]   rows: q | latent | rope key
    void* wuk_t;   // [heads][latent rows][nope]   row (h, c) = wuk[c, h nope .. + nope)
    void* wuv_t;   // [heads v_dim rows][latent]
    void* wo;      // [dim rows][heads v_dim]
    void* wr;      // [n_experts rows][dim]
    void* w13;     // this rank's routed experts: [n_local][2 hidden rows, (w1, w3) interleaved][dim]
    void* w2;      // [n_local][dim rows][hidden]
    void* ws13;    // shared FFN, this rank's columns: [2 shared_cols rows][dim]
    void* ws2;     // [dim rows][shared_cols]
    float *gamma1, *gamma2, *gamma_kv;
};
struct cd_moe_state {
    cd_moe_config mc;
    void* arena = nullptr;
    std::vector<cd_moe_layer_dev> layers;
    int e0 = 0, n_local = 0;        // routed experts this rank holds
    int shared_cols = 0, sc0 = 0;   // its columns of the shared FFN
    int nsplit = 1;                 // attention slices
    void* ws = nullptr;
    float *qa = nullptr, *qabs = nullptr, *part_acc = nullptr, *part_ml = nullptr, *xn2 = nullptr, *sel_w = nullptr, *gate = nullptr;
    int* sel_ids = nullptr;         // [nlayers][top_k]: the router's choice per layer at the last position
    // the router's scratch: logits of all experts, the arrival counter of its CTAs, and the compact list of the
    // chosen experts this rank holds (local index, weight, count) that the expert kernels walk
    float *router_logits = nullptr, *loc_w = nullptr;
    unsigned int* router_counter = nullptr;
    int *loc_ids = nullptr, *n_loc = nullptr;
    void* qsplit = nullptr;         // [2][16][latent + rope] in the cache's type: the absorbed query as a 16-bit head and a 16-bit remainder
    bool stream_ffn = false;        // the experts' rows go through the streamed GEMV (else: the plain-load kernels)
};

struct cd_model {
    cd_moe_state* moe = nullptr;  // set: the handle is a MoE + MLA decoder
    cd_config cfg;       // what this GPU holds: under tensor parallelism heads, kv_heads, hidden, q_dim, kv_dim are per rank
    cd_config full_cfg;  // the model as the caller described it
    int tp_world = 1, tp_rank = 0;
    int v_loc = 0, v0 = 0;          // vocabulary rows of this rank's LM-head shard and the first of them
    int tp_nb = 0;                   // head blocks per rank in the tensor-parallel candidate exchange
    float* tp_topk_vals = nullptr;   // [world][tp_nb * 32] gathered top-k candidates (every rank holds all of them)
    uint32_t* tp_topk_idxs = nullptr;
    char* link_region = nullptr;     // cd::TpRegion, mapped by the peers through CUDA IPC
    size_t tp_pf_rows = 0;           // rows of the prompt pass's partial-sum buffers in the link region (0: no batched prompt pass under tensor parallelism)
    unsigned int tp_pf_seq = 0;      // all-reduces the batched prompt pass has issued (the same on every rank)
    bool tp_connected = false;
    cd::TpLink tp = {};
    struct { int in_reduce = 0; const float* res = nullptr; float* x_out = nullptr; } tp_in;  // set before a GEMV launch that consumes an all-reduce
    void* peer_maps[8] = {nullptr};  // what cudaIpcOpenMemHandle returned, to close on destroy
    cd_options opt;
    int untied = 0;
    int device = 0;
    int sm_count = 0;
    int page_tokens = 64, pages_per_seq = 0, num_pages = 0, nsplit = 1;
    bool pdl = true;     // programmatic dependent launch between the kernels of a token
    int kv_dtype = 0;    // CD_DTYPE_F32 / F16 / BF16: storage of the KV cache (cd_options.kv_dtype resolved)
    unsigned long long wait_ns = 2000000000ull;  // bound of a device-side wait on a peer GPU
    // persistent one-kernel-per-token path (mega.cuh)
    bool mega = false;       // one persistent kernel per token
    int mega_nd = 0, mega_nh = 0;  // GEMV tiling of the K = dim and K = hidden phases; 0 = shape not supported
    void* mega_layers = nullptr;   // device array of cd::MegaLayer
    unsigned long long* grid_counter = nullptr;
    unsigned long long* mega_trace = nullptr;  // per-phase timestamps of the persistent kernel
    int prefetch_kb = 192;  // head of the next kernel's weight stream pulled into L2 by each CTA (0 = off)
    int ring_kb = 220;  // shared memory per GEMV CTA: one CTA per SM
    int nblocks = 0;
    float alpha = 0.f;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f;
    uint64_t launches = 0;
    size_t len = 0;

    // weights
    void* weight_arena = nullptr;
    size_t weight_bytes = 0;
    void* embed = nullptr;
    void* lm_head = nullptr;  // == embed when tied
    float* gamma_final = nullptr;
    std::vector<cd_layer_dev> layers;
    void* kv_arena = nullptr;
    size_t kv_layer_bytes = 0;

    // workspace
    void* ws_arena = nullptr;
    float *x_a = nullptr, *x_b = nullptr, *q = nullptr, *attn = nullptr, *gate = nullptr;
    float *logits = nullptr, *logits_capped = nullptr, *norm_final = nullptr, *part_acc = nullptr, *part_ml = nullptr;
    unsigned int* counters = nullptr;  // [heads] attention + [1] head
    float *block_vals = nullptr, *topk_vals = nullptr, *maxes = nullptr, *sums = nullptr;
    uint32_t *block_idxs = nullptr, *topk_idxs = nullptr, *out_token = nullptr, *out_ring = nullptr;
    uint32_t* prompt_dev = nullptr;
    cd::DevState* st = nullptr;
    int* page_table = nullptr;
    float2* rope = nullptr;
    void* staging = nullptr;  // fp32 upload staging (construction only)
    size_t staging_bytes = 0;
    void* staging2 = nullptr;  // one matrix shard in GEMV orientation as fp32, ahead of quantisation (construction only)
    size_t staging2_bytes = 0;

    // pinned host mirrors for small read-backs
    uint32_t* h_ring = nullptr;
    uint32_t* h_in = nullptr;  // {pos, token} staging for the per-token entry points
    cd::DevState* h_state = nullptr;

    // per-class timing (cd_profile_decode_step)
    bool profiling = false;
    int cur_cls = 0;
    std::vector<cudaEvent_t> prof_events;
    std::vector<int> prof_classes;

    cd::NextStream next_stream = {nullptr, 0, 0, 0, 0};  // set before a GEMV launch, consumed by it
    void* prefill_ctx = nullptr;  // workspace and tensor maps of the batched prompt pass (prefill.cu), built on first use

    std::map<cd_graph_key, cd_graph_entry> graphs;
    std::string err;
};

namespace cd {
// status helpers (model.cu)
int fail(cd_model* m, int code, const std::string& msg);
int device_wait_failed(cd_model* m, int dev_code, const char* where);
void set_global_error(const std::string& msg);
// builder: allocate, fill tensors given in the reference's layouts, finish
int model_alloc(const cd_config* cfg, const cd_options* opts, int untied, cd_model** out, const cd_moe_config* moe = nullptr);
void moe_release(cd_model* m);
size_t model_tensor_elems(const cd_model* m, int which);
int model_set_tensor_f32(cd_model* m, int layer, int which, const float* host);
int model_set_tensor_synth(cd_model* m, int layer, int which, uint64_t seed, float std);
// stored quantised linears (checkpoint.cu): the whole matrix's rows in the device's row format
size_t model_quant_tensor_bytes(const cd_model* m, int which);
int model_set_quant_rows(cd_model* m, int layer, int which, const void* host);
int model_get_quant_rows(cd_model* m, int layer, int which, void* host, size_t cap);
int model_get_plain(cd_model* m, int layer, int which, void* host, size_t cap);
int model_finish(cd_model* m);
// batched prompt pass (prefill.cu): on CD_OK the cache holds positions len .. len+n-1 of the prompt in
// m->prompt_dev and m->x_a holds the last position's hidden state; CD_ERR_UNSUPPORTED: use the per-token path
int prefill_batched(cd_model* m, size_t n);
void prefill_release(cd_model* m);
// ns samples continuing the cached prompt together (prefill.cu); mode 0 greedy, 1 top-k, 2 full-vocabulary
int decode_samples(cd_model* m, const uint32_t* first, int ns, size_t nsteps, int mode, int top_k, float t, float softcap, uint64_t* rng,
                   uint32_t* out_ids);
}  // namespace cd
