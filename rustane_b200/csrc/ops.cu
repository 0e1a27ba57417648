// Stand-alone operator entry points: one kernel of the token loop on caller-supplied data,
// for kernel-level tests and for callers that want a single op rather than a whole model.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "kernels.cuh"
#include "model.h"

using namespace cd;

namespace {
inline size_t esize(int dtype) { return dtype == CD_DTYPE_F32 ? 4 : 2; }

// [attn_len, kv_heads*hd] row-major rows -> pages [page][2][kv_heads][page_tokens][hd]
template <typename KT>
__global__ void pack_pages_kernel(const KT* __restrict__ k, const KT* __restrict__ v, KT* __restrict__ pool, int attn_len,
                                  int kv_heads, int hd, int page_tokens) {
    const int KV = kv_heads * hd;
    const size_t total = (size_t)attn_len * KV;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(j / KV), c = (int)(j % KV), head = c / hd, d = c % hd;
        const int page = t / page_tokens, off = t % page_tokens;
        pool[((((size_t)page * 2 + 0) * kv_heads + head) * page_tokens + off) * hd + d] = k[j];
        pool[((((size_t)page * 2 + 1) * kv_heads + head) * page_tokens + off) * hd + d] = v[j];
    }
}

template <typename KT>
cudaError_t launch_flash(int hd, dim3 grid, cudaStream_t s, const float* q, const void* pool, const int* pt, const DevState* st,
                         float* pacc, float* pml, unsigned* counters, float* out, int kv_heads, int gqa, int page_tokens, int nsplit) {
    const float scale = 1.0f / std::sqrt((float)hd);
    if (hd == 128)
        attn_decode_kernel<KT, 128><<<grid, 128, 0, s>>>(q, (const KT*)pool, pt, st, pacc, pml, counters, out, kv_heads, gqa, page_tokens, nsplit, scale);
    else
        attn_decode_kernel<KT, 64><<<grid, 128, 0, s>>>(q, (const KT*)pool, pt, st, pacc, pml, counters, out, kv_heads, gqa, page_tokens, nsplit, scale);
    return cudaGetLastError();
}
}  // namespace

namespace cd {
// shared with noalloc.cu
cudaError_t flash_decode_launch(int dtype, int hd, int heads, int nsplit, cudaStream_t s, const float* q, const void* pool,
                                const int* pt, const DevState* st, float* pacc, float* pml, unsigned* counters, float* out,
                                int kv_heads, int page_tokens) {
    const dim3 grid(heads, nsplit);
    const int gqa = heads / kv_heads;
    switch (dtype) {
        case CD_DTYPE_F32: return launch_flash<float>(hd, grid, s, q, pool, pt, st, pacc, pml, counters, out, kv_heads, gqa, page_tokens, nsplit);
        case CD_DTYPE_F16: return launch_flash<__half>(hd, grid, s, q, pool, pt, st, pacc, pml, counters, out, kv_heads, gqa, page_tokens, nsplit);
        default: return launch_flash<__nv_bfloat16>(hd, grid, s, q, pool, pt, st, pacc, pml, counters, out, kv_heads, gqa, page_tokens, nsplit);
    }
}
int flash_decode_check(int dtype, int heads, int kv_heads, int hd, int attn_len, int page_tokens, int nsplit) {
    if (dtype < CD_DTYPE_F32 || dtype > CD_DTYPE_BF16) return fail(nullptr, CD_ERR_INVALID, "unknown dtype");
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return fail(nullptr, CD_ERR_INVALID, "heads must be a positive multiple of kv_heads");
    if (hd != 64 && hd != 128) return fail(nullptr, CD_ERR_UNSUPPORTED, "head dimension must be 64 or 128");
    if (attn_len <= 0) return fail(nullptr, CD_ERR_INVALID, "attn_len must be positive");
    if (page_tokens <= 0 || nsplit <= 0 || nsplit > 64) return fail(nullptr, CD_ERR_INVALID, "page_tokens must be positive and nsplit in 1..64");
    return CD_OK;
}
}  // namespace cd

#define CKG(call)                                                                                    \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ != cudaSuccess) { rc = fail(nullptr, CD_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); goto done; } \
    } while (0)

extern "C" int cd_flash_decode(int dtype, int heads, int kv_heads, int hd, size_t attn_len, int nsplit, const float* q,
                               const void* k, const void* v, float* out) {
    if (!q || !k || !v || !out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    const int page_tokens = 64;
    if (nsplit <= 0) nsplit = (int)std::max<size_t>(1, std::min<size_t>(32, (attn_len + page_tokens - 1) / page_tokens));
    int rc = flash_decode_check(dtype, heads, kv_heads, hd, (int)attn_len, page_tokens, nsplit);
    if (rc) return rc;
    const size_t es = esize(dtype), KV = (size_t)kv_heads * hd, Q = (size_t)heads * hd;
    const int npages = (int)((attn_len + page_tokens - 1) / page_tokens);
    const size_t pool_bytes = (size_t)npages * 2 * KV * page_tokens * es, rows_bytes = attn_len * KV * es;
    void *d_k = nullptr, *d_v = nullptr, *d_pool = nullptr;
    float *d_q = nullptr, *d_out = nullptr, *d_pacc = nullptr, *d_pml = nullptr;
    unsigned* d_cnt = nullptr;
    int* d_pt = nullptr;
    DevState* d_st = nullptr;
    std::vector<int> pt(npages);
    DevState st;
    memset(&st, 0, sizeof st);
    st.pos = (int)attn_len - 1;
    for (int i = 0; i < npages; ++i) pt[i] = i;
    CKG(cudaMalloc(&d_k, rows_bytes));
    CKG(cudaMalloc(&d_v, rows_bytes));
    CKG(cudaMalloc(&d_pool, pool_bytes));
    CKG(cudaMalloc(&d_q, Q * 4));
    CKG(cudaMalloc(&d_out, Q * 4));
    CKG(cudaMalloc(&d_pacc, (size_t)heads * nsplit * hd * 4));  // scratch: per-slice weighted V
    CKG(cudaMalloc(&d_pml, (size_t)heads * nsplit * 2 * 4));    // scratch: per-slice (max, sum)
    CKG(cudaMalloc(&d_cnt, (size_t)heads * 4));                 // scratch: arrival counters
    CKG(cudaMalloc(&d_pt, (size_t)npages * 4));
    CKG(cudaMalloc(&d_st, sizeof(DevState)));
    CKG(cudaMemset(d_pool, 0, pool_bytes));
    CKG(cudaMemset(d_cnt, 0, (size_t)heads * 4));
    CKG(cudaMemcpy(d_k, k, rows_bytes, cudaMemcpyHostToDevice));
    CKG(cudaMemcpy(d_v, v, rows_bytes, cudaMemcpyHostToDevice));
    CKG(cudaMemcpy(d_q, q, Q * 4, cudaMemcpyHostToDevice));
    CKG(cudaMemcpy(d_pt, pt.data(), (size_t)npages * 4, cudaMemcpyHostToDevice));
    CKG(cudaMemcpy(d_st, &st, sizeof st, cudaMemcpyHostToDevice));
    switch (dtype) {
        case CD_DTYPE_F32: pack_pages_kernel<float><<<256, 256>>>((const float*)d_k, (const float*)d_v, (float*)d_pool, (int)attn_len, kv_heads, hd, page_tokens); break;
        case CD_DTYPE_F16: pack_pages_kernel<__half><<<256, 256>>>((const __half*)d_k, (const __half*)d_v, (__half*)d_pool, (int)attn_len, kv_heads, hd, page_tokens); break;
        default: pack_pages_kernel<__nv_bfloat16><<<256, 256>>>((const __nv_bfloat16*)d_k, (const __nv_bfloat16*)d_v, (__nv_bfloat16*)d_pool, (int)attn_len, kv_heads, hd, page_tokens); break;
    }
    CKG(cudaGetLastError());
    CKG(flash_decode_launch(dtype, hd, heads, nsplit, nullptr, d_q, d_pool, d_pt, d_st, d_pacc, d_pml, d_cnt, d_out, kv_heads, page_tokens));
    CKG(cudaMemcpy(out, d_out, Q * 4, cudaMemcpyDeviceToHost));
done:
    cudaFree(d_k); cudaFree(d_v); cudaFree(d_pool); cudaFree(d_q); cudaFree(d_out); cudaFree(d_pacc); cudaFree(d_pml);
    cudaFree(d_cnt); cudaFree(d_pt); cudaFree(d_st);
    return rc;
}
