// cd_flash_decode_static: the split-K flash-decode attention of cd_flash_decode for callers
// that must not allocate device memory.
//
// Who that is: code running inside an engine that has already handed every byte of HBM
// to its own arena (a serving runtime that reserves the whole GPU at start-up, leaving
// cudaMalloc nothing to give), code on a latency-critical thread where cudaMalloc's
// device-wide synchronisation and driver lock are not acceptable, and plug-ins whose host
// forbids driver allocations after initialisation.  Such a caller already owns its inputs
// and outputs in device memory; what it cannot provide is the kernel's scratch
// (per-slice partial results and the arrival counters).  Here that scratch lives in a
// fixed array inside the library image, so the call allocates nothing — no cudaMalloc,
// no cudaFree, no allocating library routine.
//
// Limits that follow from the fixed array: heads <= 64, slices <= 32, head dimension
// <= 128 (about 1.1 MB, resident on every GPU that loads the library until the process
// exits).  Larger shapes are rejected with CD_ERR_UNSUPPORTED.  All calls share the one
// array: two calls whose kernels overlap on the GPU (different streams, or different host
// threads) race on it and must be serialised by the caller.  The array keeps the previous
// call's contents; the arrival counters and the position word, which must start from
// known values, are rewritten by a small kernel at the start of every call.
//
// The first call on each device looks up the array's device address; make that call
// before starting any stream capture.
#include <mutex>

#include "kernels.cuh"
#include "model.h"

using namespace cd;

namespace cd {
cudaError_t flash_decode_launch(int dtype, int hd, int heads, int nsplit, cudaStream_t s, const float* q, const void* pool,
                                const int* pt, const DevState* st, float* pacc, float* pml, unsigned* counters, float* out,
                                int kv_heads, int page_tokens);
int flash_decode_check(int dtype, int heads, int kv_heads, int hd, int attn_len, int page_tokens, int nsplit);
}  // namespace cd

namespace {

constexpr int MAX_HEADS = 64, MAX_SPLITS = 32, MAX_HD = 128, MAX_DEVICES = 64;

struct StaticScratch {
    float part_acc[MAX_HEADS * MAX_SPLITS * MAX_HD];  // per-slice weighted V
    float part_ml[MAX_HEADS * MAX_SPLITS * 2];        // per-slice (max, sum)
    unsigned int counters[MAX_HEADS];                 // arrivals per head
    DevState state;                                   // the position word the kernel reads
};

// In host code this name is only a handle for the runtime's symbol table, never a device
// address: the address is fetched once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) StaticScratch g_scratch;

static __global__ void reset_scratch_kernel(StaticScratch* s, int heads, int pos) {
    for (int i = threadIdx.x; i < heads; i += blockDim.x) s->counters[i] = 0u;
    if (threadIdx.x == 0) {
        s->state.pos = pos;
        s->state.error = 0;
    }
}

std::mutex g_lock;
StaticScratch* g_addr[MAX_DEVICES];  // per device, filled on first use

// Set-up, once per device, with that device current.
int scratch_for_current_device(StaticScratch** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(nullptr, CD_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(nullptr, CD_ERR_UNSUPPORTED, "device ordinal out of range");
    std::lock_guard<std::mutex> guard(g_lock);
    if (g_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(nullptr, CD_ERR_CUDA, std::string("cudaGetSymbolAddress(g_scratch): ") + cudaGetErrorString(e));
        g_addr[dev] = static_cast<StaticScratch*>(p);
    }
    *out = g_addr[dev];
    return CD_OK;
}

}  // namespace

extern "C" int cd_flash_decode_static(int dtype, int heads, int kv_heads, int hd, size_t attn_len, int nsplit, int page_tokens,
                                      const float* d_q, const void* d_kv_pages, const int* d_page_table, float* d_out,
                                      void* stream) {
    if (!d_q || !d_kv_pages || !d_page_table || !d_out) return fail(nullptr, CD_ERR_INVALID, "null argument");
    if (attn_len == 0 || attn_len > (size_t)1 << 24)
        return fail(nullptr, CD_ERR_INVALID, "cd_flash_decode_static: attn_len must be between 1 and 16,777,216");
    if (page_tokens <= 0) page_tokens = 64;
    if (nsplit <= 0) nsplit = (int)std::max<size_t>(1, std::min<size_t>(MAX_SPLITS, (attn_len + page_tokens - 1) / page_tokens));
    int rc = flash_decode_check(dtype, heads, kv_heads, hd, (int)attn_len, page_tokens, nsplit);
    if (rc) return rc;
    if (heads > MAX_HEADS || nsplit > MAX_SPLITS || hd > MAX_HD)
        return fail(nullptr, CD_ERR_UNSUPPORTED,
                    "cd_flash_decode_static: the fixed scratch holds at most 64 heads, 32 slices and head dimension 128");
    StaticScratch* s = nullptr;
    if ((rc = scratch_for_current_device(&s))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    reset_scratch_kernel<<<1, 64, 0, st>>>(s, heads, (int)attn_len - 1);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess)
        e = flash_decode_launch(dtype, hd, heads, nsplit, st, d_q, d_kv_pages, d_page_table, &s->state, s->part_acc, s->part_ml,
                                s->counters, d_out, kv_heads, page_tokens);
    if (e != cudaSuccess) return fail(nullptr, CD_ERR_CUDA, std::string("cd_flash_decode_static launch: ") + cudaGetErrorString(e));
    return CD_OK;
}
