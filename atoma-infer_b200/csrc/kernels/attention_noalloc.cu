// attn_decode_noalloc: see attention_noalloc.h for what it is for and what it promises.
//
// The kernels are those of attention_bf16.cu, compiled into this library as well
// (same -DHEAD_DIM); only the home of the split scratch differs.
#include <cstdio>

#include "attention_bf16.cu"
#include "attention_noalloc.h"

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol calls, not an address a kernel could use: the device address comes from
// cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) float g_noalloc_scratch[ATTN_NOALLOC_SCRATCH_FLOATS];
// Arrival counters of the splits, one per (request, key/value head).  They must be zero when a
// launch starts: the loader zero-fills the array and every launch leaves it zero again.
static __device__ __align__(256) int g_noalloc_counters[ATTN_NOALLOC_MAX_GROUPS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device ordinal
int* g_counters_ptr[kMaxDevices] = {};

int fail(int code, char* err, int cap, const char* msg) {
    if (err && cap > 0) snprintf(err, (size_t)cap, "%s", msg);
    return code;
}
}  // namespace

extern "C" int attn_decode_noalloc(const void* q, int q_stride, const void* cache, const int* meta, int group,
                                   const int* cu_tokens, const int* positions, void* out, int S, int nq, int nkv,
                                   int page_size, int num_pages, int window, float scale, int splits, int max_context,
                                   int* status, cudaStream_t stream, char* err, int err_cap) {
    char msg[256];
    if (S <= 0 || nq <= 0 || nkv <= 0 || splits < 1 || page_size <= 0)
        return fail(ATTN_NOALLOC_BAD_ARGUMENT, err, err_cap, "attn_decode_noalloc: S, heads, splits and page_size must be positive");
    if (nq % nkv || nq / nkv > 16)
        return fail(ATTN_NOALLOC_BAD_ARGUMENT, err, err_cap,
                    "attn_decode_noalloc: the query heads must be a multiple (at most 16 times) of the key/value heads");
    if (splits > attn_decode_max_splits(nq, nkv)) {
        snprintf(msg, sizeof msg, "attn_decode_noalloc: %d splits; with %d query heads per key/value head the merge takes "
                 "at most %d", splits, nq / nkv, attn_decode_max_splits(nq, nkv));
        return fail(ATTN_NOALLOC_TOO_LARGE, err, err_cap, msg);
    }
    const size_t need = attn_decode_scratch_floats(S, nq, splits);
    if ((size_t)S * nkv > (size_t)ATTN_NOALLOC_MAX_GROUPS) {
        snprintf(msg, sizeof msg, "attn_decode_noalloc: %d requests x %d key/value heads exceed the %d built-in split counters",
                 S, nkv, ATTN_NOALLOC_MAX_GROUPS);
        return fail(ATTN_NOALLOC_TOO_LARGE, err, err_cap, msg);
    }
    if (need > (size_t)ATTN_NOALLOC_SCRATCH_FLOATS) {
        snprintf(msg, sizeof msg,
                 "attn_decode_noalloc: %d requests x %d heads x %d splits x (%d + 2) = %zu floats of scratch, the built-in "
                 "array holds %u; use fewer splits or requests per call, or attn_decode with a buffer of your own",
                 S, nq, splits, D, need, ATTN_NOALLOC_SCRATCH_FLOATS);
        return fail(ATTN_NOALLOC_TOO_LARGE, err, err_cap, msg);
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        snprintf(msg, sizeof msg, "attn_decode_noalloc: no usable current device (%s)", cudaGetErrorString(e));
        return fail(e != cudaSuccess ? (int)e : ATTN_NOALLOC_BAD_ARGUMENT, err, err_cap, msg);
    }
    if (!g_scratch_ptr[dev]) {  // first call on this device, with it current
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            snprintf(msg, sizeof msg, "attn_decode_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev,
                     cudaGetErrorString(e));
            return fail(e != cudaSuccess ? (int)e : ATTN_NOALLOC_BAD_ARGUMENT, err, err_cap, msg);
        }
        int* c = nullptr;
        e = cudaGetSymbolAddress((void**)&c, g_noalloc_counters);
        if (e != cudaSuccess || !c) {
            snprintf(msg, sizeof msg, "attn_decode_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev,
                     cudaGetErrorString(e));
            return fail(e != cudaSuccess ? (int)e : ATTN_NOALLOC_BAD_ARGUMENT, err, err_cap, msg);
        }
        g_counters_ptr[dev] = c;
        g_scratch_ptr[dev] = p;
    }
    int rc = attn_decode(q, q_stride, cache, meta, group, cu_tokens, positions, out, g_scratch_ptr[dev],
                         g_counters_ptr[dev], nullptr, 0, 0, S, nq, nkv, page_size, num_pages, window, scale, splits,
                         /*cluster_merge=*/0, max_context, status, stream);
    if (rc != 0) {
        snprintf(msg, sizeof msg, "attn_decode_noalloc: launch failed (%s)", cudaGetErrorString((cudaError_t)rc));
        return fail(rc, err, err_cap, msg);
    }
    return 0;
}
