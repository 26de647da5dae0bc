// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (AtomaAI/atoma-infer), whose
// split-KV attention allocates its partial-result buffers on every call
// (csrc/src/lib.rs:1785-1800).  It exists for hosts that call this library through
// its C symbols and have no allocator to offer at call time: an embedding runtime
// that gave all free device memory to its page pool at start-up, a serving loop
// that must never reach cudaMalloc once requests flow (cudaMalloc stalls the whole
// device), or a foreign-language binding that can pass plain pointers but not a
// tensor library's allocator.
//
// It is attn_decode (attention_bf16.cu) with one difference: the float32 scratch
// that holds the partial results of the key-range splits is a fixed array inside
// the library instead of a buffer from the caller.
//
//  * Limit: S * num_q_heads * splits * (HEAD_DIM + 2) floats must not exceed
//    ATTN_NOALLOC_SCRATCH_FLOATS (1 Mi floats = 4 MiB).  Larger calls are refused
//    with ATTN_NOALLOC_TOO_LARGE and a message; nothing is launched.
//    Also splits must not exceed attn_decode_max_splits(nq, nkv) (exported by the same
//    library; 512 or more for head size 64, whatever the group size): the block that merges
//    the splits stages their (max, sum) pairs in its shared memory.
//  * Every GPU that loads this library holds the 4 MiB until the process exits.
//  * Pages are loaded with cp.async, as in the engine (the library's opt-in TMA page
//    loads, attn_set_decode_tma(1), apply to this entry point too).
//  * The first call on a device looks up the array's device address (one
//    cudaGetSymbolAddress) and sets the kernel's shared-memory attribute; make that
//    first call outside any stream capture.  Later calls do neither.  The first call
//    on a device is not guarded against a second host thread making it at the same
//    time: make it from one thread, then any thread may call.
//  * It calls no cudaMalloc, cudaFree or any allocating routine, on any path.
//    Also S * num_kv_heads must not exceed ATTN_NOALLOC_MAX_GROUPS (4096).
//  * All calls share the one array and it keeps what the last call left.  The
//    partial results need no clearing: every (request, head, split) slot that the
//    merge reads is written by the same call first, empty splits included.  The
//    small array of arrival counters beside it must be zero when a call starts; it
//    is zero when the library is loaded and every call leaves it zero.  Two
//    calls whose kernels overlap on the GPU (different streams) race on it: keep
//    calls on one stream, or order them yourself.
#pragma once
#include <cuda_runtime.h>

#define ATTN_NOALLOC_SCRATCH_FLOATS (1u << 20)
#define ATTN_NOALLOC_MAX_GROUPS 4096  // requests x key/value heads of one call
#define ATTN_NOALLOC_TOO_LARGE (-1)
#define ATTN_NOALLOC_BAD_ARGUMENT (-2)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as attn_decode's, without the scratch pointer.  Returns 0, a CUDA error
// code (> 0), or one of the negative codes above; on a non-zero return a message is
// written to `err` (if not null, at most `err_cap` bytes, always terminated).
int attn_decode_noalloc(const void* q, int q_stride, const void* cache, const int* meta, int group,
                        const int* cu_tokens, const int* positions, void* out, int S, int nq, int nkv, int page_size,
                        int num_pages, int window, float scale, int splits, int max_context, int* status,
                        cudaStream_t stream, char* err, int err_cap);

#ifdef __cplusplus
}
#endif
