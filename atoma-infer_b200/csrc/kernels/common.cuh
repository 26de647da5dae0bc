// Shared helpers of the kernel libraries: dtype codes, loads that widen to float,
// block reductions in a fixed order, and the layout of the paged cache.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// dtype codes of the C ABI
#define DT_F32 0
#define DT_BF16 1

// Step metadata: one int32 buffer per step, uploaded in one copy.  The first
// words are a header; kernels read sizes that may differ from the launch's
// (padded) sizes from there, so a captured graph serves any smaller batch.
#define META_NUM_TOKENS 0
#define META_NUM_ENTRIES 1
#define META_NUM_ROWS 2
#define META_BT_STRIDE 4   // + group (up to 8 groups)
#define META_BT_OFFSET 12  // + group: where the group's block tables start, in ints
#define META_HEADER_INTS 20

// Status words (a device int32 array the host reads after a step); non-zero = fault.
#define STATUS_BAD_TOKEN 0
#define STATUS_BAD_PAGE 1
#define STATUS_WORDS 8

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
// Four consecutive elements at once (the address must be a multiple of four elements).
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}
// The rotation of one pair by an angle whose cosine and sine are given: every product and sum rounded on
// its own (no fused multiply-add), so that every kernel that rotates gives the same bits.
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& lo, float& hi) {
    lo = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
    hi = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
}

// Paged cache of one layer: [num_pages, 2 (K, V), num_kv_heads, page_size, head_dim].
// The (page, K|V, head) block of page_size*head_dim elements is contiguous.
struct CacheLayout {
    int num_kv_heads, page_size, head_dim;
    __host__ __device__ size_t page_elems() const { return (size_t)2 * num_kv_heads * page_size * head_dim; }
    __host__ __device__ size_t offset(int page, int kv, int head, int slot) const {
        return (((size_t)page * 2 + kv) * num_kv_heads + head) * (size_t)page_size * head_dim + (size_t)slot * head_dim;
    }
};

// Sum over a block in a fixed order (warp shuffles, then warp 0 over the warp sums):
// the result depends on the values only, not on timing.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// `scratch` holds 33 floats in shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

#define LAUNCH_RETURN() return (int)cudaGetLastError()

// ----------------------------------------------------------------------------- weights ahead of time
// Up to four byte ranges that a kernel asks to be brought into L2 (a hint: nothing waits for it, the copies go on
// underneath whatever runs).  The decode attention of a small batch leaves memory bandwidth unused; it asks for the
// weights of the linear after it, which then streams them from L2.
struct PrefetchRanges {
    const char* ptr[4];
    unsigned long long bytes[4];  // multiples of 16; 0: unused
};
// Every calling thread asks for its share; `n` threads call with i = 0 .. n-1.
__device__ __forceinline__ void prefetch_ranges_l2(const PrefetchRanges& r, unsigned long long i, unsigned long long n) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        if (!r.bytes[s]) continue;
        const unsigned long long share = (((r.bytes[s] + n - 1) / n) + 255) & ~255ull;
        const unsigned long long begin = i * share, end = begin + share < r.bytes[s] ? begin + share : r.bytes[s];
        for (unsigned long long off = begin; off < end; off += 4096) {
            const unsigned len = (unsigned)(end - off < 4096ull ? end - off : 4096ull);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(r.ptr[s] + off), "r"(len) : "memory");
        }
    }
}
static inline PrefetchRanges make_prefetch_ranges(int n, const void* const* ptrs, const unsigned long long* bytes) {
    PrefetchRanges r = {};
    for (int i = 0; i < n && i < 4; ++i) {
        if ((uintptr_t)ptrs[i] & 15) continue;
        r.ptr[i] = (const char*)ptrs[i];
        r.bytes[i] = bytes[i] & ~15ull;
    }
    return r;
}

// ----------------------------------------------------------------------------- dependent launches
// Kernels of a step run back to back on one stream.  Launched with programmatic stream
// serialization, a kernel may start while its predecessor is still draining: what it does
// before pdl_wait() (index arithmetic, loads of weights, which no kernel writes) overlaps the
// predecessor's tail; pdl_wait() returns once all earlier kernels have finished and their
// writes are visible.  Every kernel calls pdl_launch_dependents() at its start and pdl_wait()
// before it reads anything an earlier kernel wrote or writes anything an earlier kernel
// reads.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// per library, set through kernels_set_pdl: bit 0 all kernels, bit 1 the large few-row linears, bit 2 the norm kernel
extern int g_use_pdl;

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel_pdl(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_use_pdl & 1) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
