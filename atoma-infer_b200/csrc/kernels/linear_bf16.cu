// Weight-streaming linear layer for few rows: y[M, N] = x[M, K] * w[N, K]^T, bfloat16 in,
// float32 accumulate, bfloat16 or float32 out.
//
// A decode step multiplies a handful of rows by every weight matrix: its time is the
// time to read the weights once, so the kernel is built around the weight stream.
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows = 16 output
// columns per block), the few rows of x the B operand (8 per n-tile).  Every thread
// fetches 16 contiguous bytes of a weight row per load, straight from global memory
// into its fragment: the k index inside a 32-wide block is permuted the same way
// for both operands, which a dot product does not notice.  The warps of a block
// split K between them and add up through shared memory in a fixed order; when a
// matrix has too few 16-row tiles to fill the GPU, the blocks of a thread-block
// cluster split K further and the first block adds the others' partial sums from
// their shared memory (distributed shared memory), again in a fixed order.  A
// 128-row tensor-core tile would be nearly all padding here; the reference calls
// cuBLAS for these products (models/src/llama.rs:269-271, 311, 364-365, 476).
//
// Epilogues: plain; silu(gate) * up for a stacked [gate; up] weight (N/2 output
// columns; a block then takes 8 gate rows and the 8 up rows that belong to them).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#ifndef SM_WARPS
#define SM_WARPS 8        // warps of a block, splitting K
#endif
#ifndef SM_UNROLL
#define SM_UNROLL 4       // 32-wide k blocks in flight per warp
#endif
#ifndef SM_BLOCKS
#define SM_BLOCKS 3       // blocks a multiprocessor should hold (bounds the registers)
#endif
#define SM_MAX_ROWS 16    // rows of x (two n-tiles)

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TO, int NT, int EPI>  // NT n-tiles of 8 rows of x; EPI 1: silu(gate) * up
__global__ void __launch_bounds__(SM_WARPS * 32, SM_BLOCKS)  // blocks a multiprocessor: loads in flight
linear_small_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, TO* __restrict__ y,
                    int M, int N, int K, int ksplits) {
    __shared__ float red[SM_WARPS][16][NT * 8 + 1];
    __shared__ float part[16][NT * 8];  // this block's sum over its warps; read by the cluster's first block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tig = lane & 3;
    const int n_out = EPI == 1 ? N / 2 : N;
    // weight rows of this block's m16 tile: rows 0-7 and 8-15
    int row_lo, row_hi;
    if (EPI == 1) {
        int c = blockIdx.x * 8 + g;
        row_lo = min(c, n_out - 1);
        row_hi = n_out + row_lo;
    } else {
        row_lo = min(blockIdx.x * 16 + g, N - 1);
        row_hi = min(blockIdx.x * 16 + g + 8, N - 1);
    }
    const __nv_bfloat16* wa = w + (size_t)row_lo * K;
    const __nv_bfloat16* wb = w + (size_t)row_hi * K;
    const __nv_bfloat16* xr[NT];
    bool xok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        int m = t * 8 + g;
        xok[t] = m < M;
        xr[t] = x + (size_t)(xok[t] ? m : 0) * K;
    }
    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

    const int nblocks_all = (K + 31) / 32;
    const int per_split = (nblocks_all + ksplits - 1) / ksplits;
    const int kb_begin = blockIdx.y * per_split, nblocks = min(nblocks_all, kb_begin + per_split);
    uint4 va[SM_UNROLL], vb[SM_UNROLL];
    auto load_weights = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            int k = (kb0 + u) * 32 + tig * 8;
            bool ok = kb0 + u < nblocks && k < K;  // K is a multiple of 8: a 16-byte chunk is all inside or all outside
            va[u] = ok ? ldg_stream(wa + k) : make_uint4(0u, 0u, 0u, 0u);
            vb[u] = ok ? ldg_stream(wb + k) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    int kb0 = kb_begin + warp * SM_UNROLL;
    if (kb0 < nblocks) load_weights(kb0);  // weights depend on no earlier kernel: in flight before the wait
    pdl_wait();                            // x is what the kernel before wrote
    pdl_launch_dependents();
    while (kb0 < nblocks) {
        uint4 vx[SM_UNROLL][NT];
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            int k = (kb0 + u) * 32 + tig * 8;
            bool ok = kb0 + u < nblocks && k < K;
#pragma unroll
            for (int t = 0; t < NT; ++t)
                vx[u][t] = (ok && xok[t]) ? *reinterpret_cast<const uint4*>(xr[t] + k) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                mma16816(acc[t], va[u].x, vb[u].x, va[u].y, vb[u].y, vx[u][t].x, vx[u][t].y);
                mma16816(acc[t], va[u].z, vb[u].z, va[u].w, vb[u].w, vx[u][t].z, vx[u][t].w);
            }
        kb0 += SM_WARPS * SM_UNROLL;
        if (kb0 < nblocks) load_weights(kb0);
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        red[warp][g][t * 8 + tig * 2] = acc[t][0];
        red[warp][g][t * 8 + tig * 2 + 1] = acc[t][1];
        red[warp][g + 8][t * 8 + tig * 2] = acc[t][2];
        red[warp][g + 8][t * 8 + tig * 2 + 1] = acc[t][3];
    }
    __syncthreads();
    const int out_rows = EPI == 1 ? 8 : 16;
    if (ksplits > 1) {
        for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += SM_WARPS * 32) {
            int r = idx / (NT * 8), m = idx % (NT * 8);
            float v = 0.f;
#pragma unroll
            for (int wi = 0; wi < SM_WARPS; ++wi) v += red[wi][r][m];
            part[r][m] = v;
        }
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // every block's partial sums are written
        if (blockIdx.y == 0) {
            for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += SM_WARPS * 32) {
                int r = idx / (NT * 8), m = idx % (NT * 8);
                float v = part[r][m];
                for (int rank = 1; rank < ksplits; ++rank)
                    v += cluster.map_shared_rank(&part[0][0], rank)[r * (NT * 8) + m];
                red[0][r][m] = v;
            }
        }
        cluster.sync();  // nobody leaves while its shared memory may still be read
        if (blockIdx.y != 0) return;
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < out_rows * NT * 8; idx += SM_WARPS * 32) {
        int m = idx / out_rows, r = idx % out_rows;  // consecutive threads write consecutive columns
        int col = blockIdx.x * out_rows + r;
        if (m >= M || col >= n_out) continue;
        float v = 0.f, u = 0.f;
        if (ksplits > 1) {
            v = red[0][r][m];
            if (EPI == 1) u = red[0][r + 8][m];
        } else {
#pragma unroll
            for (int wi = 0; wi < SM_WARPS; ++wi) {
                v += red[wi][r][m];
                if (EPI == 1) u += red[wi][r + 8][m];
            }
        }
        if (EPI == 1) v = v / (1.f + expf(-v)) * u;
        y[(size_t)m * n_out + col] = from_float<TO>(v);
    }
}

static int g_ksplit_override = 0;
// For the kernel tests: a fixed number of K splits (0: chosen from the number of tiles, as usual).
extern "C" void linear_skinny_set_ksplit(int k) { g_ksplit_override = k; }

namespace {
int device_sms() {  // multiprocessors of the current device
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 132;
    if (!sms[dev] && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 132;
    return sms[dev];
}
}  // namespace

// x [M, K] and w [N, K] bfloat16, rows 16-byte aligned (K % 8 == 0); M <= 16.
extern "C" int linear_skinny(const void* x, const void* w, void* y, int out_dtype, int epilogue, const int* meta,
                             int use_rows, int M, int N, int K, cudaStream_t stream) {
    (void)meta; (void)use_rows;  // padded rows are computed too: they are rows of the same buffers
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 != 0 || M > SM_MAX_ROWS) return (int)cudaErrorInvalidValue;
    if (epilogue == 1 && ((N % 2) || out_dtype != DT_BF16)) return (int)cudaErrorInvalidValue;
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    const int n_out = epilogue == 1 ? N / 2 : N;
    const int tiles = epilogue == 1 ? (n_out + 7) / 8 : (N + 15) / 16;
    // Too few tiles to fill the GPU: clusters of blocks split K (at least one 32-wide k block per warp each).
    const int sms = device_sms();
    int ksplits = (2 * sms + tiles - 1) / tiles;
    if (g_ksplit_override > 0) ksplits = g_ksplit_override;
    ksplits = max(1, min(min(ksplits, 8), ((K + 31) / 32) / SM_WARPS));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, ksplits, 1);
    cfg.blockDim = dim3(SM_WARPS * 32, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    // a cluster only when K is split; the dependent-launch attribute when it is switched on
    cfg.attrs = ksplits > 1 ? attr : attr + 1;
    cfg.numAttrs = (ksplits > 1 ? 1 : 0) + (((g_use_pdl & 1) || ((g_use_pdl & 2) && (size_t)N * K >= ((size_t)1 << 22))) ? 1 : 0);
    cudaError_t err;
#define SMALL(TO, NT, EPI) err = cudaLaunchKernelEx(&cfg, linear_small_kernel<TO, NT, EPI>, xb, wb, (TO*)y, M, N, K, ksplits)
    if (epilogue == 1) {
        if (M <= 8) SMALL(__nv_bfloat16, 1, 1); else SMALL(__nv_bfloat16, 2, 1);
    } else if (out_dtype == DT_F32) {
        if (M <= 8) SMALL(float, 1, 0); else SMALL(float, 2, 0);
    } else {
        if (M <= 8) SMALL(__nv_bfloat16, 1, 0); else SMALL(__nv_bfloat16, 2, 0);
    }
#undef SMALL
    if (err != cudaSuccess) return (int)err;
    LAUNCH_RETURN();
}
