// bfloat16 GEMM on the 5th-generation tensor cores: C = A * B^T with A [RA, K] and B [RB, K], both
// row-major (K contiguous), float32 accumulation in tensor memory.
//
//  * operand tiles (128 x 64 of A, BN x 64 of B) travel from global to shared memory by TMA
//    (cp.async.bulk.tensor, 128-byte swizzle) through a ring of stages guarded by mbarriers;
//  * one elected thread issues tcgen05.mma (M = 128, N = BN, K = 16) from shared-memory matrix
//    descriptors; the accumulator [128 x BN] float32 lives in tensor memory (TMEM);
//  * tcgen05.commit hands a stage back to the TMA thread when the MMAs that read it are done, and
//    signals the epilogue when the whole K loop is done;
//  * the four warps read the accumulator with tcgen05.ld (each its 32 TMEM lanes = 32 rows of the
//    tile), apply the epilogue and store.
//
// Two uses.  Many rows (prompts): A = activations, B = weights, C[row of A, row of B].  Few rows
// (decode batches above 16): A = weights, B = activations, and the tile is stored transposed,
// C[row of B, row of A]: the 128-row side of the MMA is filled by the weight matrix, which is what
// has to stream from memory, instead of by padding.  Epilogues: plain (bfloat16 or float32 out),
// and silu(gate) * up for a stacked [gate; up] weight (many-row form).
//
// The reference has no GEMM of its own: candle calls cuBLAS (models/src/llama.rs:269-271, 311, 364-365).
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises a status word,
// stops issuing work, releases its tensor memory and returns (a wrong result, reported, instead
// of a hang).
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"

int g_use_pdl = 0;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

namespace cg = cooperative_groups;

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr uint32_t WAIT_LIMIT = 1u << 22;  // polls of a barrier before giving up (each poll may sleep a little)
#define STATUS_GEMM_TIMEOUT 2

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the status word) when the barrier did not flip in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&status[STATUS_GEMM_TIMEOUT], 1 + (int)blockIdx.x);
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// ---- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols));
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes (64 bfloat16 along K)
// with the 128-byte swizzle, eight rows to a 1024-byte atom: start address, stride between 8-row
// groups (1024 bytes), descriptor version 1, swizzle mode 2 (128 bytes).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                  // leading byte offset: unused for swizzled K-major tiles
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset
    d |= (uint64_t)1 << 46;                  // version
    d |= (uint64_t)2 << 61;                  // 128-byte swizzle
    return d;
}
// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major, N and M.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

}  // namespace

// EPI 0: plain.  EPI 1: the B tile is [BN/2 gate rows; BN/2 up rows] and the output has BN/2 columns
// per tile: silu(gate) * up.  TRANS: store C[row of B, row of A].
template <int BN, int STAGES, typename TO, int EPI, bool TRANS>
__global__ void __launch_bounds__(128)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_b2, TO* __restrict__ c, int rows_a, int rows_b, int K,
                    int ldc, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    unsigned char* tiles = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile_a = blockIdx.x, tile_b = blockIdx.y;
    const int a0 = tile_a * BM;
    const int b0 = tile_b * (EPI == 1 ? BN / 2 : BN);  // first output column (row of B) of the tile
    // K may be split over the blocks of a thread-block cluster (gridDim.z of them): each takes a range
    // of 64-wide k blocks and the partial tiles are added through distributed shared memory.
    const int ksplit = gridDim.z;
    const int kb_all = (K + BK - 1) / BK, kb_per = (kb_all + ksplit - 1) / ksplit;
    const int kb_first = blockIdx.z * kb_per;
    const int num_kb = max(0, min(kb_all, kb_first + kb_per) - kb_first);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer
        int armed = 0;  // k blocks whose copies were started
        for (int kb = 0; kb < num_kb; ++kb) {
            int s = kb % STAGES;
            uint32_t parity = ((kb / STAGES) & 1) ^ 1;  // a fresh barrier passes a wait on parity 1
            if (!mbar_wait(&empty_bar[s], parity, status, abort_flag)) break;
            unsigned char* a_dst = tiles + s * STAGE_BYTES;
            unsigned char* b_dst = a_dst + A_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, (kb_first + kb) * BK, a0, &full_bar[s]);
            if (EPI == 1) {
                tma_load_2d(b_dst, &map_b, (kb_first + kb) * BK, b0, &full_bar[s]);               // gate rows
                tma_load_2d(b_dst + B_BYTES / 2, &map_b2, (kb_first + kb) * BK, b0, &full_bar[s]);  // up rows
            } else {
                tma_load_2d(b_dst, &map_b, (kb_first + kb) * BK, b0, &full_bar[s]);
            }
            armed = kb + 1;
        }
        if (*abort_flag) {
            // gave up: let the copies already in flight land (bounded) before the block goes away
            for (int kb = max(0, armed - STAGES); kb < armed; ++kb)
                for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(&full_bar[kb % STAGES], (kb / STAGES) & 1); ++i) {}
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = make_idesc(BM, BN);
        bool ok = true;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
            int s = kb % STAGES;
            uint32_t parity = (kb / STAGES) & 1;
            ok = mbar_wait(&full_bar[s], parity, status, abort_flag);
            if (!ok) break;
            tc_fence_after();
            uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                uint64_t a_desc = make_desc(a_addr + k * UMMA_K * 2), b_desc = make_desc(b_addr + k * UMMA_K * 2);
                umma_bf16(tmem_base, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[s]);  // the stage is free again when these MMAs have read it
        }
        umma_commit(accum_bar);          // arrives when every MMA issued so far is complete
    }
    __syncwarp();

    // ---- epilogue: warp w owns TMEM lanes 32w .. 32w+31 = rows a0 + 32w + lane of the tile
    bool ready = mbar_wait(accum_bar, 0, status, abort_flag);
    tc_fence_after();
    if (ksplit > 1) {
        // Partial tile -> this block's shared memory (the stages are idle now), then every block of
        // the cluster adds up a band of rows over all ranks, in rank order, and stores it.
        float* part = reinterpret_cast<float*>(tiles);  // [128][BN]
        if (ready && !*abort_flag) {
            const bool any = num_kb > 0;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (any) tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) part[(warp * 32 + lane) * BN + c0 + i] = any ? v[i] : 0.f;
            }
        }
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int band = (BM + ksplit - 1) / ksplit, r_lo = blockIdx.z * band, r_hi = min(BM, r_lo + band);
        for (int idx = tid; idx < (r_hi - r_lo) * BN; idx += 128) {
            // consecutive threads take consecutive rows of A: in the transposed store they are neighbours in memory
            int r = r_lo + idx % (r_hi - r_lo), j = idx / (r_hi - r_lo);
            float v = 0.f;
            for (int rank = 0; rank < ksplit; ++rank) v += cluster.map_shared_rank(part, rank)[r * BN + j];
            int ra = a0 + r, rb = b0 + j;
            if (ra < rows_a && rb < rows_b) {
                if (TRANS) c[(size_t)rb * ldc + ra] = from_float<TO>(v);
                else c[(size_t)ra * ldc + rb] = from_float<TO>(v);
            }
        }
        cluster.sync();  // nobody leaves while its partial tile may still be read
    } else if (ready && !*abort_flag) {
        const int ra = a0 + warp * 32 + lane;
        constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;
#pragma unroll 1
        for (int c0 = 0; c0 < OUT_COLS; c0 += 16) {
            float v[16];
            tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
            if (EPI == 1) {
                float u[16];
                tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(BN / 2 + c0), u);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.f + expf(-v[i])) * u[i];
            }
            if (TRANS) {
                if (ra < rows_a) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        int rb = b0 + c0 + i;
                        if (rb < rows_b) c[(size_t)rb * ldc + ra] = from_float<TO>(v[i]);
                    }
                }
            } else if (ra < rows_a) {
                TO* dst = c + (size_t)ra * ldc + b0 + c0;
                const int limit = (EPI == 1 ? rows_b : rows_b) - (b0 + c0);  // columns left in the matrix
                if (limit >= 16 && (((size_t)dst) & 15) == 0) {
                    if (sizeof(TO) == 2) {
                        uint32_t w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                            w[i] = *reinterpret_cast<uint32_t*>(&p);
                        }
                        reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (i < limit) dst[i] = from_float<TO>(v[i]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

// The many-row form as a persistent kernel: one block per multiprocessor walks tiles blockIdx.x,
// blockIdx.x + gridDim.x, ... (row tiles fastest, so the blocks that run together share a few weight
// tiles through the L2).  Warp 0 copies (the stage ring runs on across tiles), warp 1 issues the MMAs
// into one of two accumulators in tensor memory, warps 2..5 are the epilogue: they drain one
// accumulator (each warp its 32 lanes) while the tensor core fills the other, so the store of a
// tile costs no tensor-core time.
template <int BN, int STAGES, typename TO, int EPI>
__global__ void __launch_bounds__(192)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_b2, TO* __restrict__ c, int rows_a, int rows_b, int K,
                       int ldc, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators
    static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "two accumulators of 128 or 256 columns");
    constexpr int OUT_COLS = EPI == 1 ? BN / 2 : BN;  // output columns of a tile
    unsigned char* tiles = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;   // [2]: an accumulator is complete
    uint64_t* acc_empty = acc_full + 2;        // [2]: the epilogue warps have read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_a = (rows_a + BM - 1) / BM, tiles_b = (rows_b + OUT_COLS - 1) / OUT_COLS;
    const int num_tiles = tiles_a * tiles_b, num_kb = (K + BK - 1) / BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }  // one arrival per epilogue warp
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer
            int it = 0, armed = 0;  // k blocks over all my tiles; those whose copies were started
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int a0 = (tile % tiles_a) * BM, b0 = (tile / tiles_a) * OUT_COLS;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    int s = it % STAGES;
                    uint32_t parity = ((it / STAGES) & 1) ^ 1;  // a fresh barrier passes a wait on parity 1
                    ok = mbar_wait(&empty_bar[s], parity, status, abort_flag);
                    if (!ok) break;
                    unsigned char* a_dst = tiles + s * STAGE_BYTES;
                    unsigned char* b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * BK, a0, &full_bar[s]);
                    if (EPI == 1) {
                        tma_load_2d(b_dst, &map_b, kb * BK, b0, &full_bar[s]);                // gate rows
                        tma_load_2d(b_dst + B_BYTES / 2, &map_b2, kb * BK, b0, &full_bar[s]);  // up rows
                    } else {
                        tma_load_2d(b_dst, &map_b, kb * BK, b0, &full_bar[s]);
                    }
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // gave up: let the copies already in flight land (bounded) before the block goes away
                for (int j = max(0, armed - STAGES); j < armed; ++j)
                    for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(&full_bar[j % STAGES], (j / STAGES) & 1); ++i) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int it = 0, n = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++n) {
                const int buf = n & 1;
                ok = mbar_wait(&acc_empty[buf], (((uint32_t)n >> 1) & 1u) ^ 1u, status, abort_flag);  // its last tile is stored
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, status, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        uint64_t a_desc = make_desc(a_addr + k * UMMA_K * 2), b_desc = make_desc(b_addr + k * UMMA_K * 2);
                        umma_bf16(tmem_base + buf * BN, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);  // the stage is free again when these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[buf]);  // arrives when every MMA issued so far is complete
            }
        }
    } else {
        // ---- epilogue: a warp reaches the 32 lanes of its quarter = rows a0 + 32 * quarter + lane of the tile
        const int quarter = warp & 3;
        int n = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++n) {
            const int a0 = (tile % tiles_a) * BM, b0 = (tile / tiles_a) * OUT_COLS;
            const int buf = n & 1;
            ok = mbar_wait(&acc_full[buf], ((uint32_t)n >> 1) & 1u, status, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            const int ra = a0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 16) {
                float v[16];
                if (num_kb > 0) {
                    tmem_ld16(acc + (uint32_t)c0, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
                if (EPI == 1 && num_kb > 0) {
                    float u[16];
                    tmem_ld16(acc + (uint32_t)(BN / 2 + c0), u);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.f + __expf(-v[i])) * u[i];
                }
                if (ra < rows_a) {
                    TO* dst = c + (size_t)ra * ldc + b0 + c0;
                    const int limit = rows_b - (b0 + c0);  // columns left in the matrix
                    if (limit >= 16 && (((size_t)dst) & 15) == 0) {
                        if (sizeof(TO) == 2) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                w[i] = *reinterpret_cast<uint32_t*>(&p);
                            }
                            reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i < limit) dst[i] = from_float<TO>(v[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);  // this warp has read its lanes of the accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ----------------------------------------------------------------------------- host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix seen as tiles of box_rows x 64 elements with the 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, typename TO, int EPI, bool TRANS>
int launch(const void* a, const void* b, void* c, int rows_a, int rows_b, int K, int ldc, int ksplit, int* status,
           cudaStream_t stream) {
    constexpr int STAGE_BYTES = BM * BK * 2 + BN * BK * 2;
    constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8 + 16 + 1024;
    CUtensorMap ma, mb, mb2;
    constexpr int BOX_B = EPI == 1 ? BN / 2 : BN;
    if (!make_map(&ma, a, rows_a, K, BM)) return (int)cudaErrorInvalidValue;
    if (!make_map(&mb, b, rows_b, K, BOX_B)) return (int)cudaErrorInvalidValue;
    // the up half of a stacked [gate; up] weight starts rows_b rows further down
    const void* b2 = EPI == 1 ? (const void*)((const bf16*)b + (size_t)rows_b * K) : b;
    if (!make_map(&mb2, b2, rows_b, K, BOX_B)) return (int)cudaErrorInvalidValue;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, TO, EPI, TRANS>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (EPI != 0 && ksplit != 1) return (int)cudaErrorInvalidValue;
    if (ksplit < 1 || ksplit > 8 || (size_t)BM * BN * 4 > (size_t)STAGES * STAGE_BYTES) return (int)cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((rows_a + BM - 1) / BM, (rows_b + BOX_B - 1) / BOX_B, ksplit);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = ksplit;
    cfg.attrs = attr;
    cfg.numAttrs = ksplit > 1 ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, ma, mb, mb2, (TO*)c, rows_a, rows_b, K, ldc, status);
}

template <int BN, typename TO, int EPI>
int launch_persistent(const void* a, const void* b, void* c, int rows_a, int rows_b, int K, int ldc, int* status,
                      cudaStream_t stream) {
    constexpr int STAGE_BYTES = BM * BK * 2 + BN * BK * 2;
    constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16 + 1024;
    CUtensorMap ma, mb, mb2;
    constexpr int BOX_B = EPI == 1 ? BN / 2 : BN;
    if (!make_map(&ma, a, rows_a, K, BM)) return (int)cudaErrorInvalidValue;
    if (!make_map(&mb, b, rows_b, K, BOX_B)) return (int)cudaErrorInvalidValue;
    const void* b2 = EPI == 1 ? (const void*)((const bf16*)b + (size_t)rows_b * K) : b;
    if (!make_map(&mb2, b2, rows_b, K, BOX_B)) return (int)cudaErrorInvalidValue;
    auto kernel = gemm_persistent_kernel<BN, STAGES, TO, EPI>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((rows_a + BM - 1) / BM) * ((rows_b + BOX_B - 1) / BOX_B);
    kernel<<<tiles < sms ? tiles : sms, 192, SMEM, stream>>>(ma, mb, mb2, (TO*)c, rows_a, rows_b, K, ldc, status);
    LAUNCH_RETURN();
}

}  // namespace

// C = A * B^T.  a [rows_a, K], b [rows_b, K] (for epilogue 1: [2 * rows_b, K], gate rows then up rows),
// bfloat16, K % 8 == 0, 16-byte aligned.  transpose = 0: c[rows_a, ldc] gets row ra, column rb;
// transpose = 1: c[rows_b, ldc] gets row rb, column ra.  bn: columns of B per tile (32, 64, 128 or 256).
// ksplit: blocks (of one cluster) that share a tile's K range, 1..8.
// persistent (transpose = 0, ksplit = 1 only): one block per multiprocessor walks the tiles and stores a tile while the next is computed.
extern "C" int gemm_tcgen05(const void* a, const void* b, void* c, int rows_a, int rows_b, int K, int ldc, int out_dtype,
                            int epilogue, int transpose, int bn, int ksplit, int persistent, int* status, cudaStream_t stream) {
    if (rows_a <= 0 || rows_b <= 0) return 0;
    if (K % 8 || K <= 0) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)a | (uintptr_t)b) & 15) return (int)cudaErrorInvalidValue;
#define GO(BN, TO, EPI, TR) return launch<BN, TO, EPI, TR>(a, b, c, rows_a, rows_b, K, ldc, ksplit, status, stream)
    const bool f32 = out_dtype == DT_F32;
    if (!transpose && ksplit == 1 && persistent) {
#define GOP(BN, TO, EPI) return launch_persistent<BN, TO, EPI>(a, b, c, rows_a, rows_b, K, ldc, status, stream)
        if (epilogue == 1) {
            if (f32) return (int)cudaErrorInvalidValue;
            if (bn == 256) GOP(256, bf16, 1);
            if (bn == 128) GOP(128, bf16, 1);
        } else {
            if (bn == 256) { if (f32) GOP(256, float, 0); else GOP(256, bf16, 0); }
            if (bn == 128) { if (f32) GOP(128, float, 0); else GOP(128, bf16, 0); }
        }
#undef GOP
        return (int)cudaErrorInvalidValue;
    }
    if (!transpose) {
        if (epilogue == 1) {
            if (f32) return (int)cudaErrorInvalidValue;
            if (bn == 256) GO(256, bf16, 1, false);
            if (bn == 128) GO(128, bf16, 1, false);
        } else {
            if (bn == 256) { if (f32) GO(256, float, 0, false); else GO(256, bf16, 0, false); }
            if (bn == 128) { if (f32) GO(128, float, 0, false); else GO(128, bf16, 0, false); }
        }
    } else if (epilogue == 0) {
        if (bn == 128) { if (f32) GO(128, float, 0, true); else GO(128, bf16, 0, true); }
        if (bn == 64) { if (f32) GO(64, float, 0, true); else GO(64, bf16, 0, true); }
        if (bn == 32) { if (f32) GO(32, float, 0, true); else GO(32, bf16, 0, true); }
    }
#undef GO
    return (int)cudaErrorInvalidValue;
}
