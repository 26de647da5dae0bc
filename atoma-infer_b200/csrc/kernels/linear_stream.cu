// Weight-streaming linear layer for few rows, fed by the copy engine: y[M, N] = x[M, K] * w[N, K]^T, bfloat16 in,
// float32 accumulate, bfloat16 or float32 out, M <= 16, K a multiple of 64.
//
// One persistent block per multiprocessor.  A warp of its own streams the block's 16-row weight tiles through a ring
// of 16 KB shared-memory stages, one tensor-map box a stage (the [N, K] matrix seen as [K / 64][N][64], so a box of
// 16 rows x 512 k lands as eight 128-byte-swizzled [16][64] blocks that ldmatrix reads without bank conflicts; the
// stacked gate/up matrix as two boxes of 8 rows).  Eight arithmetic warps split a stage's k between them, multiply with
// mma.sync m16n8k16 (weights the A operand, rows of x the B operand) and add up through shared memory in a fixed
// order.  x comes by TMA too: all rows at once when they fit beside the ring (up to 128 KB), else in 512-wide
// chunks through a small ring of its own.  The weights depend on no earlier kernel, so the stream starts before the
// dependency wait of a programmatic dependent launch; x is asked for after it.
//
// A tile is the unit of work; 128 tiles on 148 multiprocessors leave 20 blocks idle, 192 tiles make a second round that
// is a third full.  Cutting a tile's k range into 2 to 8 parts that different blocks take (partial sums to scratch, the
// last part to arrive adds them up) was measured and is not kept: the fence, the atomic and the read of the partial
// sums cost each part 2 to 3 us, more than the idle blocks (q/k/v of Llama 3.2 1B at 8 rows: 3.7 -> 9.7 us; down:
// 7.7 -> 22.4 us).  Also measured and not kept: blocks of half the shared memory (a ring of 4 or 5 stages), so that
// the blocks of the next streamed linear find room beside them and fill their rings while these drain: the decode
// step of Llama 3.2 1B at 8 rows 0.826 -> 0.926 ms; sixteen arithmetic warps instead of eight: 0.840 ms.
//
// Against the few-row linear that loads weights with 16-byte loads straight into fragments (linear_bf16.cu) this one
// keeps more bytes in flight per multiprocessor with one instruction per 16 KB and keeps two n-tiles (9 to 16 rows) as
// fast as one; it needs K % 64 == 0 and the whole GPU to itself.  Every wait is bounded; a block that gives up raises
// status word 5 and stops waiting.  The reference calls cuBLAS for these products (models/src/llama.rs:269-271, 311,
// 364-365, 476).
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstring>

#include "common.cuh"

#define STATUS_STREAM_WAIT 5  // a block of this kernel gave up a wait: 1 + block index

namespace {

typedef __nv_bfloat16 bf16;

constexpr int LS_WARPS = 8;                    // arithmetic warps
constexpr int LS_KB = 16 / LS_WARPS;           // 32-wide k blocks of a stage per warp
constexpr int LS_CONSUMERS = LS_WARPS * 32;
constexpr int LS_THREADS = LS_CONSUMERS + 32;  // and the warp that streams weights
constexpr int LS_KC = 512;                     // k per ring stage: eight groups of 64
constexpr int LS_STAGE_BYTES = 16 * LS_KC * 2;
constexpr int LS_MAX_STAGES = 12;
constexpr int LS_MIN_STAGES = 3;
constexpr int LS_XRING = 6;                    // slots of the ring of x chunks
constexpr int LS_MAX_ROWS = 16;
constexpr size_t LS_X_RESIDENT = 128 * 1024;   // rows of x up to this size stay in shared memory whole
constexpr uint32_t LS_WAIT_POLLS = 1u << 22;
constexpr int BAR_LS_CONSUMERS = 1, BAR_LS_ALL = 2;

__device__ __forceinline__ uint32_t ls_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ls_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ls_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ls_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ls_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ls_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ls_smem(bar)) : "memory");
}
__device__ __forceinline__ bool ls_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(ls_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void ls_tma_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(ls_smem(bar)) : "memory");
}
__device__ __forceinline__ void ls_tma_3d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar,
                                               uint64_t hint) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(ls_smem(bar)), "l"(hint) : "memory");
}
__device__ __forceinline__ void ls_fence_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void ls_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ls_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ls_consumer_sync() { asm volatile("bar.sync %0, %1;" ::"n"(BAR_LS_CONSUMERS), "n"(LS_CONSUMERS) : "memory"); }

// What a block knows about its own failure: once `flag` is set nothing waits any more.
struct LsGiveup {
    volatile int* flag;
    int* status;
    int code;
    __device__ __forceinline__ void raise() const {
        *flag = 1;
        if (status) atomicCAS(status + STATUS_STREAM_WAIT, 0, code);
    }
};
__device__ __forceinline__ bool ls_wait(uint64_t* bar, uint32_t parity, const LsGiveup& gu, bool heed_flag = true) {
    if (ls_mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < LS_WAIT_POLLS; ++i) {
        if (heed_flag && *gu.flag) return false;
        if (ls_mbar_try_wait(bar, parity)) return true;
        if (i > 32) __nanosleep(32);
    }
    gu.raise();
    return false;
}

// An RMSNorm folded into the linears around it (optional).  The linear BEFORE the norm (EPI 2) adds its product into the
// float32 residual stream and leaves, for the norm: the new residual times the norm's weight in bfloat16 (the next
// linear's x), and per 16-column tile and row the sum of squares of the new residual.  The linear AFTER the norm gets
// those sums (`ss_in`, `ss_parts` tiles of 16 floats), adds them up in tile order, and scales its products' rows by
// 1 / sqrt(sum / width + eps): a factor per row commutes with the product.
struct LsNorm {
    const float* ss_in;    // [ss_parts][16] sums of squares left by the linear before (null: x is used as it is)
    int ss_parts, width;   // width: the norm's (the residual's) width
    float eps;
    float* resid;          // EPI 2: [M, N] float32, updated in place
    const float* next_w;   // EPI 2: weight of the norm that follows (null: nothing follows, only the residual is updated)
    bf16* xw_out;          // EPI 2: [M, N] residual * next_w
    float* ss_out;         // EPI 2: [tiles][16]
};

// NT: n-tiles of 8 rows of x.  XMODE 0: all rows of x lie in shared memory; 1: x comes in chunks through a ring.
// EPI 1: w is [gate; up] stacked, the result silu(gate) * up of N / 2 columns.  EPI 2: added into the residual (LsNorm).
template <int NT, int XMODE, int EPI, typename TO>
__global__ void __launch_bounds__(LS_THREADS, 1)
linear_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, TO* __restrict__ y, int M,
                     int N, int K, int stages, int inflight, const LsNorm norm, int* __restrict__ status) {
    constexpr int ROWS = NT * 8;
    constexpr int RED_STRIDE = ROWS + 1;
    constexpr int RED_FLOATS = LS_WARPS * 16 * RED_STRIDE;
    constexpr int XGROUP = ROWS * 128;   // a group of 64 k of all rows
    constexpr int XSLOT = ROWS * 1024;   // a chunk: eight groups
    extern __shared__ __align__(1024) unsigned char ls_smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char* smem = ls_smem_raw + ((1024u - (ls_smem(ls_smem_raw) & 1023u)) & 1023u);
    const int nchunks = (K + LS_KC - 1) / LS_KC, groups = K / 64;
    const uint32_t ring = ls_smem(smem);
    unsigned char* region_ptr = smem + (size_t)stages * LS_STAGE_BYTES;
    const uint32_t region = ls_smem(region_ptr);
    const size_t region_bytes = XMODE == 0 ? (size_t)nchunks * XSLOT : (size_t)LS_XRING * XSLOT;
    float* redbuf = reinterpret_cast<float*>(region_ptr + region_bytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(redbuf + 2 * RED_FLOATS + (2 * RED_FLOATS & 1));
    uint64_t* empty = full + LS_MAX_STAGES;
    uint64_t* xfull = empty + LS_MAX_STAGES;
    uint64_t* xempty = xfull + LS_XRING;
    uint64_t* xbar = xempty + LS_XRING;
    volatile int* gave_up = reinterpret_cast<volatile int*>(xbar + 1);
    float* inv = reinterpret_cast<float*>(const_cast<int*>(gave_up) + 2);  // [16] 1 / rms of the rows (norm.ss_in)
    const LsGiveup gu{gave_up, status, 1 + (int)blockIdx.x};
    const int n_out = EPI == 1 ? N / 2 : N, out_rows = EPI == 1 ? 8 : 16;
    const int tiles = EPI == 1 ? (n_out + 7) / 8 : (N + 15) / 16;
    const int ncta = gridDim.x, cta = blockIdx.x;

    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            ls_mbar_init(full + s, 1);
            ls_mbar_init(empty + s, LS_WARPS);
        }
        for (int s = 0; s < LS_XRING; ++s) {
            ls_mbar_init(xfull + s, 1);
            ls_mbar_init(xempty + s, LS_WARPS);
        }
        ls_mbar_init(xbar, 1);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == LS_WARPS) {
        // ---- the weight stream (no earlier kernel writes weights: it starts at once); one lane does it all
        if (lane == 0) {
            uint64_t policy;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
            unsigned count = 0, slot = 0, free_parity = 1u, gate = 0, gate_parity = 0u;
            bool on = true;
            for (int tile = cta; tile < tiles && on; tile += ncta) {
                for (int c = 0; c < nchunks; ++c) {
                    if (!ls_wait(empty + slot, free_parity, gu)) { on = false; break; }
                    if (count >= (unsigned)inflight) {  // not too much on its way at once
                        if (!ls_wait(full + gate, gate_parity, gu)) { on = false; break; }
                        if (++gate == (unsigned)stages) { gate = 0; gate_parity ^= 1u; }
                    }
                    const uint32_t dst = ring + slot * LS_STAGE_BYTES;
                    ls_mbar_expect_tx(full + slot, (uint32_t)LS_STAGE_BYTES);  // rows and k beyond the matrix arrive as zeros
                    if (EPI == 1) {
                        ls_tma_3d_hint(dst, &wmap, 0, tile * 8, c * (LS_KC / 64), full + slot, policy);
                        ls_tma_3d_hint(dst + LS_STAGE_BYTES / 2, &wmap, 0, n_out + tile * 8, c * (LS_KC / 64), full + slot, policy);
                    } else {
                        ls_tma_3d_hint(dst, &wmap, 0, tile * 16, c * (LS_KC / 64), full + slot, policy);
                    }
                    ++count;
                    if (++slot == (unsigned)stages) { slot = 0; free_parity ^= 1u; }
                }
            }
            // nothing this lane asked for may still be on its way when the block leaves
            const unsigned issued = count, back = issued < (unsigned)stages ? issued : (unsigned)stages;
            for (unsigned i = issued - back; i < issued; ++i)
                ls_wait(full + i % (unsigned)stages, (i / (unsigned)stages) & 1u, gu, false);
        }
    } else {
        // ---- the arithmetic
        const int g = lane >> 2, tig = lane & 3;
        const int mine = cta < tiles ? (tiles - cta + ncta - 1) / ncta : 0;
        const uint32_t half_stride = EPI == 1 ? LS_STAGE_BYTES / 2 : 1024u, group_stride = EPI == 1 ? 1024u : 2048u;
        const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, akc = lane >> 4, brow = lane & 7, bkc = lane >> 3;
        const uint32_t a_lane = (uint32_t)(arow >> 3) * half_stride + (uint32_t)(arow & 7) * 128u;
        pdl_wait();               // x is what the kernel before wrote
        pdl_launch_dependents();
        unsigned slot = 0, parity = 0, xslot = 0, xparity = 0, xissue = 0, xiparity = 1u;
        const unsigned ahead = LS_XRING - 1, xtotal = (unsigned)mine * (unsigned)nchunks;
        int xc = 0;
        auto x_issue = [&]() {  // thread 0: the next chunk of x into the next slot of the x ring
            ls_wait(xempty + xissue, xiparity, gu);
            ls_mbar_expect_tx(xfull + xissue, (uint32_t)XSLOT);
            ls_tma_3d(region + xissue * XSLOT, &xmap, 0, 0, xc * (LS_KC / 64), xfull + xissue);
            if (++xc == nchunks) xc = 0;
            if (++xissue == (unsigned)LS_XRING) { xissue = 0; xiparity ^= 1u; }
        };
        if (tid == 0 && mine > 0) {
            ls_fence_async();
            if (XMODE == 0) {
                ls_mbar_expect_tx(xbar, (uint32_t)ROWS * (uint32_t)groups * 128u);
                ls_tma_3d(region, &xmap, 0, 0, 0, xbar);
            } else {
                for (unsigned f = 0; f < ahead && f < xtotal; ++f) x_issue();
            }
        }
        if (norm.ss_in) {  // the rows' scales, from the sums of squares the linear before left (in tile order)
            for (int m = warp; m < LS_MAX_ROWS; m += LS_WARPS) {
                float ss = 0.f;
                if (m < M)
                    for (int i = lane; i < norm.ss_parts; i += 32) ss += __ldcg(norm.ss_in + (size_t)i * LS_MAX_ROWS + m);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) inv[m] = m < M ? rsqrtf(ss / (float)norm.width + norm.eps) : 0.f;
            }
            ls_consumer_sync();
        }
        if (XMODE == 0 && mine > 0) {
            // beyond the last group of the rows a stage holds zeros, but the region holds whatever was there, and zero
            // times NaN is NaN: the rest of the last chunk is zeroed
            const int upto = nchunks * 8;
            if (upto > groups) {
                unsigned char* tail = region_ptr + (size_t)groups * XGROUP;
                for (int i = tid * 16; i < (upto - groups) * XGROUP; i += LS_CONSUMERS * 16)
                    *reinterpret_cast<uint4*>(tail + i) = make_uint4(0u, 0u, 0u, 0u);
            }
            ls_consumer_sync();
            ls_wait(xbar, 0u, gu);
        }
        unsigned f = 0, done = 0;
        for (int tile = cta; tile < tiles; tile += ncta) {
            float acc[LS_KB][NT][4];
#pragma unroll
            for (int u = 0; u < LS_KB; ++u)
#pragma unroll
                for (int t = 0; t < NT; ++t) acc[u][t][0] = acc[u][t][1] = acc[u][t][2] = acc[u][t][3] = 0.f;
            for (int c = 0; c < nchunks; ++c, ++f) {
                uint32_t xbase;
                unsigned xs = 0;
                if (XMODE == 1) {
                    if (tid == 0 && f + ahead < xtotal) x_issue();
                    xs = xslot;
                    ls_wait(xfull + xs, xparity, gu);
                    xbase = region + xs * XSLOT;
                } else {
                    xbase = region + (uint32_t)c * XSLOT;
                }
                const unsigned s = slot;
                ls_wait(full + s, parity, gu);
                const uint32_t st = ring + s * LS_STAGE_BYTES;
                uint32_t a[LS_KB][2][4], bq[LS_KB][NT][4];
#pragma unroll
                for (int u = 0; u < LS_KB; ++u) {  // every load of the stage first
                    const int kb = warp * LS_KB + u, ko = kb >> 1, hb = kb & 1;
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int kc = (hb * 2 + jj) * 2 + akc;  // 16-byte chunk of the 128-byte row
                        ls_ldsm_x4(a[u][jj], st + (uint32_t)ko * group_stride + a_lane + (uint32_t)((kc ^ (arow & 7)) << 4));
                    }
#pragma unroll
                    for (int t = 0; t < NT; ++t)
                        ls_ldsm_x4(bq[u][t], xbase + (uint32_t)ko * XGROUP + (uint32_t)(t * 8 + brow) * 128u + (uint32_t)(((hb * 4 + bkc) ^ brow) << 4));
                }
#pragma unroll
                for (int u = 0; u < LS_KB; ++u)
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        ls_mma(acc[u][t], a[u][0], bq[u][t][0], bq[u][t][1]);
                        ls_mma(acc[u][t], a[u][1], bq[u][t][2], bq[u][t][3]);
                    }
                __syncwarp();
                if (lane == 0) {
                    ls_mbar_arrive(empty + s);
                    if (XMODE == 1) ls_mbar_arrive(xempty + xs);
                }
                if (++slot == (unsigned)stages) { slot = 0; parity ^= 1u; }
                if (XMODE == 1 && ++xslot == (unsigned)LS_XRING) { xslot = 0; xparity ^= 1u; }
            }
#pragma unroll
            for (int u = 1; u < LS_KB; ++u)  // in k order
#pragma unroll
                for (int t = 0; t < NT; ++t)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[0][t][e] += acc[u][t][e];
            // the tile's sums over the warps, in warp order
            float* red = redbuf + (done & 1u) * RED_FLOATS;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float* r0 = red + (warp * 16 + g) * RED_STRIDE + t * 8 + tig * 2;
                float* r1 = red + (warp * 16 + g + 8) * RED_STRIDE + t * 8 + tig * 2;
                r0[0] = acc[0][t][0]; r0[1] = acc[0][t][1];
                r1[0] = acc[0][t][2]; r1[1] = acc[0][t][3];
            }
            ls_consumer_sync();
            for (int idx = tid; idx < out_rows * ROWS; idx += LS_CONSUMERS) {  // whole warps take part or stay out
                const int m = idx / out_rows, r = idx % out_rows;  // consecutive threads, consecutive columns
                const int col = tile * out_rows + r;
                const bool on = m < M && col < n_out;
                float v = 0.f, u = 0.f;
#pragma unroll
                for (int wi = 0; wi < LS_WARPS; ++wi) {
                    v += red[(wi * 16 + r) * RED_STRIDE + m];
                    if (EPI == 1) u += red[(wi * 16 + r + 8) * RED_STRIDE + m];
                }
                if (EPI == 2) {
                    // into the residual; for the norm after it: the new value times the norm's weight, and the tile's
                    // share of the row's sum of squares (the 16 lanes that hold a row's 16 columns add up)
                    float now = 0.f;
                    if (on) {
                        float* dst = norm.resid + (size_t)m * n_out + col;
                        now = *dst + v;
                        *dst = now;
                        if (norm.next_w) norm.xw_out[(size_t)m * n_out + col] = __float2bfloat16_rn(now * norm.next_w[col]);
                    }
                    if (norm.next_w) {
                        float sq = now * now;
                        sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                        sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                        sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                        if (r == 0) norm.ss_out[(size_t)tile * LS_MAX_ROWS + m] = m < M ? sq : 0.f;
                    }
                } else if (on) {
                    if (norm.ss_in) { v *= inv[m]; u *= inv[m]; }
                    if (EPI == 1) v = v / (1.f + expf(-v)) * u;
                    y[(size_t)m * n_out + col] = from_float<TO>(v);
                }
            }
            ++done;  // the other reduction buffer next: this one may still be read
        }
    }
    asm volatile("bar.sync %0, %1;" ::"n"(BAR_LS_ALL), "n"(LS_THREADS) : "memory");
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*LsEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
LsEncodeFn ls_encode_fn() {
    static LsEncodeFn fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<LsEncodeFn>(q);
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix (K a multiple of 64) seen as [K / 64][rows][64], boxes of `groups` x `box_rows`
// x 64 with the 128-byte swizzle; what lies beyond the matrix arrives as zeros.
bool ls_make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows, int groups) {
    LsEncodeFn fn = ls_encode_fn();
    if (!fn || K % 64 || rows <= 0 || groups < 1 || groups > 256 || ((uintptr_t)base & 15)) return false;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)groups};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct LsPlan { int blocks, stages, xmode; size_t smem; };

template <int NT, int XMODE, int EPI, typename TO>
int ls_launch(const CUtensorMap& wmap, const CUtensorMap& xmap, void* y, int M, int N, int K, const LsPlan& plan, int tiles,
              const LsNorm& norm, int* status, cudaStream_t stream) {
    auto kernel = linear_stream_kernel<NT, XMODE, EPI, TO>;
    static size_t configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (plan.smem > configured[dev]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
        if (err != cudaSuccess) return (int)err;
        configured[dev] = plan.smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.blocks < tiles ? plan.blocks : tiles, 1, 1);
    cfg.blockDim = dim3(LS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_use_pdl & 3) ? 1 : 0;
    int inflight = plan.stages < 6 ? plan.stages : 6;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, wmap, xmap, (TO*)y, M, N, K, plan.stages, inflight, norm, status);
    if (err != cudaSuccess) return (int)err;
    LAUNCH_RETURN();
}

}  // namespace

// Whether linear_stream takes this product on the current device (1) or not (0): M <= 16, K % 64 == 0, and shared
// memory for the rows of x (or its chunk ring) beside at least three weight stages.
extern "C" int linear_stream_supports(int M, int N, int K, int epilogue) {
    if (M <= 0 || M > LS_MAX_ROWS || K <= 0 || K % 64 || N <= 0 || (epilogue == 1 && (N % 2))) return 0;
    return 1;
}

// x [M, K] and w [N, K] bfloat16, both 16-byte aligned; y [M, N] (epilogue 1: [M, N / 2] = silu(gate) * up for w =
// [gate; up]) bfloat16 or float32 (out_dtype).  status: the device status words (may be null).
// A norm folded in (see LsNorm), all optional: ss_in ([ss_parts][16] floats, with norm_width and eps): the rows of the
// result are scaled by the rows' 1 / rms.  epilogue 2: nothing is written to y; the product is added into resid [M, N]
// (float32) and, if next_w is given, xw_out [M, N] (bfloat16) and ss_out [ceil(N / 16)][16] are left for the linear after
// the next norm.
extern "C" int linear_stream_norm(const void* x, const void* w, void* y, int out_dtype, int epilogue, int M, int N, int K,
                                  const float* ss_in, int ss_parts, int norm_width, float eps, float* resid, const float* next_w,
                                  void* xw_out, float* ss_out, int* status, cudaStream_t stream) {
    if (!linear_stream_supports(M, N, K, epilogue)) return (int)cudaErrorInvalidValue;
    if (epilogue == 1 && out_dtype != DT_BF16) return (int)cudaErrorInvalidValue;
    if (epilogue == 2 && (!resid || (next_w && (!xw_out || !ss_out)))) return (int)cudaErrorInvalidValue;
    if (ss_in && (ss_parts <= 0 || norm_width <= 0)) return (int)cudaErrorInvalidValue;
    LsNorm norm;
    norm.ss_in = ss_in; norm.ss_parts = ss_parts; norm.width = norm_width; norm.eps = eps;
    norm.resid = resid; norm.next_w = next_w; norm.xw_out = (bf16*)xw_out; norm.ss_out = ss_out;
    int dev = 0, sms = 0, smem_max = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return (int)cudaErrorInvalidDevice;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return (int)cudaErrorInvalidDevice;
    if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return (int)cudaErrorInvalidDevice;
    const int rows = M <= 8 ? 8 : 16, nchunks = (K + LS_KC - 1) / LS_KC;
    const size_t x_all = (size_t)nchunks * rows * 1024;
    LsPlan plan;
    plan.xmode = x_all <= LS_X_RESIDENT ? 0 : 1;
    const size_t region = plan.xmode == 0 ? x_all : (size_t)LS_XRING * rows * 1024;
    const size_t red = (size_t)(2 * LS_WARPS * 16 * (rows + 1) + 1) * sizeof(float);
    const size_t fixed = region + red + (2 * LS_MAX_STAGES + 2 * LS_XRING + 1) * sizeof(uint64_t) + 64 + LS_MAX_ROWS * sizeof(float) + 1024;
    if (fixed + (size_t)LS_MIN_STAGES * LS_STAGE_BYTES > (size_t)smem_max) return (int)cudaErrorInvalidConfiguration;
    plan.stages = (int)(((size_t)smem_max - fixed) / LS_STAGE_BYTES);
    if (plan.stages > LS_MAX_STAGES) plan.stages = LS_MAX_STAGES;
    plan.smem = fixed + (size_t)plan.stages * LS_STAGE_BYTES;
    plan.blocks = sms;
    const int n_out = epilogue == 1 ? N / 2 : N;
    const int tiles = epilogue == 1 ? (n_out + 7) / 8 : (N + 15) / 16;
    alignas(64) CUtensorMap wmap, xmap;
    if (!ls_make_map(&wmap, w, N, K, epilogue == 1 ? 8 : 16, LS_KC / 64)) return (int)cudaErrorInvalidValue;
    const int xgroups = plan.xmode == 0 ? K / 64 : LS_KC / 64;
    if (xgroups > 256 || !ls_make_map(&xmap, x, M, K, rows, xgroups)) return (int)cudaErrorInvalidValue;
#define LS_CASE(NT, XM) \
    if (epilogue == 2) return ls_launch<NT, XM, 2, float>(wmap, xmap, y, M, N, K, plan, tiles, norm, status, stream); \
    if (epilogue == 1) return ls_launch<NT, XM, 1, __nv_bfloat16>(wmap, xmap, y, M, N, K, plan, tiles, norm, status, stream); \
    if (out_dtype == DT_F32) return ls_launch<NT, XM, 0, float>(wmap, xmap, y, M, N, K, plan, tiles, norm, status, stream); \
    return ls_launch<NT, XM, 0, __nv_bfloat16>(wmap, xmap, y, M, N, K, plan, tiles, norm, status, stream)
    if (rows == 8) {
        if (plan.xmode == 0) { LS_CASE(1, 0); }
        LS_CASE(1, 1);
    }
    if (plan.xmode == 0) { LS_CASE(2, 0); }
    LS_CASE(2, 1);
#undef LS_CASE
}

// The plain product (no norm folded in).
extern "C" int linear_stream(const void* x, const void* w, void* y, int out_dtype, int epilogue, int M, int N, int K, int* status,
                             cudaStream_t stream) {
    if (epilogue == 2) return (int)cudaErrorInvalidValue;
    return linear_stream_norm(x, w, y, out_dtype, epilogue, M, N, K, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr, nullptr, status,
                              stream);
}
