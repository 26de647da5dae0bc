// bfloat16 attention over the paged cache, specialised by head size (-DHEAD_DIM=...).
//
// Two kernels share one tile machinery (cp.async loads through the block table into
// padded shared-memory tiles, ldmatrix, mma.sync m16n8k16 with float32 accumulators,
// online softmax in float32 in base 2, P rounded to bfloat16 before P*V):
//
//  * attn_prefill: one block per (query tile, key/value head, request).  The rows of
//    a tile are (token, query head of the group) pairs, so the query heads that share
//    a key/value head share every key tile read.  A portion of a prompt that starts
//    inside a cached context attends to all of it: keys come from the block table,
//    whatever step wrote them.
//  * attn_decode: one block per (split, key/value head, request) for steps in which
//    every request brings one token.  The group's query heads are the rows of one
//    m16 tile, each key byte is read once; the four warps walk different key tiles
//    (more loads in flight) and merge at the end; several splits of a key range are a
//    thread-block cluster that merges through distributed shared memory (or, beyond the
//    cluster size, through scratch memory, merged by whichever block arrives last).
//
// The reference does both with FlashAttention-2 for sm80 (csrc/kernels/flash_fwd_kernel.h:
// compute_attn_1rowblock :56-500, compute_attn_1rowblock_splitkv :504-1092, combine
// :1131-1313), one query head per block in the paged case (csrc/src/lib.rs:1576-1602).
#include <cooperative_groups.h>
#include <cuda.h>

#include <cstring>

#include "common.cuh"

namespace cg = cooperative_groups;

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head sizes 16..256 in steps of 16");

namespace {

constexpr int D = HEAD_DIM;
// Tiles are [rows][LDS].  Head sizes that are multiples of 64 use dense rows whose 16-byte chunks are
// XOR-swizzled by the row (chunk ^ (row & 7)); other head sizes pad each row by 16 bytes.  Either way
// the eight rows an ldmatrix reads fall into different banks.
constexpr bool SWZ = D % 64 == 0;
constexpr int LDS = SWZ ? D : D + 8;
constexpr int KSTEPS = D / 16;        // k-steps of Q*K^T
constexpr int DTILES = D / 8;         // n-tiles of the output
constexpr bool Q_IN_REGS = D <= 128;  // larger heads reload Q fragments from shared memory
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

// ---- TMA page loads for the decode kernel (head size 64: a page's rows are exactly one 128-byte swizzle row)
constexpr bool DEC_TMA = D == 64;
constexpr uint32_t TMA_WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(map), "r"(x), "r"(y),
                   "r"((uint32_t)__cvta_generic_to_shared(bar)) : "memory");
}

// element offset of (row, col) in a tile; vector accesses pass a col that is a multiple of 8
__device__ __forceinline__ int toff(int row, int col) {
    if (SWZ) return row * D + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7));
    return row * LDS + col;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies the block-table entries of pages page_lo .. page_lo+count-1 into shared memory, once
// per block: a tile load then finds its pages without a dependent global load per row.
// An entry that names no valid page becomes -1 and raises the status word.
__device__ __forceinline__ void stage_block_table(int* bt_s, const int* __restrict__ bt, int page_lo, int count,
                                                  int num_pages, int tid, int nthreads, int* status) {
    for (int i = tid; i < count; i += nthreads) {
        int page = bt[page_lo + i];
        if (page <= 0 || page >= num_pages) {
            atomicExch(&status[STATUS_BAD_PAGE], 1 + (page_lo + i));
            page = -1;
        }
        bt_s[i] = page;
    }
}

// Loads `rows` key rows into ktile and value rows into vtile ([rows][LDS] each), positions
// k0 .. k0+rows-1 of one request and head.  Positions outside [lo, hi) are zero filled (a
// value row of a page nobody wrote must not reach P*V, even times zero).
__device__ __forceinline__ void load_kv_tile(bf16* ktile, bf16* vtile, const bf16* __restrict__ cache,
                                             const CacheLayout& L, const int* bt_s, int page_lo, int kvh, int k0,
                                             int rows, int lo, int hi, int tid, int nthreads) {
    constexpr int PAIRS = D / 16;  // 32-byte sectors per row: one address computation serves four copies
    const int ps = L.page_size;
    const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;
    const size_t v_off = (size_t)L.num_kv_heads * ps * D;  // from a page's K block to its V block
    const size_t page_stride = 2 * v_off, head_off = (size_t)kvh * ps * D;
    for (int idx = tid; idx < rows * PAIRS; idx += nthreads) {
        int r = idx / PAIRS, c = (idx % PAIRS) * 16;
        int pos = k0 + r;
        const int o0 = toff(r, c), o1 = toff(r, c + 8);
        int page = -1, slot = 0;
        if (pos >= lo && pos < hi) {
            int pidx = ps_shift >= 0 ? pos >> ps_shift : pos / ps;
            slot = pos - pidx * ps;
            page = bt_s[pidx - page_lo];
        }
        if (page > 0) {
            const bf16* src = cache + (size_t)page * page_stride + head_off + (size_t)slot * D + c;
            cp_async_16(ktile + o0, src);
            cp_async_16(ktile + o1, src + 8);
            cp_async_16(vtile + o0, src + v_off);
            cp_async_16(vtile + o1, src + v_off + 8);
        } else {
            uint4 z = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(ktile + o0) = z;
            *reinterpret_cast<uint4*>(ktile + o1) = z;
            *reinterpret_cast<uint4*>(vtile + o0) = z;
            *reinterpret_cast<uint4*>(vtile + o1) = z;
        }
    }
}

// A fragments (16 rows x 16 dims, k-step ks) of a row-major tile [16][LDS]
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const bf16* tile16, int ks, int lane) {
    int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = ks * 16 + (lane >> 4) * 8;
    ldmatrix_x4(a, tile16 + toff(row, col));
}

// S[16 x NK*8] = Q (fragments) * K^T for NK n-tiles of keys starting at tile row 0
template <int NK>
__device__ __forceinline__ void qk_tile(float (&s)[NK][4], const uint32_t (*qf)[4], const bf16* qtile16,
                                        const bf16* ktile, int lane) {
#pragma unroll
    for (int n = 0; n < NK; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        if (Q_IN_REGS) { a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3]; }
        else load_a_frag(a, qtile16, ks, lane);
#pragma unroll
        for (int np = 0; np < NK / 2; ++np) {  // two n-tiles (16 keys) per ldmatrix.x4
            uint32_t b[4];
            int j = lane >> 3;
            int key = np * 16 + (lane & 7) + (j >> 1) * 8, dim = ks * 16 + (j & 1) * 8;
            ldmatrix_x4(b, ktile + toff(key, dim));
            mma_bf16(s[2 * np], a, b[0], b[1]);
            mma_bf16(s[2 * np + 1], a, b[2], b[3]);
        }
    }
}

// O[16 x D] += P (from the S accumulators, bfloat16) * V for NK n-tiles of keys
template <int NK>
__device__ __forceinline__ void pv_tile(float (&o)[DTILES][4], const float (&s)[NK][4], const bf16* vtile, int lane) {
#pragma unroll
    for (int ks = 0; ks < NK / 2; ++ks) {  // 16 keys per k-step
        uint32_t a[4] = {pack_bf16(s[2 * ks][0], s[2 * ks][1]), pack_bf16(s[2 * ks][2], s[2 * ks][3]),
                         pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {  // two n-tiles (16 dims) per ldmatrix.x4.trans
            uint32_t b[4];
            int j = lane >> 3;
            int key = ks * 16 + (lane & 7) + (j & 1) * 8, dim = dp * 16 + (j >> 1) * 8;
            ldmatrix_x4_trans(b, vtile + toff(key, dim));
            mma_bf16(o[2 * dp], a, b[0], b[1]);
            mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
        }
    }
}

// Online softmax over one tile of scores (already masked with -inf, in base-2 units).
// Each thread owns rows g = lane/4 and g + 8; a row's values live in the 4 lanes of a quad.
template <int NK>
__device__ __forceinline__ void softmax_tile(float (&s)[NK][4], float (&m)[2], float (&l)[2], float (&o)[DTILES][4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < NK; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * h], s[n][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float m_new = fmaxf(m[h], mx);
        float base = m_new == -INFINITY ? 0.f : m_new;  // a row with no visible key yet stays at zero
        float corr = fast_exp2(m[h] - base);
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < NK; ++n) {
            s[n][2 * h] = fast_exp2(s[n][2 * h] - base);
            s[n][2 * h + 1] = fast_exp2(s[n][2 * h + 1] - base);
            sum += s[n][2 * h] + s[n][2 * h + 1];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[h] = l[h] * corr + sum;
        m[h] = m_new;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            o[dt][2 * h] *= corr;
            o[dt][2 * h + 1] *= corr;
        }
    }
}

}  // namespace

// ----------------------------------------------------------------------------- decode
namespace {
constexpr int DEC_KT = 32;                       // keys per warp tile
constexpr int DEC_NK = DEC_KT / 8;
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = D <= 64 ? 2 : 1;  // above 64 one stage: more blocks a multiprocessor beat a second stage (head size 128: 2.3 -> 3.8 TB/s at 16 requests)
constexpr int DEC_WARP_ELEMS = DEC_STAGES * 2 * DEC_KT * LDS;  // bf16 elements of one warp's K/V stages
constexpr size_t DEC_MERGE_BYTES = (size_t)DEC_WARPS * (32 + 16 * D) * sizeof(float);
constexpr int DEC_MAX_CLUSTER = 8;                     // splits that can merge through the cluster's shared memory
constexpr size_t DEC_SHARE_BYTES = (size_t)(16 * D + 32) * sizeof(float);  // a block's result for its cluster: o[16][D], (m, l)[16]
// The query tile, then one region that holds the warps' key/value stages while keys are walked and afterwards the
// warps' partial results (the merge buffer) followed by the block's result for its cluster.
constexpr size_t DEC_MAIN_BYTES = 16 * LDS * sizeof(bf16) +
    (DEC_WARPS * DEC_WARP_ELEMS * sizeof(bf16) > DEC_MERGE_BYTES + DEC_SHARE_BYTES ? DEC_WARPS * DEC_WARP_ELEMS * sizeof(bf16)
                                                                                   : DEC_MERGE_BYTES + DEC_SHARE_BYTES);
constexpr size_t DEC_SMEM = DEC_MAIN_BYTES;
constexpr int DEC_BLOCKS_PER_SM = (int)((227 * 1024) / (DEC_SMEM + 1024)) < 8 ? (int)((227 * 1024) / (DEC_SMEM + 1024)) : 8;
}  // namespace

// One block per (split, key/value head, request).  Optional fusions for decode steps:
//  * inv_freq != null: the row of the fused projection is still unrotated; the kernel rotates the
//    group's query heads itself and (store_kv) the block that owns the newest position rotates
//    the new key, writes it and the new value to their page, and only then loads that tile;
//  * splits > 1, cluster_merge: the splits of a (request, head group) are one thread-block cluster;
//    every block leaves its partial result in its own shared memory, the cluster meets at its
//    barrier, and the first block reads the others' results through distributed shared memory and
//    merges them in split order.  No global scratch, no fence, no atomic.
//  * splits > 1 otherwise: every block leaves its partial result in scratch and counts itself in;
//    the last block to arrive for a (request, head group) merges all splits in split order.  No
//    block waits for another: whoever comes last does the merge.  `counters` must be zero before
//    the launch and is zero again after it.
// Before the dependency wait the kernel only touches what no kernel of the step writes: the
// step's metadata (block table, positions) and keys and values of earlier steps.
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const __grid_constant__ CUtensorMap map_kv, int use_tma, bf16* __restrict__ q, int q_stride,
                   bf16* __restrict__ cache, CacheLayout L,
                   const int* __restrict__ meta, int group, const int* __restrict__ cu_tokens,
                   const int* __restrict__ positions, bf16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int* __restrict__ counters, const float* __restrict__ inv_freq, int rot,
                   int store_kv, int nq, int window, float scale_log2, int num_pages, int splits, int cluster_merge,
                   int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // tiles start on 1024-byte boundaries: TMA writes them with the 128-byte swizzle, whose pattern follows the address
    unsigned char* smem_al = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    bf16* qtile = reinterpret_cast<bf16*>(smem_al);
    bf16* tiles = qtile + 16 * LDS;
    float* share = reinterpret_cast<float*>(tiles) + DEC_WARPS * (32 + 16 * D);  // behind the merge buffer, once the stages are done
    __shared__ int s_last;
    __shared__ __align__(8) uint64_t tile_bar[DEC_WARPS][2];  // a warp's stage is full (TMA path)
    pdl_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool tma = DEC_TMA && use_tma;
    if (tma && tid == 0) {
        for (int w = 0; w < DEC_WARPS; ++w) { mbar_init(&tile_bar[w][0], 1); mbar_init(&tile_bar[w][1], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const bool live = e < meta[META_NUM_ENTRIES];
    const int G = nq / L.num_kv_heads;
    const int row0 = live ? cu_tokens[e] : 0;
    const int kv_len = live ? positions[row0] + 1 : 0;
    const int kstart = window > 0 ? max(0, kv_len - window) : 0;
    const int per = (((kv_len - kstart + splits - 1) / splits + DEC_KT - 1) / DEC_KT) * DEC_KT;
    const int lo = kstart + split * per, hi = min(kv_len, lo + per);
    const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)e * meta[META_BT_STRIDE + group];
    // A lane copies the same rows of every tile; the pages of a tile's rows are fetched from the block
    // table into registers one tile ahead, so no copy waits for a table lookup.
    constexpr int PAIRS = D / 16, RPL = DEC_KT * PAIRS / 32;  // 32-byte sectors per row; rows*sectors per lane
    const int ps = L.page_size;
    const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;
    const size_t v_off = (size_t)L.num_kv_heads * ps * D, page_stride = 2 * v_off, head_off = (size_t)kvh * ps * D;
    bf16* mine = tiles + warp * DEC_WARP_ELEMS;
    const int ntiles = lo < hi ? (hi - lo + DEC_KT - 1) / DEC_KT : 0;
    auto fetch_pages = [&](int t, int (&pg)[RPL]) {
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            int pos = lo + t * DEC_KT + (lane + 32 * i) / PAIRS;
            pg[i] = -1;
            if (pos < hi) pg[i] = __ldg(bt + (ps_shift >= 0 ? pos >> ps_shift : pos / ps));
        }
    };
    auto load_tile = [&](int t, int stage, const int (&pg)[RPL]) {
        bf16* ktile = mine + stage * 2 * DEC_KT * LDS;
        bf16* vtile = ktile + DEC_KT * LDS;
        if (tma) {
            // One box per page and per K|V instead of 16 sixteen-byte copies per lane.  Lane 0 holds the
            // pages of tile rows 0, 8, 16, 24 in pg[0..3]; the page size is 8, 16 or 32 here.
            const int k0 = lo + t * DEC_KT;
            uint32_t bytes = 0;
            bool okp[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int pos0 = k0 + 8 * i;
                okp[i] = i < RPL && (8 * i) % ps == 0 && pos0 < hi && pg[i < RPL ? i : 0] > 0 && pg[i < RPL ? i : 0] < num_pages;
                if (okp[i]) bytes += (uint32_t)ps * 128u * 2u;
                if (i < RPL && (8 * i) % ps == 0 && pos0 < hi && !okp[i] && lane == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + pos0);
            }
            // rows of pages that are not loaded: zeros (all lanes; a value row nobody wrote must not reach P*V)
            for (int r = lane; r < DEC_KT; r += 32) {
                if (!okp[(r / ps) * ps / 8]) {
#pragma unroll
                    for (int c = 0; c < D; c += 8) {
                        *reinterpret_cast<uint4*>(ktile + toff(r, c)) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(vtile + toff(r, c)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // this warp's reads and zero stores come before the copies
            __syncwarp();
            if (lane == 0) {
                mbar_expect_tx(&tile_bar[warp][stage], bytes);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (!okp[i]) continue;
                    int row_k = ((pg[i < RPL ? i : 0] * 2 + 0) * L.num_kv_heads + kvh) * ps;
                    int row_v = ((pg[i < RPL ? i : 0] * 2 + 1) * L.num_kv_heads + kvh) * ps;
                    tma_load_2d(ktile + 8 * i * LDS, &map_kv, 0, row_k, &tile_bar[warp][stage]);
                    tma_load_2d(vtile + 8 * i * LDS, &map_kv, 0, row_v, &tile_bar[warp][stage]);
                }
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < RPL; ++i) {
            int idx = lane + 32 * i, r = idx / PAIRS, c = (idx % PAIRS) * 16;
            int pos = lo + t * DEC_KT + r;
            int o0 = toff(r, c), o1 = toff(r, c + 8);
            int page = pg[i];
            if (pos < hi && (page <= 0 || page >= num_pages)) {
                atomicExch(&status[STATUS_BAD_PAGE], 1 + pos);
                page = -1;
            }
            if (page > 0) {
                int slot = ps_shift >= 0 ? pos & (ps - 1) : pos % ps;
                const bf16* src = cache + (size_t)page * page_stride + head_off + (size_t)slot * D + c;
                cp_async_16(ktile + o0, src);
                cp_async_16(ktile + o1, src + 8);
                cp_async_16(vtile + o0, src + v_off);
                cp_async_16(vtile + o1, src + v_off + 8);
            } else {  // beyond the split: zeros (a value row nobody wrote must not reach P*V)
                uint4 z = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(ktile + o0) = z;
                *reinterpret_cast<uint4*>(ktile + o1) = z;
                *reinterpret_cast<uint4*>(vtile + o0) = z;
                *reinterpret_cast<uint4*>(vtile + o1) = z;
            }
        }
    };
    int pg_cur[RPL], pg_nxt[RPL];
    if (live && warp < ntiles) fetch_pages(warp, pg_cur);
    if (live && warp + DEC_WARPS < ntiles) fetch_pages(warp + DEC_WARPS, pg_nxt);
    // The newest position (kv_len - 1) is written during this step, by the kernel before this one
    // or by this block; every other key is older than the step and may be fetched at once.
    const bool first_is_old = live && warp < ntiles && lo + (warp + 1) * DEC_KT <= kv_len - 1;
    if (first_is_old) load_tile(warp, 0, pg_cur);
    cp_async_commit();

    pdl_wait();
    if (!live) return;
    const bool owns_newest = lo < hi && hi == kv_len;
    if (inv_freq) {
        const int half = rot / 2, pos = kv_len - 1;
        const bf16* row = q + (size_t)row0 * q_stride;
        // queries of the group, rotated into the tile (rows beyond the group are zero)
        for (int idx = tid; idx < 16 * (D / 2); idx += DEC_WARPS * 32) {
            int r = idx / (D / 2), i = idx % (D / 2);
            float a = 0.f, b = 0.f;
            if (r < G) {
                const bf16* x = row + (size_t)(kvh * G + r) * D;
                if (i < half) {
                    float sn, cs;
                    sincosf((float)pos * inv_freq[i], &sn, &cs);
                    rotate_pair(__bfloat162float(x[i]), __bfloat162float(x[i + half]), cs, sn, a, b);
                    qtile[toff(r, i)] = __float2bfloat16_rn(a);
                    qtile[toff(r, i + half)] = __float2bfloat16_rn(b);
                } else {
                    // dims beyond the rotated part, two to a slot: rot + 2j and rot + 2j + 1, j = i - half
                    int j = rot + 2 * (i - half);
                    qtile[toff(r, j)] = x[j];
                    qtile[toff(r, j + 1)] = x[j + 1];
                }
            } else {
                qtile[toff(r, 2 * i)] = __float2bfloat16_rn(0.f);
                qtile[toff(r, 2 * i + 1)] = __float2bfloat16_rn(0.f);
            }
        }
        if (store_kv && owns_newest) {  // the newest key and value go to their page before their tile is read
            int page = bt[pos / L.page_size];
            if (page > 0 && page < num_pages) {
                const int nkv = L.num_kv_heads;
                const bf16* kx = row + (size_t)(nq + kvh) * D;
                const bf16* vx = row + (size_t)(nq + nkv + kvh) * D;
                bf16* kd = cache + L.offset(page, 0, kvh, pos % L.page_size);
                bf16* vd = cache + L.offset(page, 1, kvh, pos % L.page_size);
                for (int i = tid; i < half; i += DEC_WARPS * 32) {
                    float sn, cs;
                    sincosf((float)pos * inv_freq[i], &sn, &cs);
                    float lo, hi;
                    rotate_pair(__bfloat162float(kx[i]), __bfloat162float(kx[i + half]), cs, sn, lo, hi);
                    kd[i] = __float2bfloat16_rn(lo);
                    kd[i + half] = __float2bfloat16_rn(hi);
                }
                for (int i = rot + tid; i < D; i += DEC_WARPS * 32) kd[i] = kx[i];
                for (int i = tid; i < D; i += DEC_WARPS * 32) vd[i] = vx[i];
                __threadfence();
                asm volatile("fence.proxy.async.global;" ::: "memory");  // the page may be fetched by TMA next
            }
        }
    } else {
        for (int idx = tid; idx < 16 * (D / 8); idx += DEC_WARPS * 32) {
            int r = idx / (D / 8), c = idx % (D / 8);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < G) v = *reinterpret_cast<const uint4*>(q + (size_t)row0 * q_stride + (size_t)(kvh * G + r) * D + c * 8);
            *reinterpret_cast<uint4*>(qtile + toff(r, c * 8)) = v;
        }
    }
    __syncthreads();
    if (warp < ntiles && !first_is_old) load_tile(warp, 0, pg_cur);
    cp_async_commit();

    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[ks], qtile, ks, lane);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

    for (int t = warp, it = 0; t < ntiles; t += DEC_WARPS, ++it) {
        int stage = 0;
        if (DEC_STAGES == 2) {
            stage = it & 1;
            if (t + DEC_WARPS < ntiles) load_tile(t + DEC_WARPS, stage ^ 1, pg_nxt);
            cp_async_commit();
            if (t + 2 * DEC_WARPS < ntiles) fetch_pages(t + 2 * DEC_WARPS, pg_nxt);  // arrives while this tile is computed
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        bf16* ktile = mine + stage * 2 * DEC_KT * LDS;
        bf16* vtile = ktile + DEC_KT * LDS;
        if (tma) {
            // the stage's it/2-th use: its barrier flips once per use (bounded wait)
            const uint32_t parity = (uint32_t)(it >> 1) & 1u;
            bool arrived = false;
            for (uint32_t spin = 0; spin < TMA_WAIT_LIMIT && !arrived; ++spin) arrived = mbar_try_wait(&tile_bar[warp][stage], parity);
            if (!arrived) {
                if (lane == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + lo);
                break;
            }
            // a page is copied whole: value rows beyond the split's last key are zeroed (0 * garbage must stay 0)
            const int k0z = lo + t * DEC_KT;
            if (k0z + DEC_KT > hi) {
                for (int r = max(hi - k0z, 0) + lane; r < DEC_KT; r += 32)
#pragma unroll
                    for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(vtile + toff(r, c)) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        __syncwarp();
        float s[DEC_NK][4];
        qk_tile<DEC_NK>(s, qf, qtile, ktile, lane);
        const int k0 = lo + t * DEC_KT;
#pragma unroll
        for (int n = 0; n < DEC_NK; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int key = k0 + n * 8 + (lane & 3) * 2 + (c & 1);
                s[n][c] = key < hi ? s[n][c] * scale_log2 : -INFINITY;
            }
        softmax_tile<DEC_NK>(s, m, l, o);
        pv_tile<DEC_NK>(o, s, vtile, lane);
        __syncwarp();
        if (DEC_STAGES == 1) {
            if (t + DEC_WARPS < ntiles) {
                load_tile(t + DEC_WARPS, 0, pg_nxt);
                if (t + 2 * DEC_WARPS < ntiles) fetch_pages(t + 2 * DEC_WARPS, pg_nxt);
            }
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its tiles: the space becomes the merge buffer
    float* mbuf = reinterpret_cast<float*>(tiles);
    float* wm = mbuf + warp * (32 + 16 * D);  // m[16], l[16], o[16][D]
    const int g = lane >> 2, tig = lane & 3;
    if (tig == 0) {
        wm[g] = m[0]; wm[g + 8] = m[1];
        wm[16 + g] = l[0]; wm[16 + g + 8] = l[1];
    }
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
        int dim = dt * 8 + tig * 2;
        wm[32 + g * D + dim] = o[dt][0]; wm[32 + g * D + dim + 1] = o[dt][1];
        wm[32 + (g + 8) * D + dim] = o[dt][2]; wm[32 + (g + 8) * D + dim + 1] = o[dt][3];
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += DEC_WARPS * 32) {
        int r = idx / D, i = idx % D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, mbuf[w * (32 + 16 * D) + r]);
        float lsum = 0.f, acc = 0.f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float* p = mbuf + w * (32 + 16 * D);
                float f = fast_exp2(p[r] - mx);
                lsum += p[16 + r] * f;
                acc += p[32 + r * D + i] * f;
            }
        }
        const int head = kvh * G + r;
        if (splits == 1) {
            out[((size_t)row0 * nq + head) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
        } else if (cluster_merge) {
            share[r * D + i] = acc;
            if (i == 0) { share[16 * D + 2 * r] = mx; share[16 * D + 2 * r + 1] = lsum; }
        } else {
            size_t slot = ((size_t)e * nq + head) * splits + split;
            part_o[slot * D + i] = acc;
            if (i == 0) { part_ml[slot * 2] = mx; part_ml[slot * 2 + 1] = lsum; }
        }
    }
    if (splits == 1) return;
    if (cluster_merge) {
        // Every block of the cluster reaches both barriers (a dead request leaves as a whole cluster, above).
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // every split's result is in its block's shared memory
        if (split == 0) {
            for (int idx = tid; idx < G * D; idx += DEC_WARPS * 32) {
                int r = idx / D, i = idx % D;
                float pm[DEC_MAX_CLUSTER], pl[DEC_MAX_CLUSTER], po[DEC_MAX_CLUSTER];
#pragma unroll
                for (int s = 0; s < DEC_MAX_CLUSTER; ++s) {  // independent loads, all in flight together
                    pm[s] = -INFINITY; pl[s] = 0.f; po[s] = 0.f;
                    if (s < splits) {
                        const float* remote = cluster.map_shared_rank(share, s);
                        pm[s] = remote[16 * D + 2 * r];
                        pl[s] = remote[16 * D + 2 * r + 1];
                        po[s] = remote[r * D + i];
                    }
                }
                float mx = -INFINITY;
#pragma unroll
                for (int s = 0; s < DEC_MAX_CLUSTER; ++s) mx = fmaxf(mx, pm[s]);
                float lsum = 0.f, acc = 0.f;
                if (mx > -INFINITY) {
#pragma unroll
                    for (int s = 0; s < DEC_MAX_CLUSTER; ++s)
                        if (s < splits) {
                            float f = fast_exp2(pm[s] - mx);
                            lsum += pl[s] * f;
                            acc += po[s] * f;
                        }
                }
                out[((size_t)row0 * nq + kvh * G + r) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
            }
        }
        cluster.sync();  // nobody leaves while its shared memory may still be read
        return;
    }
    // count this block in; the last one merges the splits of its (request, head group)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* c = counters + e * L.num_kv_heads + kvh;
        int old = atomicAdd(c, 1);
        s_last = old == splits - 1;
        if (s_last) *c = 0;  // as it was found, for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // All loads of the merge are independent: first the (max, sum) pairs of every (head, split) into
    // shared memory, then every thread walks the splits of its (head, dim) eight loads at a time.
    float* ml = reinterpret_cast<float*>(tiles);  // [G][splits][2]
    for (int idx = tid; idx < G * splits * 2; idx += DEC_WARPS * 32) {
        int r = idx / (splits * 2), j = idx % (splits * 2);
        ml[idx] = __ldcg(part_ml + (((size_t)e * nq + kvh * G + r) * splits) * 2 + j);
    }
    __syncthreads();
    for (int idx = tid; idx < G * D; idx += DEC_WARPS * 32) {
        int r = idx / D, i = idx % D;
        const int head = kvh * G + r;
        const float* po = part_o + (((size_t)e * nq + head) * splits) * D + i;
        const float* mlr = ml + r * splits * 2;
        float mx = -INFINITY;
        for (int s = 0; s < splits; ++s) mx = fmaxf(mx, mlr[2 * s]);
        float lsum = 0.f, acc = 0.f;
        if (mx > -INFINITY) {
            for (int s0 = 0; s0 < splits; s0 += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = s0 + j < splits ? __ldcg(po + (size_t)(s0 + j) * D) : 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (s0 + j < splits) {
                        float f = fast_exp2(mlr[2 * (s0 + j)] - mx);
                        lsum += mlr[2 * (s0 + j) + 1] * f;
                        acc += v[j] * f;
                    }
            }
        }
        out[((size_t)row0 * nq + head) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    }
}

// ----------------------------------------------------------------------------- decode, large batches
// The same attention for batches with more (request, head group) pairs than about half the blocks the GPU
// holds: there, one block per pair (or per fixed split of a pair) leaves a last partial wave of blocks that
// run almost alone.  Here the grid is as many blocks as the GPU holds at once and the 32-key tiles of all
// pairs, in (request, head group, key) order, are dealt out evenly: a block takes a contiguous run of
// tiles, which may end one pair and begin the next (a run is cut into segments at pair boundaries).  A
// pair that one block covers alone is written directly; otherwise every segment's partial result goes to
// scratch slot (block index + pair index), a pair's slots being consecutive, and the last block to arrive
// for the pair merges its slots in order.  No block waits for another.
namespace {
constexpr size_t FLAT_SMEM_FIXED = DEC_MAIN_BYTES;  // then (requests + 1) ints: tiles before each request
}

__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_flat_kernel(bf16* __restrict__ q, int q_stride, bf16* __restrict__ cache, CacheLayout L,
                        const int* __restrict__ meta, int group, const int* __restrict__ cu_tokens,
                        const int* __restrict__ positions, bf16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* __restrict__ counters, const float* __restrict__ inv_freq, int rot,
                        int store_kv, int nq, int window, float scale_log2, int num_pages, int S,
                        int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qtile = reinterpret_cast<bf16*>(smem_raw);
    bf16* tiles = qtile + 16 * LDS;
    int* prefix = reinterpret_cast<int*>(smem_raw + FLAT_SMEM_FIXED);  // [S + 1]
    __shared__ int s_last;
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nkv = L.num_kv_heads, G = nq / nkv;
    // tiles of every request (one head group's worth), then their running sum; only the step's metadata is read
    const int live = min(S, meta[META_NUM_ENTRIES]);
    for (int e = tid; e < S; e += DEC_WARPS * 32) {
        int n = 0;
        if (e < live) {
            const int kv_len = positions[cu_tokens[e]] + 1;
            const int ks = window > 0 ? max(0, kv_len - window) : 0;
            n = (kv_len - ks + DEC_KT - 1) / DEC_KT;
        }
        prefix[e + 1] = n;
    }
    if (tid == 0) prefix[0] = 0;
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 1; base <= S; base += 32) {
            const int i = base + lane;
            int v = i <= S ? prefix[i] : 0;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int u = __shfl_up_sync(0xffffffffu, v, off);
                if (lane >= off) v += u;
            }
            if (i <= S) prefix[i] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
    const int total = prefix[S] * nkv;
    const int per = (total + (int)gridDim.x - 1) / (int)gridDim.x;  // tiles per block
    int t = blockIdx.x * per;
    const int t_end = min(total, t + per);
    pdl_wait();  // q (and, without the fused rotation, the newest key and value) come from the kernels before
    if (t >= t_end) return;
    int e = 0;
    {   // the request that holds tile t: the last one whose first tile is not beyond it
        int lo_e = 0, hi_e = S - 1;
        while (lo_e < hi_e) {
            int mid = (lo_e + hi_e + 1) >> 1;
            if (prefix[mid] * nkv <= t) lo_e = mid; else hi_e = mid - 1;
        }
        e = lo_e;
    }
    constexpr int PAIRS = D / 16, RPL = DEC_KT * PAIRS / 32;  // 32-byte sectors per row; rows*sectors per lane
    const int ps = L.page_size;
    const int ps_shift = (ps & (ps - 1)) == 0 ? 31 - __clz(ps) : -1;
    const size_t v_off = (size_t)nkv * ps * D, page_stride = 2 * v_off;
    bf16* mine = tiles + warp * DEC_WARP_ELEMS;
    const int g = lane >> 2, tig = lane & 3;

    while (t < t_end) {
        while (prefix[e + 1] * nkv <= t) ++e;  // requests without tiles are stepped over
        const int nt_e = prefix[e + 1] - prefix[e];
        const int rel = t - prefix[e] * nkv;
        const int kvh = rel / nt_e, tile0 = rel % nt_e;
        const int tile1 = min(nt_e, tile0 + (t_end - t));
        const int ntiles = tile1 - tile0;
        const int pair = e * nkv + kvh, pair_begin = prefix[e] * nkv + kvh * nt_e;
        const int first_block = pair_begin / per, parts = (pair_begin + nt_e - 1) / per - first_block + 1;
        const int row0 = cu_tokens[e], kv_len = positions[row0] + 1;
        const int kstart = window > 0 ? max(0, kv_len - window) : 0;
        const int lo = kstart + tile0 * DEC_KT, hi = min(kv_len, kstart + tile1 * DEC_KT);
        const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)e * meta[META_BT_STRIDE + group];
        const size_t head_off = (size_t)kvh * ps * D;
        auto fetch_pages = [&](int tt, int (&pg)[RPL]) {
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                int pos = lo + tt * DEC_KT + (lane + 32 * i) / PAIRS;
                pg[i] = -1;
                if (pos < hi) pg[i] = __ldg(bt + (ps_shift >= 0 ? pos >> ps_shift : pos / ps));
            }
        };
        auto load_tile = [&](int tt, int stage, const int (&pg)[RPL]) {
            bf16* ktile = mine + stage * 2 * DEC_KT * LDS;
            bf16* vtile = ktile + DEC_KT * LDS;
#pragma unroll
            for (int i = 0; i < RPL; ++i) {
                int idx = lane + 32 * i, r = idx / PAIRS, c = (idx % PAIRS) * 16;
                int pos = lo + tt * DEC_KT + r;
                int o0 = toff(r, c), o1 = toff(r, c + 8);
                int page = pg[i];
                if (pos < hi && (page <= 0 || page >= num_pages)) {
                    atomicExch(&status[STATUS_BAD_PAGE], 1 + pos);
                    page = -1;
                }
                if (page > 0) {
                    int slot = ps_shift >= 0 ? pos & (ps - 1) : pos % ps;
                    const bf16* src = cache + (size_t)page * page_stride + head_off + (size_t)slot * D + c;
                    cp_async_16(ktile + o0, src);
                    cp_async_16(ktile + o1, src + 8);
                    cp_async_16(vtile + o0, src + v_off);
                    cp_async_16(vtile + o1, src + v_off + 8);
                } else {  // beyond the segment: zeros (a value row nobody wrote must not reach P*V)
                    uint4 z = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(ktile + o0) = z;
                    *reinterpret_cast<uint4*>(ktile + o1) = z;
                    *reinterpret_cast<uint4*>(vtile + o0) = z;
                    *reinterpret_cast<uint4*>(vtile + o1) = z;
                }
            }
        };
        int pg_cur[RPL], pg_nxt[RPL];
        if (warp < ntiles) fetch_pages(warp, pg_cur);
        if (warp + DEC_WARPS < ntiles) fetch_pages(warp + DEC_WARPS, pg_nxt);
        // every key but the newest is older than this step: a first tile without it can be fetched at once
        const bool first_is_old = warp < ntiles && lo + (warp + 1) * DEC_KT <= kv_len - 1;
        if (first_is_old) load_tile(warp, 0, pg_cur);
        cp_async_commit();

        // ---- the group's queries into the tile (rotated here when the rotation is fused), the newest key and value
        if (inv_freq) {
            const int half = rot / 2, pos = kv_len - 1;
            const bf16* row = q + (size_t)row0 * q_stride;
            for (int idx = tid; idx < 16 * (D / 2); idx += DEC_WARPS * 32) {
                int r = idx / (D / 2), i = idx % (D / 2);
                if (r < G) {
                    const bf16* x = row + (size_t)(kvh * G + r) * D;
                    if (i < half) {
                        float sn, cs, a, b;
                        sincosf((float)pos * inv_freq[i], &sn, &cs);
                        rotate_pair(__bfloat162float(x[i]), __bfloat162float(x[i + half]), cs, sn, a, b);
                        qtile[toff(r, i)] = __float2bfloat16_rn(a);
                        qtile[toff(r, i + half)] = __float2bfloat16_rn(b);
                    } else {  // dims beyond the rotated part, two to a slot
                        int j = rot + 2 * (i - half);
                        qtile[toff(r, j)] = x[j];
                        qtile[toff(r, j + 1)] = x[j + 1];
                    }
                } else {
                    qtile[toff(r, 2 * i)] = __float2bfloat16_rn(0.f);
                    qtile[toff(r, 2 * i + 1)] = __float2bfloat16_rn(0.f);
                }
            }
            if (store_kv && hi == kv_len) {  // this segment owns the newest position: its key and value go to their page first
                int page = bt[pos / ps];
                if (page > 0 && page < num_pages) {
                    const bf16* kx = row + (size_t)(nq + kvh) * D;
                    const bf16* vx = row + (size_t)(nq + nkv + kvh) * D;
                    bf16* kd = cache + L.offset(page, 0, kvh, pos % ps);
                    bf16* vd = cache + L.offset(page, 1, kvh, pos % ps);
                    for (int i = tid; i < half; i += DEC_WARPS * 32) {
                        float sn, cs, a, b;
                        sincosf((float)pos * inv_freq[i], &sn, &cs);
                        rotate_pair(__bfloat162float(kx[i]), __bfloat162float(kx[i + half]), cs, sn, a, b);
                        kd[i] = __float2bfloat16_rn(a);
                        kd[i + half] = __float2bfloat16_rn(b);
                    }
                    for (int i = rot + tid; i < D; i += DEC_WARPS * 32) kd[i] = kx[i];
                    for (int i = tid; i < D; i += DEC_WARPS * 32) vd[i] = vx[i];
                    __threadfence();
                }
            }
        } else {
            for (int idx = tid; idx < 16 * (D / 8); idx += DEC_WARPS * 32) {
                int r = idx / (D / 8), c = idx % (D / 8);
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (r < G) v = *reinterpret_cast<const uint4*>(q + (size_t)row0 * q_stride + (size_t)(kvh * G + r) * D + c * 8);
                *reinterpret_cast<uint4*>(qtile + toff(r, c * 8)) = v;
            }
        }
        __syncthreads();
        if (warp < ntiles && !first_is_old) load_tile(warp, 0, pg_cur);
        cp_async_commit();

        uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
        if (Q_IN_REGS) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[ks], qtile, ks, lane);
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[DTILES][4];
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
        for (int tt = warp, it = 0; tt < ntiles; tt += DEC_WARPS, ++it) {
            int stage = 0;
            if (DEC_STAGES == 2) {
                stage = it & 1;
                if (tt + DEC_WARPS < ntiles) load_tile(tt + DEC_WARPS, stage ^ 1, pg_nxt);
                cp_async_commit();
                if (tt + 2 * DEC_WARPS < ntiles) fetch_pages(tt + 2 * DEC_WARPS, pg_nxt);  // arrives while this tile is computed
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            bf16* ktile = mine + stage * 2 * DEC_KT * LDS;
            bf16* vtile = ktile + DEC_KT * LDS;
            __syncwarp();
            float s[DEC_NK][4];
            qk_tile<DEC_NK>(s, qf, qtile, ktile, lane);
            const int k0 = lo + tt * DEC_KT;
#pragma unroll
            for (int n = 0; n < DEC_NK; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    int key = k0 + n * 8 + (lane & 3) * 2 + (c & 1);
                    s[n][c] = key < hi ? s[n][c] * scale_log2 : -INFINITY;
                }
            softmax_tile<DEC_NK>(s, m, l, o);
            pv_tile<DEC_NK>(o, s, vtile, lane);
            __syncwarp();
            if (DEC_STAGES == 1) {
                if (tt + DEC_WARPS < ntiles) {
                    load_tile(tt + DEC_WARPS, 0, pg_nxt);
                    if (tt + 2 * DEC_WARPS < ntiles) fetch_pages(tt + 2 * DEC_WARPS, pg_nxt);
                }
                cp_async_commit();
            }
        }
        cp_async_wait<0>();
        __syncthreads();  // every warp is done with its tiles: the space becomes the merge buffer
        float* mbuf = reinterpret_cast<float*>(tiles);
        float* wm = mbuf + warp * (32 + 16 * D);  // m[16], l[16], o[16][D]
        if (tig == 0) {
            wm[g] = m[0]; wm[g + 8] = m[1];
            wm[16 + g] = l[0]; wm[16 + g + 8] = l[1];
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            int dim = dt * 8 + tig * 2;
            wm[32 + g * D + dim] = o[dt][0]; wm[32 + g * D + dim + 1] = o[dt][1];
            wm[32 + (g + 8) * D + dim] = o[dt][2]; wm[32 + (g + 8) * D + dim + 1] = o[dt][3];
        }
        __syncthreads();
        const size_t slot = (size_t)blockIdx.x + pair;
        for (int idx = tid; idx < G * D; idx += DEC_WARPS * 32) {
            int r = idx / D, i = idx % D;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, mbuf[w * (32 + 16 * D) + r]);
            float lsum = 0.f, acc = 0.f;
            if (mx > -INFINITY) {
#pragma unroll
                for (int w = 0; w < DEC_WARPS; ++w) {
                    const float* p = mbuf + w * (32 + 16 * D);
                    float f = fast_exp2(p[r] - mx);
                    lsum += p[16 + r] * f;
                    acc += p[32 + r * D + i] * f;
                }
            }
            if (parts == 1) {
                out[((size_t)row0 * nq + kvh * G + r) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
            } else {
                part_o[(slot * G + r) * D + i] = acc;
                if (i == 0) { part_ml[(slot * G + r) * 2] = mx; part_ml[(slot * G + r) * 2 + 1] = lsum; }
            }
        }
        if (parts > 1) {
            // count this segment in; the last one merges the pair's slots (first_block + pair ... in order)
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                int old = atomicAdd(counters + pair, 1);
                s_last = old == parts - 1;
                if (s_last) counters[pair] = 0;  // as it was found, for the next launch
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                const size_t slot0 = (size_t)first_block + pair;
                for (int idx = tid; idx < G * D; idx += DEC_WARPS * 32) {
                    int r = idx / D, i = idx % D;
                    float mx = -INFINITY;
                    for (int sp = 0; sp < parts; ++sp) mx = fmaxf(mx, __ldcg(part_ml + ((slot0 + sp) * G + r) * 2));
                    float lsum = 0.f, acc = 0.f;
                    if (mx > -INFINITY) {
                        for (int s0 = 0; s0 < parts; s0 += 4) {
                            float pm[4], pl[4], po[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {  // independent loads, in flight together
                                const bool on = s0 + j < parts;
                                const size_t sl = slot0 + (on ? s0 + j : 0);
                                pm[j] = on ? __ldcg(part_ml + (sl * G + r) * 2) : -INFINITY;
                                pl[j] = on ? __ldcg(part_ml + (sl * G + r) * 2 + 1) : 0.f;
                                po[j] = on ? __ldcg(part_o + (sl * G + r) * D + i) : 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (s0 + j < parts) {
                                    float f = fast_exp2(pm[j] - mx);
                                    lsum += pl[j] * f;
                                    acc += po[j] * f;
                                }
                        }
                    }
                    out[((size_t)row0 * nq + kvh * G + r) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
                }
            }
        }
        t += ntiles;
        __syncthreads();  // the merge buffer and the query tile are free for the next segment
    }
}

// ----------------------------------------------------------------------------- prefill (and mixed steps)
namespace {
constexpr int PF_KT = 64;                 // keys per tile
constexpr int PF_NK = PF_KT / 8;
constexpr int PF_MT = 1;  // m16 tiles per warp (two halve the fragment loads but cost half the resident warps: measured slower)
constexpr int PF_ROWS = 4 * 16 * PF_MT;   // (token, head) rows per block: 4 warps
constexpr int PF_STAGES = 2;
constexpr size_t PF_SMEM = (size_t)(PF_ROWS * LDS + PF_STAGES * 2 * PF_KT * LDS) * sizeof(bf16);
}  // namespace

__global__ void __launch_bounds__(128)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache, CacheLayout L,
                    const int* __restrict__ meta, int group, const int* __restrict__ cu_tokens,
                    const int* __restrict__ ctx_lens, bf16* __restrict__ out, int nq, int window, float scale_log2,
                    int num_pages, int bt_cap, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qtile = reinterpret_cast<bf16*>(smem_raw);
    bf16* kv = qtile + PF_ROWS * LDS;
    int* bt_s = reinterpret_cast<int*>(smem_raw + PF_SMEM);
    pdl_launch_dependents();
    pdl_wait();
    // late query tiles see the most keys: they go first, so the longest blocks are not the last to start
    const int qt = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = nq / L.num_kv_heads;
    const int TPT = PF_ROWS / G;  // tokens per tile
    const int row0 = cu_tokens[e], q_len = cu_tokens[e + 1] - row0, ctx = ctx_lens[e];
    const int t0 = qt * TPT;
    if (t0 >= q_len) return;
    const int nt = min(TPT, q_len - t0);
    const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)e * meta[META_BT_STRIDE + group];

    for (int idx = tid; idx < PF_ROWS * (D / 8); idx += 128) {
        int r = idx / (D / 8), c = idx % (D / 8);
        int tok = r / G, hd = r % G;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (tok < nt)
            v = *reinterpret_cast<const uint4*>(q + (size_t)(row0 + t0 + tok) * q_stride + (size_t)(kvh * G + hd) * D + c * 8);
        *reinterpret_cast<uint4*>(qtile + toff(r, c * 8)) = v;
    }
    const int p_first = ctx + t0, p_last = p_first + nt - 1;
    const int kbeg = window > 0 ? max(0, p_first - window + 1) : 0, kend = p_last + 1;
    const int k_first = (kbeg / PF_KT) * PF_KT;
    const int ntiles = (kend - k_first + PF_KT - 1) / PF_KT;
    const int page_lo = kbeg / L.page_size;
    int page_cnt = (kend - 1) / L.page_size - page_lo + 1;
    if (page_cnt > bt_cap) {
        if (tid == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + kend);
        page_cnt = bt_cap;
    }
    stage_block_table(bt_s, bt, page_lo, page_cnt, num_pages, tid, 128, status);
    const int kend_s = min(kend, (page_lo + page_cnt) * L.page_size);
    __syncthreads();  // the Q tile and the table slice are written
    auto load_tile = [&](int t, int stage) {
        bf16* k = kv + stage * 2 * PF_KT * LDS;
        load_kv_tile(k, k + PF_KT * LDS, cache, L, bt_s, page_lo, kvh, k_first + t * PF_KT, PF_KT, kbeg, kend_s, tid, 128);
    };
    load_tile(0, 0);
    cp_async_commit();
    const int wrow = warp * 16 * PF_MT;  // first row of this warp
    const bf16* qwarp = qtile + wrow * LDS;
    uint32_t qf[PF_MT][Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[mt][ks], qwarp + mt * 16 * LDS, ks, lane);
    }
    // positions of this thread's rows (-1: a padding row, sees nothing)
    int prow[PF_MT][2];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int tok = (wrow + mt * 16 + (lane >> 2) + 8 * h) / G;
            prow[mt][h] = tok < nt ? p_first + tok : -1;
        }
    const int warp_first_tok = wrow / G, warp_last_tok_all = (wrow + 16 * PF_MT - 1) / G;
    const int warp_last_tok = min(nt - 1, warp_last_tok_all);
    const int warp_pmax = warp_first_tok < nt ? p_first + warp_last_tok : -1;
    const int warp_pmin = p_first + warp_first_tok;
    const int warp_kmin = window > 0 ? max(0, p_first + warp_first_tok - window + 1) : 0;
    const bool has_padding = warp_last_tok_all >= nt;

    float m[PF_MT][2], l[PF_MT][2];
    float o[PF_MT][DTILES][4];
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt) {
        m[mt][0] = m[mt][1] = -INFINITY;
        l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) o[mt][dt][0] = o[mt][dt][1] = o[mt][dt][2] = o[mt][dt][3] = 0.f;
    }

    for (int t = 0; t < ntiles; ++t) {
        const int stage = t & 1;
        if (t + 1 < ntiles) {
            load_tile(t + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int k0 = k_first + t * PF_KT;
        if (k0 <= warp_pmax && k0 + PF_KT > warp_kmin) {  // the tile holds keys some row of this warp sees
            const bf16* ktile = kv + stage * 2 * PF_KT * LDS;
            const bf16* vtile = ktile + PF_KT * LDS;
            float s[PF_MT][PF_NK][4];
#pragma unroll
            for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
                for (int n = 0; n < PF_NK; ++n) s[mt][n][0] = s[mt][n][1] = s[mt][n][2] = s[mt][n][3] = 0.f;
            // S = Q K^T: a key fragment is loaded once and multiplied into every m-tile of the warp
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t a[PF_MT][4];
#pragma unroll
                for (int mt = 0; mt < PF_MT; ++mt) {
                    if (Q_IN_REGS) { a[mt][0] = qf[mt][ks][0]; a[mt][1] = qf[mt][ks][1]; a[mt][2] = qf[mt][ks][2]; a[mt][3] = qf[mt][ks][3]; }
                    else load_a_frag(a[mt], qwarp + mt * 16 * LDS, ks, lane);
                }
#pragma unroll
                for (int np = 0; np < PF_NK / 2; ++np) {
                    uint32_t b[4];
                    int j = lane >> 3;
                    ldmatrix_x4(b, ktile + toff(np * 16 + (lane & 7) + (j >> 1) * 8, ks * 16 + (j & 1) * 8));
#pragma unroll
                    for (int mt = 0; mt < PF_MT; ++mt) {
                        mma_bf16(s[mt][2 * np], a[mt], b[0], b[1]);
                        mma_bf16(s[mt][2 * np + 1], a[mt], b[2], b[3]);
                    }
                }
            }
            // only tiles that cross a row's last visible key (or a window's edge, or the range's ends) need a mask
            const bool need_mask = has_padding || window > 0 || k0 + PF_KT - 1 > warp_pmin || k0 < kbeg;
#pragma unroll
            for (int mt = 0; mt < PF_MT; ++mt) {
#pragma unroll
                for (int n = 0; n < PF_NK; ++n)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        bool vis = true;
                        if (need_mask) {
                            int key = k0 + n * 8 + (lane & 3) * 2 + (c & 1);
                            int p = prow[mt][c >> 1];
                            vis = key <= p && (window <= 0 || p - key < window);
                        }
                        s[mt][n][c] = vis ? s[mt][n][c] * scale_log2 : -INFINITY;
                    }
                softmax_tile<PF_NK>(s[mt], m[mt], l[mt], o[mt]);
            }
            // O += P V: a value fragment likewise serves every m-tile
#pragma unroll
            for (int ks = 0; ks < PF_NK / 2; ++ks) {
                uint32_t a[PF_MT][4];
#pragma unroll
                for (int mt = 0; mt < PF_MT; ++mt) {
                    a[mt][0] = pack_bf16(s[mt][2 * ks][0], s[mt][2 * ks][1]);
                    a[mt][1] = pack_bf16(s[mt][2 * ks][2], s[mt][2 * ks][3]);
                    a[mt][2] = pack_bf16(s[mt][2 * ks + 1][0], s[mt][2 * ks + 1][1]);
                    a[mt][3] = pack_bf16(s[mt][2 * ks + 1][2], s[mt][2 * ks + 1][3]);
                }
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    uint32_t b[4];
                    int j = lane >> 3;
                    ldmatrix_x4_trans(b, vtile + toff(ks * 16 + (lane & 7) + (j & 1) * 8, dp * 16 + (j >> 1) * 8));
#pragma unroll
                    for (int mt = 0; mt < PF_MT; ++mt) {
                        mma_bf16(o[mt][2 * dp], a[mt], b[0], b[1]);
                        mma_bf16(o[mt][2 * dp + 1], a[mt], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();  // the stage may be overwritten by the load of the tile after next
    }
    const int g = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int mt = 0; mt < PF_MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int r = wrow + mt * 16 + g + 8 * h;
            int tok = r / G, hd = r % G;
            if (tok >= nt) continue;
            float inv = l[mt][h] > 0.f ? 1.f / l[mt][h] : 0.f;
            bf16* orow = out + ((size_t)(row0 + t0 + tok) * nq + kvh * G + hd) * D;
#pragma unroll
            for (int dt = 0; dt < DTILES; ++dt)
                *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + tig * 2) =
                    __floats2bfloat162_rn(o[mt][dt][2 * h] * inv, o[mt][dt][2 * h + 1] * inv);
        }
}

// ----------------------------------------------------------------------------- host side
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
int g_decode_tma = 0;
}  // namespace
// 1: the decode kernel loads pages by TMA where it can (head size 64, pages of 8, 16 or 32 tokens, no window);
// measured no faster than cp.async, so it is off unless asked for.
extern "C" void attn_set_decode_tma(int on) { g_decode_tma = on; }

extern "C" int attn_head_dim() { return D; }
// How many decode blocks a multiprocessor of the current device holds at once (shared memory and registers both
// count: large heads are bound by registers); the host sizes the splits by it.
extern "C" int attn_decode_blocks_per_sm() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DEC_BLOCKS_PER_SM;
    if (!cached[dev]) {
        int n = 0;
        const size_t smem = DEC_SMEM + 1024;
        if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_kernel, DEC_WARPS * 32, smem) != cudaSuccess || n < 1)
            n = DEC_BLOCKS_PER_SM;
        cached[dev] = n;
    }
    return cached[dev];
}
// The most splits that can merge through a cluster's shared memory (the portable cluster size).
extern "C" int attn_decode_max_cluster() { return DEC_MAX_CLUSTER; }

// Float32 words of scratch that attn_decode needs for `splits` > 1: partial outputs and (max, sum) pairs.
extern "C" size_t attn_decode_scratch_floats(int S, int nq, int splits) {
    return splits > 1 ? (size_t)S * nq * splits * (D + 2) : 0;
}

// The most splits the scratch-path merge takes: the block that merges stages a (max, sum) pair per (head of
// the group, split) in the shared memory of its key tiles.
extern "C" int attn_decode_max_splits(int nq, int nkv) {
    const int G = nkv > 0 && nq >= nkv ? nq / nkv : 1;
    return (int)(DEC_WARPS * DEC_WARP_ELEMS * sizeof(bf16) / ((size_t)G * 2 * sizeof(float)));
}

extern "C" int attn_prefill(const void* q, int q_stride, const void* cache, const int* meta, int group,
                            const int* cu_tokens, const int* ctx_lens, void* out, int S, int max_q_len, int nq, int nkv,
                            int page_size, int num_pages, int window, float scale, int max_context, int* status,
                            cudaStream_t stream) {
    if (S <= 0 || max_q_len <= 0) return 0;
    if (nq % nkv || nq / nkv > 16) return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, D};
    int tpt = PF_ROWS / (nq / nkv);
    dim3 grid((max_q_len + tpt - 1) / tpt, nkv, S);
    // block-table slice: the pages of the keys a tile can see (all of the context, or a window of it)
    int span = window > 0 ? min(max_context, window + tpt + PF_KT) : max_context;
    int bt_cap = span / page_size + 2;
    size_t smem = PF_SMEM + (size_t)bt_cap * sizeof(int);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured = 0;  // grows only, and is not set again inside a stream capture once large enough
    if (smem > configured) {
        cudaError_t err = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = smem;
    }
    return (int)launch_kernel(attn_prefill_kernel, grid, 128, smem, stream, (const bf16*)q, q_stride, (const bf16*)cache, L, meta,
                              group, cu_tokens, ctx_lens, (bf16*)out, nq, window, scale * LOG2E, num_pages, bt_cap, status);
}

namespace {
// The flat kernel's dynamic shared memory limit grows only (one place for both callers), and is not set
// again inside a stream capture once it is large enough.
cudaError_t flat_allow_smem(size_t smem) {
    static size_t configured = 0;
    if (smem <= configured) return cudaSuccess;
    cudaError_t err = cudaFuncSetAttribute(attn_decode_flat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err == cudaSuccess) configured = smem;
    return err;
}
}  // namespace

// How many blocks of the flat kernel the current GPU holds at once for S requests (its grid size).
extern "C" int attn_decode_flat_blocks(int S) {
    const size_t smem = FLAT_SMEM_FIXED + (size_t)(S + 1) * sizeof(int);
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (smem > 227 * 1024 || flat_allow_smem(smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_flat_kernel, DEC_WARPS * 32, smem) != cudaSuccess) return 0;
    return sms * per_sm;
}

// Floats of scratch for attn_decode_flat: a partial result per (block, pair) slot.
extern "C" size_t attn_decode_flat_scratch_floats(int S, int nq, int nkv, int blocks) {
    return (size_t)(blocks + S * nkv) * (nq / nkv) * (D + 2);
}

// Decode attention for large batches: `blocks` blocks share all key tiles evenly (see the kernel).  `scratch`:
// attn_decode_flat_scratch_floats(...) floats; `counters`: S * nkv ints, zero before the first launch (left zero).
extern "C" int attn_decode_flat(const void* q, int q_stride, const void* cache, const int* meta, int group,
                                const int* cu_tokens, const int* positions, void* out, float* scratch, int* counters,
                                const float* inv_freq, int rot, int store_kv, int S, int nq, int nkv, int page_size,
                                int num_pages, int window, float scale, int blocks, int* status, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (nq % nkv || nq / nkv > 16 || blocks < 1 || !scratch || !counters) return (int)cudaErrorInvalidValue;
    if (inv_freq && (rot % 2 || rot > D || rot <= 0)) return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, D};
    const size_t slots = (size_t)blocks + (size_t)S * nkv;
    float* part_o = scratch;
    float* part_ml = scratch + slots * (nq / nkv) * D;
    const size_t smem = FLAT_SMEM_FIXED + (size_t)(S + 1) * sizeof(int);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t err = flat_allow_smem(smem);
    if (err != cudaSuccess) return (int)err;
    return (int)launch_kernel(attn_decode_flat_kernel, blocks, DEC_WARPS * 32, smem, stream, (bf16*)q, q_stride, (bf16*)cache, L, meta,
                              group, cu_tokens, positions, (bf16*)out, part_o, part_ml, counters, inv_freq, rot, store_kv, nq,
                              window, scale * LOG2E, num_pages, S, status);
}

// `cluster_merge` (splits <= attn_decode_max_cluster()): the splits merge through the cluster's shared memory
// and neither scratch nor counters is touched.  Otherwise `scratch`: attn_decode_scratch_floats(...) floats when
// splits > 1, and `counters`: S * nkv ints, zero before the first launch (the kernel leaves them zero).  `inv_freq` (rot/2 floats) switches the fused rotation on: q is
// then the unrotated projection row and, with store_kv, the new key and value are written here too.
extern "C" int attn_decode(const void* q, int q_stride, const void* cache, const int* meta, int group,
                           const int* cu_tokens, const int* positions, void* out, float* scratch, int* counters,
                           const float* inv_freq, int rot, int store_kv, int S, int nq, int nkv, int page_size,
                           int num_pages, int window, float scale, int splits, int cluster_merge, int max_context,
                           int* status, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (nq % nkv || nq / nkv > 16 || splits < 1) return (int)cudaErrorInvalidValue;
    if (splits == 1) cluster_merge = 0;
    if (cluster_merge && splits > DEC_MAX_CLUSTER) return (int)cudaErrorInvalidValue;
    if (splits > 1 && !cluster_merge && (!scratch || !counters)) return (int)cudaErrorInvalidValue;
    if (splits > 1 && !cluster_merge && splits > attn_decode_max_splits(nq, nkv)) return (int)cudaErrorInvalidValue;
    if (inv_freq && (rot % 2 || rot > D || rot <= 0)) return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, D};
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)S * nq * splits * D : nullptr;
    (void)max_context;
    const size_t smem = DEC_SMEM + 1024;  // room to start the tiles on a 1024-byte boundary
    // Once per device: the attribute belongs to the device's copy of the kernel, and it is not set again
    // inside a stream capture.
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return (int)cudaErrorInvalidDevice;
    if (dev >= 64 || !configured[dev]) {
        cudaError_t err = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        if (dev < 64) configured[dev] = true;
    }
    // Page loads by TMA when a page's rows tile a warp's 32-key tile and start on its boundaries.
    CUtensorMap map;
    memset(&map, 0, sizeof map);
    int use_tma = 0;
    if (DEC_TMA && g_decode_tma && window <= 0 && (page_size == 8 || page_size == 16 || page_size == 32)) {
        static EncodeTiledFn fn = nullptr;
        if (!fn) {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult qres;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
                qres == cudaDriverEntryPointSuccess)
                fn = reinterpret_cast<EncodeTiledFn>(p);
        }
        if (fn) {
            // the layer's cache as a matrix: one row per (page, K|V, head, slot), HEAD_DIM columns
            cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * 2 * nkv * page_size};
            cuuint64_t strides[1] = {(cuuint64_t)D * 2};
            cuuint32_t box[2] = {(cuuint32_t)D, (cuuint32_t)page_size};
            cuuint32_t estr[2] = {1, 1};
            use_tma = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, nkv, S);
    cfg.blockDim = dim3(DEC_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster_merge) {  // the splits of a (request, head group) are one cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_use_pdl & 1) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, attn_decode_kernel, map, use_tma, (bf16*)q, q_stride, (bf16*)cache, L, meta, group,
                                   cu_tokens, positions, (bf16*)out, part_o, part_ml, counters, inv_freq, rot, store_kv, nq,
                                   window, scale * LOG2E, num_pages, splits, cluster_merge, status);
}
