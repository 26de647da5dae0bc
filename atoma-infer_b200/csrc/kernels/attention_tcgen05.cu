// Prefill attention on the 5th-generation tensor cores (-DHEAD_DIM=64 or 128).
//
// One block = 128 query rows ((token, query head of the group) pairs of one key/value head) of one
// request, walking that request's keys 128 at a time through the block table.  The block's warps
// have three jobs and talk through mbarriers only (no block-wide barrier inside the key loop):
//   * a copy warp: K and V pages travel by TMA (one box per page, 128-byte swizzle) straight from
//     the paged cache into two-stage shared-memory rings; the page ids come from the block table
//     in shared memory;
//   * an MMA warp (one elected thread): S = Q K^T is one tcgen05.mma chain (M = 128, N = 128,
//     K = head size) into one of two tensor-memory buffers; O_tile = P V is a second chain whose A
//     operand P is read from tensor memory and whose B operand V is read MN-major from shared
//     memory (no transpose copy);
//   * eight softmax warps, two threads per query row: a thread reads its half row of S from tensor
//     memory, masks by position, keeps the running max and sum (float32, base 2), writes P as
//     packed bfloat16 back into tensor memory over the scores it has consumed, and adds its half
//     of the previous tile's O_tile into its float32 output registers with the softmax correction.
// So the tensor core computes the next tile's scores and the last tile's P V while the softmax of
// the current tile runs, and the copies run two tiles ahead.  Two blocks fit a multiprocessor for
// head size 64; the softmax warps then take registers that the other two warps give up.
// A portion of a prompt that starts inside a cached context attends to all of it.
//
// The reference's prefill kernel is FlashAttention-2 for sm80 (csrc/kernels/flash_fwd_kernel.h:56-500,
// mma.sync m16n8k16, cp.async), which also cannot see a cached prefix (models/src/flash_attention.rs:384-410).
//
// All barrier waits are bounded; on a timeout the block raises a status word, every warp leaves its
// loop, and the block frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the tcgen05 attention kernel is built for head sizes 64 and 128");

int g_use_pdl = 0;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int D = HEAD_DIM;
constexpr int BQ = 128;            // query rows per block
constexpr int BKV = 128;           // keys per tile
constexpr int HALVES = D / 64;     // 64-column (128-byte) halves of a head
constexpr int HALF_BYTES = 128 * 128;  // a [128 rows x 64 columns] bfloat16 sub-tile
// Tensor memory: two buffers.  A buffer holds a tile's scores S (128 columns of float32).  P (128 keys as
// packed bfloat16: 64 columns) goes over them as the softmax reads them: keys 0..63 into columns 0..31
// and keys 64..127 into columns 96..127, so that each of a row's two threads overwrites its own scores
// only.  The tile's P V product takes the columns from O_COL on: between the halves of P for head
// size 64, behind the scores for 128.
constexpr uint32_t P_HI_COL = 96;
constexpr uint32_t O_COL = D == 64 ? 32 : 128;
constexpr uint32_t BUF_COLS = D == 64 ? 128 : 256;
constexpr uint32_t TMEM_COLS = 2 * BUF_COLS;
constexpr int SOFTMAX_THREADS = 256, SOFTMAX_WARPS = 8;
constexpr int COPY_WARP = 8, MMA_WARP = 9;
constexpr int TC_THREADS = 384;  // three warpgroups: two of softmax warps, one with the copy and the MMA warp
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;
#define STATUS_ATTN_TIMEOUT 3

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&status[STATUS_ATTN_TIMEOUT], 1 + (int)blockIdx.y);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
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
// 32 columns of this thread's lane, written from 32 registers (used for P: two bfloat16 keys a column)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D (tensor memory) = A (tensor memory: row = lane, two bfloat16 of K per column) * B (shared memory)
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Registers move between warpgroups: the copy/MMA warpgroup gives up what the softmax warpgroups take.
template <int N> __device__ __forceinline__ void regs_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void regs_take() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Descriptors of 128-byte-swizzled tiles whose rows are 128 bytes (64 bfloat16) and whose 8-row groups
// are 1024 bytes apart.  K-major: the 64 contiguous elements run along the MMA's K.  MN-major: they run
// along M or N, rows are K; `lbo` is then the distance between 64-wide halves.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands, A K-major, B K- or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
// byte offset of (row, 16-byte chunk c of a 64-column half) in a swizzled [rows x 64] sub-tile
__device__ __forceinline__ uint32_t swz(int row, int c) { return (uint32_t)row * 128u + (uint32_t)((c ^ (row & 7)) << 4); }

}  // namespace

__global__ void __launch_bounds__(TC_THREADS, HEAD_DIM == 64 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, int q_stride,
                       CacheLayout L, const int* __restrict__ meta, int group, const int* __restrict__ cu_tokens,
                       const int* __restrict__ ctx_lens, bf16* __restrict__ out, int nq, int window, float scale_log2,
                       int num_pages, int bt_cap, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int STAGE = HALVES * HALF_BYTES;  // one K or V tile: 128 rows of the head
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + STAGE;       // two stages
    unsigned char* v_s = k_s + 2 * STAGE;   // two stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * STAGE);
    // each [2]: K / V stage filled by TMA; scores / P V product of a buffer complete (tensor core);
    // P of a buffer written / O_tile of a buffer read (softmax warps)
    uint64_t *k_full = bars, *v_full = bars + 2, *s_done = bars + 4, *o_done = bars + 6, *p_ready = bars + 8, *o_read = bars + 10;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* row_max = reinterpret_cast<float*>(tmem_slot + 2);  // [2 sets][2 halves][128 rows]
    int* bt_s = reinterpret_cast<int*>(row_max + 4 * BQ);

    // Late query tiles see the most keys: they go first, for all heads before any earlier tile (blocks start in
    // the order of their linear index, x fastest), so the longest blocks are not the last to start.
    const int qt = gridDim.y - 1 - blockIdx.y, kvh = blockIdx.x, e = blockIdx.z;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = nq / L.num_kv_heads, TPT = BQ / G, ps = L.page_size;
    const int row0 = cu_tokens[e], q_len = cu_tokens[e + 1] - row0, ctx = ctx_lens[e];
    const int t0 = qt * TPT;
    if (t0 >= q_len) return;  // before anything is allocated
    const int nt = min(TPT, q_len - t0);
    const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)e * meta[META_BT_STRIDE + group];
    const int p_first = ctx + t0, p_last = p_first + nt - 1;
    const int kbeg = window > 0 ? max(0, p_first - window + 1) : 0, kend = p_last + 1;
    const int k_first = (kbeg / BKV) * BKV;
    const int ntiles = (kend - k_first + BKV - 1) / BKV;
    const int page_lo = k_first / ps;
    int page_cnt = (kend - 1) / ps - page_lo + 1;
    if (page_cnt > bt_cap) {
        if (tid == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + kend);
        page_cnt = bt_cap;
    }
    int bad = 0;
    for (int i = tid; i < page_cnt; i += TC_THREADS) {
        int page = bt[page_lo + i];
        // pages before the window's start may have been given back (-1): they are not read
        if (page >= num_pages || (page <= 0 && (page_lo + i + 1) * ps > kbeg)) {
            atomicExch(&status[STATUS_BAD_PAGE], 1 + (page_lo + i));
            page = -1;
            bad = 1;
        }
        bt_s[i] = page;
    }
    if (tid == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(&bars[i], 1);
        for (int i = 8; i < 12; ++i) mbar_init(&bars[i], SOFTMAX_WARPS);  // one arrival per softmax warp
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    // softmax threads: my query row; my half of the keys of a tile and of the head
    const int row = tid & (BQ - 1), half = (tid >> 7) & 1;
    const int my_tok = row / G, my_hd = row % G;
    const bool my_valid = my_tok < nt && row < TPT * G;  // group sizes that do not divide 128 leave padding rows
    const int my_pos = my_valid ? p_first + my_tok : -1;
    if (tid < SOFTMAX_THREADS) {  // my half of my query row, swizzled, straight into the A-operand tile
        const bf16* src = q + (size_t)(row0 + t0 + my_tok) * q_stride + (size_t)(kvh * G + my_hd) * D;
#pragma unroll
        for (int cc = 0; cc < D / 16; ++cc) {
            int c = half * (D / 16) + cc;
            uint4 v = my_valid ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(q_s + (c / 8) * HALF_BYTES + swz(row, c % 8)) = v;
        }
    }
    fence_async_smem();
    tc_fence_before();
    const bool any_bad = __syncthreads_or(bad) != 0;  // a table with holes where keys should be: every tile checks its V rows
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= SOFTMAX_WARPS) {
        if (D == 64) regs_release<32>();
        if (warp == COPY_WARP) {
            // ------------------------------------------------------------------ copies, two tiles ahead
            // The K (kv = 0) or V (kv = 1) rows of tile t: one box of `ps` rows per page, per 64-column half.
            // Lane 0 announces the bytes, then lane i starts the boxes of page i (starting a copy costs
            // about a hundred cycles; eight pages started by one thread would take eight times as long).
            auto issue_loads = [&](int t, int kv, unsigned char* dst, uint64_t* bar) {
                const int k0 = k_first + t * BKV;
                const int pg = lane, pidx = k0 / ps + pg - page_lo;
                const bool mine = pg < BKV / ps && pidx < page_cnt && bt_s[pidx] > 0;
                const uint32_t pages = __popc(__ballot_sync(0xffffffffu, mine));
                if (lane == 0) mbar_expect_tx(bar, pages * (uint32_t)ps * 128u * HALVES);
                __syncwarp();
                if (mine) {
                    int r = ((bt_s[pidx] * 2 + kv) * L.num_kv_heads + kvh) * ps;  // row of the page's first slot in the cache as a matrix
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(dst + h * HALF_BYTES + pg * ps * 128, &map_kv, h * 64, r, bar);
                }
            };
            int last_k[2] = {-1, -1}, last_v[2] = {-1, -1};  // the last tile whose copy was started into a stage
            for (int t = 0; t < 2 && t < ntiles; ++t) { issue_loads(t, 0, k_s + t * STAGE, &k_full[t]); last_k[t] = t; }
            for (int t = 0; t < 2 && t < ntiles; ++t) { issue_loads(t, 1, v_s + t * STAGE, &v_full[t]); last_v[t] = t; }
            bool ok = true;
            for (int t = 0; t + 2 < ntiles; ++t) {
                const int b = t & 1;
                const uint32_t par = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait(&s_done[b], par, status, abort_flag);  // the scores of tile t are done: its K stage is free
                if (!ok) break;
                issue_loads(t + 2, 0, k_s + b * STAGE, &k_full[b]);
                last_k[b] = t + 2;
                ok = mbar_wait(&o_done[b], par, status, abort_flag);  // P V of tile t is done: its V stage is free
                if (!ok) break;
                issue_loads(t + 2, 1, v_s + b * STAGE, &v_full[b]);
                last_v[b] = t + 2;
            }
            if (*abort_flag && lane == 0) {
                // somebody gave up on a barrier: let the copies in flight land (bounded) before the block leaves
                for (int b = 0; b < 2; ++b) {
                    if (last_k[b] >= 0)
                        for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(&k_full[b], (uint32_t)(last_k[b] >> 1) & 1u); ++i) {}
                    if (last_v[b] >= 0)
                        for (uint32_t i = 0; i < WAIT_LIMIT && !mbar_try_wait(&v_full[b], (uint32_t)(last_v[b] >> 1) & 1u); ++i) {}
                }
            }
        } else if (warp == MMA_WARP && lane == 0) {
            // ------------------------------------------------------------------ the tensor core's instruction stream
            constexpr uint32_t idesc_s = make_idesc(BQ, BKV, false), idesc_o = make_idesc(BQ, D, true);
            bool ok = true;
            auto issue_scores = [&](int t) {  // S(t) = Q K(t)^T into buffer t & 1
                const int b = t & 1;
                ok = mbar_wait(&k_full[b], (uint32_t)(t >> 1) & 1u, status, abort_flag);
                if (!ok) return;
                tc_fence_after();
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd) {
                    uint32_t off = (kd / 4) * HALF_BYTES + (kd % 4) * 32;
                    umma_bf16(tmem_base + b * BUF_COLS, make_desc(smem_u32(q_s) + off, 0),
                              make_desc(smem_u32(k_s) + b * STAGE + off, 0), idesc_s, kd > 0);
                }
                umma_commit(&s_done[b]);
            };
            issue_scores(0);
            if (ok && ntiles > 1) issue_scores(1);  // both buffers are free at the start
            for (int t = 0; t < ntiles && ok; ++t) {
                const int b = t & 1;
                const uint32_t par = (uint32_t)(t >> 1) & 1u;
                if (t >= 1 && t + 1 < ntiles) {
                    // the other buffer: the softmax warps take its last product (tile t - 1) in the middle of
                    // this tile's softmax; then the scores of tile t + 1 may overwrite it
                    ok = mbar_wait(&o_read[b ^ 1], (uint32_t)((t - 1) >> 1) & 1u, status, abort_flag);
                    if (!ok) break;
                    issue_scores(t + 1);
                    if (!ok) break;
                }
                ok = mbar_wait(&p_ready[b], par, status, abort_flag);  // P(t) is in tensor memory, V(t) is whole
                if (!ok) break;
                ok = mbar_wait(&v_full[b], par, status, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < BKV / 16; ++ks) {
                    uint64_t bd = make_desc(smem_u32(v_s) + b * STAGE + ks * 16 * 128, HALF_BYTES);
                    umma_bf16_a_tmem(tmem_base + b * BUF_COLS + O_COL, tmem_base + b * BUF_COLS + (ks < 4 ? ks * 8 : P_HI_COL + (ks - 4) * 8), bd,
                                     idesc_o, ks > 0);
                }
                umma_commit(&o_done[b]);
            }
        }
    } else {
        // ---------------------------------------------------------------------- softmax and output
        if (D == 64) regs_take<104>();
        const uint32_t tmem_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);  // a warp reaches the lanes of its quarter
        constexpr int DH = D / 2;  // my half of the head
        float m_run = -INFINITY, l_run = 0.f;  // l_run: the sum over my half of the keys only (the halves add up at the end)
        float corr_prev = 1.f;                 // the correction that belongs to the product not yet added
        float o[DH];
#pragma unroll
        for (int i = 0; i < DH; ++i) o[i] = 0.f;
        bool ok = true;
        // o = o * correction + my half row of P V of tile u, eight columns at a time (few registers: it
        // runs in the middle of a softmax); then the buffer is free for the scores of tile u + 2
        auto add_product = [&](int u) {
            const int b = u & 1;
            if (!mbar_wait(&o_done[b], (uint32_t)(u >> 1) & 1u, status, abort_flag)) ok = false;
            tc_fence_after();
#pragma unroll
            for (int ch = 0; ch < DH / 8; ++ch) {
                float v[8];
                tmem_ld8(tmem_row + b * BUF_COLS + O_COL + half * DH + ch * 8, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[ch * 8 + i] = o[ch * 8 + i] * corr_prev + v[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_read[b]);
        };

        // After a timeout anywhere in the block every wait returns at once and `ok` stays false, but the
        // loop still runs all its tiles: the two threads of a row meet at their barrier once per tile,
        // and one of them leaving early would leave the other waiting there for ever.
        for (int t = 0; t < ntiles; ++t) {
            const int k0 = k_first + t * BKV;
            const int b = t & 1;
            const uint32_t par = (uint32_t)(t >> 1) & 1u;
            const uint32_t tmem_buf = tmem_row + b * BUF_COLS;
            if (!mbar_wait(&s_done[b], par, status, abort_flag)) ok = false;
            tc_fence_after();

            // ---- softmax of my half row, in two passes over its 64 scores in tensor memory (16 at a time, so
            // that few registers are live): first the maximum, then the exponentials
            const bool need_mask = window > 0 || k0 + BKV - 1 > p_first || k0 < kbeg || nt < TPT;  // same for the whole block
            auto load_scores = [&](int c, float (&v)[16]) {  // unscaled: the scale goes into the exponent's FMA
                tmem_ld16(tmem_buf + half * 64 + c * 16, v);
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        int key = k0 + half * 64 + c * 16 + i;
                        bool vis = key <= my_pos && (window <= 0 || my_pos - key < window);
                        v[i] = vis ? v[i] : -INFINITY;
                    }
                }
            };
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[16];
                load_scores(c, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
            }
            // the row's maximum: the two threads of a row (warps w and w + 4) swap their halves' maxima through
            // shared memory and meet at a barrier of their own, 64 threads wide
            float* slot = row_max + (t & 1) * 2 * BQ;  // two sets, so that a fast pair cannot overwrite a slow reader's value
            slot[half * BQ + row] = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
            const float mx = fmaxf(slot[row], slot[BQ + row]) * scale_log2;  // scale > 0: the max commutes with it
            const float m_new = fmaxf(m_run, mx);
            const float base = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m_run - base);
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];  // my 64 keys of P, two to a column
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[16];
                load_scores(c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float p0 = fast_exp2(fmaf(v[2 * i], scale_log2, -base));
                    float p1 = fast_exp2(fmaf(v[2 * i + 1], scale_log2, -base));
                    __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);  // .x = p0 in the low half: the lower key
                    sum4[i & 3] += p0 + p1;
                    pk[c * 8 + i] = *reinterpret_cast<uint32_t*>(&two);
                }
                // ---- in between, the product of the tile before this one: the tensor core made it while this
                // tile's maximum was found, and once it is taken the scores of the next tile can start early
                if (c == 1 && t >= 1) add_product(t - 1);
            }
            // P goes over my own scores only (my partner may still be reading theirs): the first half row's
            // keys into columns 0..31, the second's into 96..127; the product lands between them
            tmem_st32(tmem_buf + half * 96, pk);
            l_run = l_run * corr + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            m_run = m_new;
            corr_prev = corr;

            // ---- V rows that no page delivered, or that lie beyond the last key, must be zero (0 * NaN would
            // poison P V): the last tile, a tile that starts before the window, a block table with holes
            if (k0 + BKV > kend || k0 < kbeg || any_bad) {
                if (!mbar_wait(&v_full[b], par, status, abort_flag)) ok = false;
                if (half == 0) {
                    int key = k0 + row, pidx = key / ps - page_lo;
                    bool have = key < kend && pidx < page_cnt && bt_s[pidx] > 0;
                    if (!have) {
#pragma unroll
                        for (int c = 0; c < D / 8; ++c)
                            *reinterpret_cast<uint4*>(v_s + b * STAGE + (c / 8) * HALF_BYTES + swz(row, c % 8)) = make_uint4(0u, 0u, 0u, 0u);
                        fence_async_smem();
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        if (ntiles > 0) add_product(ntiles - 1);

        // the two halves of a row saw the same maxima, so their sums simply add; the set of slots that
        // the next tile would have used is free (the pair has met since anybody read it)
        float* slot = row_max + (ntiles & 1) * 2 * BQ;
        slot[half * BQ + row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
        if (ok && my_valid) {
            const float l_all = slot[row] + slot[BQ + row];
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            bf16* dst = out + ((size_t)(row0 + t0 + my_tok) * nq + kvh * G + my_hd) * D + half * DH;
#pragma unroll
            for (int c = 0; c < DH / 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 two = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
                    w[i] = *reinterpret_cast<uint32_t*>(&two);
                }
                *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
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
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}
constexpr size_t TC_SMEM_FIXED = (size_t)(5 * HALVES) * HALF_BYTES + 12 * 8 + 16 + 4 * BQ * 4 + 1024;  // Q, 2 K, 2 V; barriers; slots; alignment
}  // namespace

extern "C" int attn_tc_head_dim() { return D; }

// Page sizes this kernel takes: one TMA box per page, boxes that tile a 128-key tile and start on a swizzle atom.
extern "C" int attn_prefill_tc_supports(int page_size, int nq, int nkv) {
    bool ps_ok = page_size >= 8 && page_size <= 128 && (page_size & (page_size - 1)) == 0;
    return ps_ok && nq % nkv == 0 && nq / nkv <= 16;
}

extern "C" int attn_prefill_tc(const void* q, int q_stride, const void* cache, const int* meta, int group,
                               const int* cu_tokens, const int* ctx_lens, void* out, int S, int max_q_len, int nq, int nkv,
                               int page_size, int num_pages, int window, float scale, int max_context, int* status,
                               cudaStream_t stream) {
    if (S <= 0 || max_q_len <= 0) return 0;
    if (!attn_prefill_tc_supports(page_size, nq, nkv)) return (int)cudaErrorInvalidValue;
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    // the layer's cache as a matrix: one row per (page, K|V, head, slot), HEAD_DIM columns
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)num_pages * 2 * nkv * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    cuuint32_t estr[2] = {1, 1};
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, D};
    const int tpt = BQ / (nq / nkv);
    int span = window > 0 ? min(max_context, window + tpt + 2 * BKV) : max_context;
    int bt_cap = span / page_size + 2 + BKV / page_size;
    size_t smem = TC_SMEM_FIXED + (size_t)bt_cap * sizeof(int);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t err = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = smem;
    }
    dim3 grid(nkv, (max_q_len + tpt - 1) / tpt, S);
    attn_prefill_tc_kernel<<<grid, TC_THREADS, smem, stream>>>(map, (const bf16*)q, q_stride, L, meta, group, cu_tokens, ctx_lens,
                                                        (bf16*)out, nq, window, scale * LOG2E, num_pages, bt_cap, status);
    LAUNCH_RETURN();
}
