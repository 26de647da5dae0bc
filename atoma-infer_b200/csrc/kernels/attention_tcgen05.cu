// Prefill attention on the 5th-generation tensor cores (-DHEAD_DIM=64 or 128).
//
// One block = 128 query rows ((token, query head of the group) pairs of one key/value head) of one
// request, walking that request's keys 128 at a time through the block table.  The block's warps
// have three jobs and talk through mbarriers only (no block-wide barrier inside the key loop):
//   * a copy warp: K and V pages travel by TMA (one box per page, 128-byte swizzle) straight from
//     the paged cache into two-stage shared-memory rings; the page ids come from the block table
//     in shared memory;
//   * an MMA warp (one elected thread): S = Q K^T is one tcgen05.mma chain (M = 128, N = 128,
//     K = head size) into tensor memory; O += P V is a second chain whose A operand P is read from
//     tensor memory and whose B operand V is read MN-major from shared memory (no transpose copy); O
//     stays in tensor memory from the first tile to the last;
//   * eight softmax warps, two threads per query row: a thread reads its half row of S from tensor
//     memory once (64 registers; the scores' columns are then free for the next tile's Q K^T), masks
//     by position, finds the row maximum with its partner, and writes P as packed bfloat16 into
//     tensor memory.  The base of the exponentials follows the maximum lazily: while the maximum
//     grows by less than 2^8 the old base stays, so O (in tensor memory) and the row sum are scaled
//     down only now and then, by the softmax threads, between two P V products.
// So the tensor core computes the next tile's scores while the exponentials of the current tile run,
// and the copies run two tiles ahead.  Two blocks fit a multiprocessor for
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
// Tensor memory of a block: the scores S of one tile (128 columns of float32), P (the tile's 128 keys as packed
// bfloat16, 64 columns) and the output accumulator O (head size columns of float32), which stays there for the whole
// key loop: P V of every tile is added to it by the tensor core itself.
constexpr uint32_t S_COL = 0, P_COL = 128, O_COL = 192;
constexpr uint32_t TMEM_COLS = D == 64 ? 256 : 512;
// The exponentials of a row use one base until the row's maximum has grown by more than this (in powers of two):
// only then are O and the row's sum scaled down.  P then stays below 2^8, far inside the range of bfloat16.
constexpr float RESCALE_STEP = 8.f;
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\ttcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 columns in two loads of 32 and one wait
__device__ __forceinline__ void tmem_ld32x2(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
                 "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
                 "tcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr), "r"(taddr + 32) : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 columns of this thread's lane, written from 32 float registers
__device__ __forceinline__ void tmem_st32f(uint32_t taddr, const float (&v)[32]) {
    uint32_t r[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(v[i]);
    tmem_st32(taddr, r);
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
    // k_full, v_full [2]: a K / V stage filled by TMA.  s_done, pv_done [2, by tile parity]: the scores / the P V
    // product of a tile complete (tensor core); they also free the tile's K / V stage.  s_free: every softmax warp has
    // the tile's scores in registers (the next Q K^T may overwrite them).  p_ready: every softmax warp has stored its
    // part of P (and scaled O if it had to).
    uint64_t *k_full = bars, *v_full = bars + 2, *s_done = bars + 4, *pv_done = bars + 6, *s_free = bars + 8, *p_ready = bars + 9;
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
        for (int i = 8; i < 10; ++i) mbar_init(&bars[i], SOFTMAX_WARPS);  // one arrival per softmax warp
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
                ok = mbar_wait(&pv_done[b], par, status, abort_flag);  // P V of tile t is done: its V stage is free
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
            auto issue_scores = [&](int t) {  // S(t) = Q K(t)^T
                const int b = t & 1;
                ok = mbar_wait(&k_full[b], (uint32_t)(t >> 1) & 1u, status, abort_flag);
                if (!ok) return;
                tc_fence_after();
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd) {
                    uint32_t off = (kd / 4) * HALF_BYTES + (kd % 4) * 32;
                    umma_bf16(tmem_base + S_COL, make_desc(smem_u32(q_s) + off, 0),
                              make_desc(smem_u32(k_s) + b * STAGE + off, 0), idesc_s, kd > 0);
                }
                umma_commit(&s_done[b]);
            };
            issue_scores(0);
            for (int t = 0; t < ntiles && ok; ++t) {
                const int b = t & 1;
                const uint32_t par = (uint32_t)(t >> 1) & 1u;
                if (t + 1 < ntiles) {
                    // the softmax warps hold the scores of tile t in registers: the next tile's may take their place
                    ok = mbar_wait(s_free, (uint32_t)t & 1u, status, abort_flag);
                    if (!ok) break;
                    issue_scores(t + 1);
                    if (!ok) break;
                }
                ok = mbar_wait(p_ready, (uint32_t)t & 1u, status, abort_flag);  // P(t) is in tensor memory, O is scaled
                if (!ok) break;
                ok = mbar_wait(&v_full[b], par, status, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < BKV / 16; ++ks) {
                    uint64_t bd = make_desc(smem_u32(v_s) + b * STAGE + ks * 16 * 128, HALF_BYTES);
                    umma_bf16_a_tmem(tmem_base + O_COL, tmem_base + P_COL + ks * 8, bd, idesc_o, (t > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(&pv_done[b]);
            }
        }
    } else {
        // ---------------------------------------------------------------------- softmax and output
        if (D == 64) regs_take<104>();
        const uint32_t tmem_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);  // a warp reaches the lanes of its quarter
        constexpr int DH = D / 2;  // my half of the head
        // m_run: the row's maximum so far; m_base: the base of the exponentials, which follows it lazily;
        // l_run: the sum over my half of the keys, in units of 2^m_base (the halves add up at the end)
        float m_run = -INFINITY, m_base = -INFINITY, l_run = 0.f;
        bool ok = true;

        // After a timeout anywhere in the block every wait returns at once and `ok` stays false, but the
        // loop still runs all its tiles: the two threads of a row meet at their barrier once per tile,
        // and one of them leaving early would leave the other waiting there for ever.
        for (int t = 0; t < ntiles; ++t) {
            const int k0 = k_first + t * BKV;
            const int b = t & 1;
            const uint32_t par = (uint32_t)(t >> 1) & 1u;
            if (!mbar_wait(&s_done[b], par, status, abort_flag)) ok = false;
            tc_fence_after();
            // ---- my half row of the scores, once, into registers; then the scores' columns are free
            float v[64];
            tmem_ld32x2(tmem_row + S_COL + half * 64, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);
            const bool need_mask = window > 0 || k0 + BKV - 1 > p_first || k0 < kbeg || nt < TPT;  // same for the whole block
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    int key = k0 + half * 64 + i;
                    bool vis = key <= my_pos && (window <= 0 || my_pos - key < window);
                    v[i] = vis ? v[i] : -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], v[i]);
            // the row's maximum: the two threads of a row (warps w and w + 4) swap their halves' maxima through
            // shared memory and meet at a barrier of their own, 64 threads wide
            float* slot = row_max + (t & 1) * 2 * BQ;  // two sets, so that a fast pair cannot overwrite a slow reader's value
            slot[half * BQ + row] = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
            const float mx = fmaxf(slot[row], slot[BQ + row]) * scale_log2;  // scale > 0: the max commutes with it
            m_run = fmaxf(m_run, mx);
            // The base moves only when the maximum has outgrown it by more than RESCALE_STEP (or at the first key
            // the row sees): both threads of a row decide alike, they hold the same numbers.
            const bool rebase = m_run > m_base + RESCALE_STEP || (m_base == -INFINITY && m_run > -INFINITY);
            const float corr = rebase ? fast_exp2(m_base - m_run) : 1.f;  // 0 for the first base
            if (rebase) m_base = m_run;
            const float base = m_base == -INFINITY ? 0.f : m_base;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[32];  // my 64 keys of P, two to a column
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float p0 = fast_exp2(fmaf(v[2 * i], scale_log2, -base));
                float p1 = fast_exp2(fmaf(v[2 * i + 1], scale_log2, -base));
                __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);  // .x = p0 in the low half: the lower key
                sum4[i & 3] += p0 + p1;
                pk[i] = *reinterpret_cast<uint32_t*>(&two);
            }
            l_run = l_run * corr + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            // ---- the product of the tile before must be complete before P is overwritten and before O is touched
            if (t >= 1) {
                if (!mbar_wait(&pv_done[b ^ 1], (uint32_t)((t - 1) >> 1) & 1u, status, abort_flag)) ok = false;
                tc_fence_after();
                // O (my half of the row) times the correction, if any row of this warp moved its base
                // (the loads and stores of tensor memory are warp-wide)
                if (__any_sync(0xffffffffu, rebase)) {
#pragma unroll
                    for (int ch = 0; ch < DH / 32; ++ch) {
                        float o[32];
                        tmem_ld32(tmem_row + O_COL + half * DH + ch * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= corr;
                        tmem_st32f(tmem_row + O_COL + half * DH + ch * 32, o);
                    }
                }
            }
            tmem_st32(tmem_row + P_COL + half * 32, pk);

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
            if (lane == 0) mbar_arrive(p_ready);
        }
        if (ntiles > 0) {
            if (!mbar_wait(&pv_done[(ntiles - 1) & 1], (uint32_t)((ntiles - 1) >> 1) & 1u, status, abort_flag)) ok = false;
            tc_fence_after();
        }

        // the two halves of a row used the same bases, so their sums simply add; the set of slots that
        // the next tile would have used is free (the pair has met since anybody read it)
        float* slot = row_max + (ntiles & 1) * 2 * BQ;
        slot[half * BQ + row] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
        const float l_all = slot[row] + slot[BQ + row];
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        bf16* dst = out + ((size_t)(row0 + t0 + my_tok) * nq + kvh * G + my_hd) * D + half * DH;
#pragma unroll
        for (int ch = 0; ch < DH / 32; ++ch) {
            float o[32];
            if (ntiles > 0) tmem_ld32(tmem_row + O_COL + half * DH + ch * 32, o);  // warp-wide: every lane takes part
            if (ok && my_valid) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 two = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&two);
                    }
                    *reinterpret_cast<uint4*>(dst + ch * 32 + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
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
