// A run of decoder layers of a decode step (at most 16 rows) as ONE persistent kernel, specialised by head
// size (-DHEAD_DIM=...).
//
// A decode step's time is the time to read every weight once.  Launched kernel by kernel, the weight stream
// stops at every kernel boundary: a linear of a few microseconds spends a third of its time starting and
// draining, and the norms and the attention between the linears read no weights at all.  Here one block per
// multiprocessor stays resident for all layers, and a warp of its own does nothing but stream the block's share
// of every weight matrix, in the order the layers use them, through a ring of 16 KB shared-memory stages: one
// tensor-map box a stage (`cp.async.bulk.tensor`, completion on an mbarrier), the matrix seen in 64-wide column
// groups so that a box lands as 128-byte-swizzled [rows][64] blocks that ldmatrix reads without bank conflicts.
// The stream depends on nothing the step computes, so it runs ahead of the arithmetic by the depth of the ring:
// while the blocks wait for each other between two phases or merge attention results, the next linears' weights
// keep arriving.  With pages of 16 keys and head size 64 or 128 the same warp streams the layer's keys and values.
//
// A layer is five phases with a grid-wide barrier after each (the layer of models/src/llama.rs:393-410):
//   1. the rows of x for the q/k/v projection by TMA into shared memory, and the projection;
//   2. rotation of q and k, the new key and value written to their page, attention over the cached pages: the
//      (request, head group) pairs dealt to the blocks, cut into blocks / pairs parts each;
//   3. output projection, added into the float32 residual;
//   4. the rows of x again, gate/up projection with the SwiGLU epilogue;
//   5. down projection (x in 512-wide chunks through a second, small ring), added into the residual.
// RMSNorm has no phase of its own: the epilogue of a phase that adds into the residual (3 and 5) also writes the new
// residual times the following norm's weight in bfloat16 (the next linear's x) and, per tile and row, the sum of
// squares; the next linear adds those up in a fixed order and scales its products' rows by 1 / rms, which commutes
// with the product.  (Every block computing the norm for itself, from the float32 rows, cost 8 to 9 us a norm: 148
// blocks reading the same fresh lines from L2, half of them across the two dies.)
// A linear's 16-row weight tiles (16 output columns) are dealt to the blocks like cards, the deal going on from
// phase to phase, so over a layer every block streams the same number of bytes, give or take a tile; a block
// multiplies a whole tile (all of K) itself: its arithmetic warps split each 512-wide stage between them
// and add up through shared memory in a fixed order, so a result does not depend on timing.  The weights are
// the A operand of mma.sync m16n8k16 and the rows of x the B operand, as in the stand-alone few-row linear.
//
// Every wait is bounded (mbarriers and the grid barrier alike).  A block whose wait runs out raises a status
// word and an abort flag and from then on waits for nothing: it walks the rest of the schedule (its results
// are void, the host sees the status word) and keeps counting itself in at the grid barriers, so no other
// block waits for it in vain, and it leaves only when the copies it issued have landed.
//
// The reference launches about 25 kernels a layer through candle (models/src/llama.rs:259-410).
#include <cuda.h>

#include <cstring>

#include "attention_tiles.cuh"

int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

#define STATUS_STACK_WAIT 4  // a block of this kernel gave up a wait: 1 + block index

namespace {

int g_stack_stream_kv = 1;           // set through decode_stack_set_stream_kv: keys and values through the ring where possible
int g_stack_max_split = 1 << 20;     // set through decode_stack_set_max_split
int g_stack_inflight = 0;            // set through decode_stack_set_inflight (0: ST_INFLIGHT)
long long* g_stack_times = nullptr;  // set through decode_stack_set_times: where the next launches leave their clocks

// Arithmetic warps.  Eight (two a scheduler, which hides the latencies of a stage's loads and multiply-adds behind
// each other) where the attention's registers allow it: with the stream warp that is 288 threads and at most 168
// registers a thread, which the walk over the keys fits into up to head size 64.  Larger heads: four (255 registers).
// (Eight at head size 128, with the query fragments read from shared memory for every tile, still spilt 400 bytes:
// the linears got slower, gate/up at Llama 3.1 8B sizes 42 -> 48 us, and the attention no faster.)
// The first four (DEC_WARPS) walk the keys when the stream cannot bring them.
constexpr int ST_WARPS = D <= 64 ? 8 : 4;
constexpr bool ST_Q_IN_REGS = Q_IN_REGS;
constexpr int ST_KB = 16 / ST_WARPS;           // 32-wide k blocks of a stage per warp
constexpr int ST_CONSUMERS = ST_WARPS * 32;
constexpr int ST_THREADS = ST_CONSUMERS + 32;  // and the warp that streams weights
constexpr int ST_KC = 512;                     // k per ring stage: eight groups of 64
constexpr int ST_STAGE_BYTES = 16 * ST_KC * 2; // 16 weight rows
constexpr int ST_MAX_STAGES = 12;
constexpr int ST_MIN_STAGES = 3;
// Stages asked for and not yet landed, per block.  What is in flight queues in the memory system ahead of every
// other read of the GPU, the arithmetic warps' dependent reads (the barrier's counter, queries, block tables) among
// them; the ring's other stages hold weights that have landed and wait to be used.
constexpr int ST_INFLIGHT = 6;
constexpr int ST_MAX_ROWS = 16;
constexpr int ST_XRING = 8;                    // most slots of the ring of x chunks
constexpr uint32_t ST_WAIT_POLLS = 1u << 22;   // about a quarter of a second
constexpr int BAR_CONSUMERS = 1, BAR_ATTENTION = 2, BAR_ALL = 3;

// A layer as the kernel sees it.  The weight matrices are tensor maps: a [N, K] row-major matrix seen as
// [K / 64][N][64] (the 64 contiguous, 128 bytes), so that one copy brings 16 rows x 512 k (or 8 x 512 for the
// stacked gate/up matrix: eight gate rows, then the eight up rows that belong to them) into shared memory as eight
// 128-byte-swizzled blocks of [rows][64], which ldmatrix reads without bank conflicts.
struct alignas(64) StackLayer {
    CUtensorMap map_qkv;      // [(nq + 2 nkv) D, H], box of 16 rows
    CUtensorMap map_o;        // [H, nq D], 16 rows
    CUtensorMap map_gate_up;  // [2 I, H], 8 rows
    CUtensorMap map_down;     // [H, I], 16 rows
    CUtensorMap map_cache;    // this layer's pages as rows of one head's keys (or values) at one slot, [pages * 2 * nkv * page_size][D] in 64-wide column blocks; a box is one page of one head
    const float* norm1;       // [H]
    const float* norm2;
    const float* inv_freq;    // [rot / 2]
    bf16* cache;              // this layer's pages
    int store_kv;             // 0: the layer reads another layer's cache and writes nothing
    int pad[7 + 16];
};
static_assert(sizeof(StackLayer) % 64 == 0, "descriptors lie back to back on 64-byte boundaries");

struct StackParams {
    const StackLayer* layers;
    float* resid;               // [M, H] float32 residual stream, updated in place
    const bf16* delta;          // optional [M, H]: still to be added to resid (done before the first layer)
    bf16* qkv;                  // workspace [M, (nq + 2 nkv) D]
    bf16* attn_out;             // workspace [M, nq D]
    bf16* act;                  // workspace [M, I]
    bf16* xw;                   // workspace [M, H]: the residual times the next norm's weight
    float* ss_part;             // workspace [ceil(H / 16)][16]: shares of the rows' sums of squares
    float* part_o;              // attention partial results: (blocks + S nkv) G D floats
    float* part_ml;             // and their (max, sum): (blocks + S nkv) G 2 floats
    int* counters;              // S nkv ints, zero before and after
    unsigned long long* arrivals;  // the grid barrier's counter: only ever grows, by the same amount every launch
    const int* meta;
    const int* cu_tokens;
    const int* positions;
    int* status;
    int num_layers, group, M, H, I, nq, nkv, rot, window, num_pages, page_size, S, stages, inflight, stream_kv, max_split;
    float eps, scale_log2;
    long long* times;           // optional [blocks][layers][10]: the clock after every phase and every barrier (measurements)
};

struct Linear {
    const CUtensorMap* map;
    int N, K, epi, tiles;  // epi 0: bfloat16 rows out; 1: silu(gate) * up; 2: added into the residual
};

__device__ __forceinline__ Linear phase_linear(const StackParams& p, const StackLayer* ly, int phase) {
    Linear l;
    if (phase == 0) { l.map = &ly->map_qkv; l.N = (p.nq + 2 * p.nkv) * D; l.K = p.H; l.epi = 0; }
    else if (phase == 1) { l.map = &ly->map_o; l.N = p.H; l.K = p.nq * D; l.epi = 2; }
    else if (phase == 2) { l.map = &ly->map_gate_up; l.N = 2 * p.I; l.K = p.H; l.epi = 1; }
    else { l.map = &ly->map_down; l.N = p.H; l.K = p.I; l.epi = 2; }
    l.tiles = l.epi == 1 ? (p.I + 7) / 8 : (l.N + 15) / 16;
    return l;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One box of a 3-d tensor map into shared memory; `hint`: an L2 eviction policy (weights are read once a step).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar,
                                                 uint64_t hint) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)), "l"(hint) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
// Before the copy engine reads global memory, or writes shared memory, that threads have written or used in the ordinary way.
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync %0, %1;" ::"n"(BAR_CONSUMERS), "n"(ST_CONSUMERS) : "memory"); }

// What a block knows about its own failure: once `flag` is set nothing waits any more.
struct Giveup {
    volatile int* flag;
    int* status;
    int code;
    __device__ __forceinline__ void raise() const {
        *flag = 1;
        atomicCAS(status + STATUS_STACK_WAIT, 0, code);
    }
};

// Bounded wait for a phase of a shared-memory barrier.  false: given up (now or earlier).
__device__ __forceinline__ bool wait_phase(uint64_t* bar, uint32_t parity, const Giveup& gu, bool heed_flag = true) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < ST_WAIT_POLLS; ++i) {
        if (heed_flag && *gu.flag) return false;
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 32) __nanosleep(32);
    }
    gu.raise();
    return false;
}

__device__ __forceinline__ void stamp(const StackParams& p, int layer, int slot, int tid) {
    if (p.times && tid == 0) {
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.times[((size_t)blockIdx.x * p.num_layers + layer) * 10 + slot] = t;
    }
}

// All blocks meet: everything written before it by any block is visible after it to every block.  The block's threads
// meet first; one of them counts the block in with release semantics (which covers what the others wrote before they
// met) and polls with acquire semantics; then the threads meet again.  (Without the fence below, a block's own tile of
// a linear came out as NaN now and then: the copy engine read a row of x that the block's other threads had just
// written, before it had left the multiprocessor.)
__device__ __forceinline__ void grid_barrier(const StackParams& p, unsigned long long& target, int tid, const Giveup& gu) {
    // What this thread wrote in the ordinary way (rows of x in global memory, tiles in shared memory) the copy engine
    // may read, or overwrite, after the barrier: every writer orders its own writes before the copy engine's accesses.
    fence_async();
    consumer_sync();
    if (tid == 0) {
        target += gridDim.x;
        asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p.arrivals), "l"(1ull) : "memory");
        if (!*gu.flag) {
            uint32_t polls = 0;
            while (ld_acquire(p.arrivals) < target) {
                if (++polls > ST_WAIT_POLLS || *gu.flag) { gu.raise(); break; }
                if (polls > 4096) __nanosleep(64);
            }
        }
    }
    consumer_sync();
}

// What a block keeps in shared memory.  Ring, region and the slots of the x ring start on 1,024-byte boundaries (the
// swizzle of a 128-byte row is a function of address bits 7 to 9).
struct BlockMem {
    unsigned char* ring_ptr;  // the ring as a generic pointer
    uint32_t ring;         // weight stages (shared-window addresses)
    unsigned char* region_ptr;  // the region as a generic pointer
    uint32_t region;       // rows of x for a linear, as [K / 64][rows][64] swizzled; or a ring of x chunks (eight groups
                           // of 64 each); or the attention's query tile and key/value stages
    uint64_t* full;        // [ST_MAX_STAGES] a stage has landed
    uint64_t* empty;       // [ST_MAX_STAGES] the arithmetic warps are done with a stage
    int xdepth;            // slots of the x ring
    uint64_t* xbar;        // the rows of x have landed
    uint64_t* xfull;       // [ST_XRING] a chunk of x has landed
    uint64_t* xempty;      // [ST_XRING]
    float* redbuf;         // two reduction buffers
    float* inv;            // [16] 1 / rms of the rows
};

// Where a block stands in its rings.
struct RingCursor {
    unsigned slot, parity;      // the weight stage that comes next and the parity of its "landed" phase
    unsigned deal;              // tiles dealt so far, over all phases
    unsigned tiles;             // tiles this block has finished (picks the reduction buffer)
    unsigned xslot, xparity;    // the same for the ring of x chunks
    unsigned xissue, xiparity;  // thread 0: the slot its next chunk of x goes to, and the parity of that slot's "free" phase
    unsigned xuse;              // parity of the next "rows of x have landed"
};

// All rows of x (a [M, width] bfloat16 matrix under `map`, boxes of `rows` rows) into the region; every arithmetic
// thread returns when they have landed.  The caller has made sure nobody still uses the region.
__device__ __forceinline__ void rows_to_region(const BlockMem& b, const CUtensorMap* map, int rows, int width, RingCursor& cur,
                                               int tid, const Giveup& gu) {
    if (tid == 0) {
        fence_async();
        mbar_expect_tx(b.xbar, (uint32_t)rows * (uint32_t)((width + 63) / 64) * 128u);
        tma_load_3d(b.region, map, 0, 0, 0, b.xbar);
    }
    // A linear reads x in chunks of eight groups of 64; beyond the last group of the rows the weights' stage holds
    // zeros, but the region holds whatever was there (a merge buffer of the attention, say), and zero times NaN is
    // NaN: the rest of the last chunk is zeroed.
    const int groups = (width + 63) / 64, upto = (groups + 7) / 8 * 8;
    if (upto > groups) {
        unsigned char* tail = b.region_ptr + (size_t)groups * rows * 128;
        for (int i = tid * 16; i < (upto - groups) * rows * 128; i += ST_CONSUMERS * 16)
            *reinterpret_cast<uint4*>(tail + i) = make_uint4(0u, 0u, 0u, 0u);
        consumer_sync();
    }
    wait_phase(b.xbar, cur.xuse, gu);
    cur.xuse ^= 1u;
}

// 1 / rms of every row from the sums of squares that `np` blocks left for it ([np][16] floats), added in a fixed order.
__device__ __forceinline__ void row_scales(float* inv, const float* ss_part, int np, int M, int H, float eps, int warp, int lane) {
    for (int m = warp; m < ST_MAX_ROWS; m += ST_WARPS) {
        float s = 0.f;
        if (m < M)
            for (int i = lane; i < np; i += 32) s += __ldcg(ss_part + (size_t)i * ST_MAX_ROWS + m);
        s = warp_sum(s);
        if (lane == 0) inv[m] = m < M ? rsqrtf(s / (float)H + eps) : 0.f;
    }
}

// What the epilogue of a linear that adds into the residual leaves for the norm after it.
struct NormFeed {
    const float* w;   // weight of the next norm (null: nothing follows inside this launch)
    bf16* xw;         // [M, H]: residual * w, rounded to bfloat16
    float* ss_part;   // [tiles][16]: this tile's share of every row's sum of squares
};

// One linear: this block's tiles, the weights from the ring.  XMODE 0: the rows of x lie in the region; 1: chunks of x
// (512 wide, like the weight stages) come through a ring in the region, asked for by thread 0 a few chunks ahead
// (`xmap`).  `inv` (optional): every row's result is scaled by inv[row] (the norm's 1 / rms, which commutes with the
// product).
template <int NT, int XMODE>
__device__ __forceinline__ void linear_phase(const StackParams& p, const Linear& lin, const BlockMem& b, RingCursor& cur,
                                             const CUtensorMap* xmap, bf16* out_bf16, const float* inv, const NormFeed& feed,
                                             int tid, const Giveup& gu) {
    constexpr int ROWS = NT * 8;
    constexpr int RED_STRIDE = ROWS + 1;
    constexpr int RED_FLOATS = ST_WARPS * 16 * RED_STRIDE;
    constexpr int XSLOT = ROWS * 1024;       // a chunk of x: eight groups of [ROWS][64]
    constexpr int XGROUP = ROWS * 128;       // one group
    const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
    const int ncta = gridDim.x, cta = blockIdx.x;
    const int K = lin.K, nchunks = (K + ST_KC - 1) / ST_KC;
    const int n_out = lin.epi == 1 ? lin.N / 2 : lin.N, out_rows = lin.epi == 1 ? 8 : 16;
    const int stages = p.stages, M = p.M;
    const int first = (cta + ncta - (int)(cur.deal % (unsigned)ncta)) % ncta;
    const int mine = first < lin.tiles ? (lin.tiles - first + ncta - 1) / ncta : 0;
    const unsigned xdepth = (unsigned)b.xdepth, ahead = xdepth - 1;
    const unsigned xtotal = (unsigned)mine * (unsigned)nchunks;
    // where the two halves of a tile's 16 rows lie in a stage: one box of 16 rows ([group][16][64]), or, for the stacked
    // gate/up matrix, two boxes of 8 ([group][8][64] twice)
    const uint32_t half_stride = lin.epi == 1 ? ST_STAGE_BYTES / 2 : 1024u, group_stride = lin.epi == 1 ? 1024u : 2048u;
    // this lane's part of the ldmatrix addresses: A takes matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15) of a 16 x 16
    // block, B the four k eighths of an 8-row, 32-wide block of x
    const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, akc = lane >> 4, brow = lane & 7, bkc = lane >> 3;
    const uint32_t a_lane = (uint32_t)(arow >> 3) * half_stride + (uint32_t)(arow & 7) * 128u;
    int xc = 0;  // chunk index of the next chunk of x to ask for
    auto x_issue = [&]() {  // thread 0: the next chunk of x into the next slot of the x ring
        const unsigned slot = cur.xissue;
        wait_phase(b.xempty + slot, cur.xiparity, gu);
        mbar_expect_tx(b.xfull + slot, (uint32_t)XSLOT);
        tma_load_3d(b.region + slot * XSLOT, xmap, 0, 0, xc * (ST_KC / 64), b.xfull + slot);
        if (++xc == nchunks) xc = 0;
        if (++cur.xissue == xdepth) { cur.xissue = 0; cur.xiparity ^= 1u; }
    };
    if (XMODE == 1 && tid == 0) {
        fence_async();
        for (unsigned f = 0; f < ahead && f < xtotal; ++f) x_issue();
    }
    unsigned f = 0;
    for (int tile = first; tile < lin.tiles; tile += ncta) {
        // a sum of its own for each of the warp's k blocks of a stage: the multiply-adds of a stage do not wait for each other
        float acc[ST_KB][NT][4];
#pragma unroll
        for (int u = 0; u < ST_KB; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) acc[u][t][0] = acc[u][t][1] = acc[u][t][2] = acc[u][t][3] = 0.f;
        for (int c = 0; c < nchunks; ++c, ++f) {
            uint32_t xbase;  // group 0 of this chunk of x
            unsigned xslot = 0;
            if (XMODE == 1) {
                if (tid == 0 && f + ahead < xtotal) x_issue();
                xslot = cur.xslot;
                wait_phase(b.xfull + xslot, cur.xparity, gu);
                xbase = b.region + xslot * XSLOT;
            } else {
                xbase = b.region + (uint32_t)c * (ST_KC / 64) * XGROUP;
            }
            const unsigned s = cur.slot;
            wait_phase(b.full + s, cur.parity, gu);
            const uint32_t st = b.ring + s * ST_STAGE_BYTES;
            uint32_t a[ST_KB][2][4], bq[ST_KB][NT][4];
#pragma unroll
            for (int u = 0; u < ST_KB; ++u) {  // every load of the stage first
                const int kb = warp * ST_KB + u, ko = kb >> 1, hb = kb & 1;
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int kc = (hb * 2 + jj) * 2 + akc;  // 16-byte chunk of the 128-byte row
                    ldsm_x4(a[u][jj], st + (uint32_t)ko * group_stride + a_lane + (uint32_t)((kc ^ (arow & 7)) << 4));
                }
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    ldsm_x4(bq[u][t], xbase + (uint32_t)ko * XGROUP + (uint32_t)(t * 8 + brow) * 128u + (uint32_t)(((hb * 4 + bkc) ^ brow) << 4));
            }
#pragma unroll
            for (int u = 0; u < ST_KB; ++u)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    mma_bf16(acc[u][t], a[u][0], bq[u][t][0], bq[u][t][1]);
                    mma_bf16(acc[u][t], a[u][1], bq[u][t][2], bq[u][t][3]);
                }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(b.empty + s);
                if (XMODE == 1) mbar_arrive(b.xempty + xslot);
            }
            if (++cur.slot == (unsigned)stages) { cur.slot = 0; cur.parity ^= 1u; }
            if (XMODE == 1 && ++cur.xslot == xdepth) { cur.xslot = 0; cur.xparity ^= 1u; }
        }
#pragma unroll
        for (int u = 1; u < ST_KB; ++u)  // in k order
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[0][t][e] += acc[u][t][e];
        // the tile's sums over the warps, in warp order
        float* red = b.redbuf + (cur.tiles & 1u) * RED_FLOATS;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float* r0 = red + (warp * 16 + g) * RED_STRIDE + t * 8 + tig * 2;
            float* r1 = red + (warp * 16 + g + 8) * RED_STRIDE + t * 8 + tig * 2;
            r0[0] = acc[0][t][0]; r0[1] = acc[0][t][1];
            r1[0] = acc[0][t][2]; r1[1] = acc[0][t][3];
        }
        consumer_sync();
        for (int idx = tid; idx < out_rows * ROWS; idx += ST_CONSUMERS) {  // whole warps take part or stay out
            const int m = idx / out_rows, r = idx % out_rows;  // consecutive threads, consecutive columns
            const int col = tile * out_rows + r;
            const bool on = m < M && col < n_out;
            float v = 0.f, u = 0.f;
#pragma unroll
            for (int wi = 0; wi < ST_WARPS; ++wi) {
                v += red[(wi * 16 + r) * RED_STRIDE + m];
                if (lin.epi == 1) u += red[(wi * 16 + r + 8) * RED_STRIDE + m];
            }
            if (lin.epi == 2) {
                // into the residual; and for the norm after it: the new value times the norm's weight, and the
                // tile's share of the row's sum of squares (the 16 lanes that hold a row's 16 columns add up)
                float now = 0.f;
                if (on) {
                    float* dst = p.resid + (size_t)m * n_out + col;
                    now = __ldcg(dst) + v;
                    __stcg(dst, now);
                    if (feed.w) feed.xw[(size_t)m * n_out + col] = __float2bfloat16_rn(now * feed.w[col]);
                }
                if (feed.w) {
                    float sq = now * now;
                    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                    if (r == 0) feed.ss_part[(size_t)tile * ST_MAX_ROWS + m] = m < M ? sq : 0.f;
                }
            } else if (on) {
                if (inv) { v *= inv[m]; u *= inv[m]; }
                if (lin.epi == 1) v = v / (1.f + expf(-v)) * u;
                out_bf16[(size_t)m * n_out + col] = __float2bfloat16_rn(v);
            }
        }
        ++cur.tiles;  // the other reduction buffer next: this one may still be read
    }
    cur.deal += (unsigned)lin.tiles;
}

// Before the first layer: every row's residual (plus what is still to be added to it) times the first norm's
// weight, and its sum of squares; a row a block.
__device__ __forceinline__ void feed_first_norm(const StackParams& p, const float* w, float* scratch, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    for (int m = blockIdx.x; m < p.M; m += gridDim.x) {
        float* r = p.resid + (size_t)m * p.H;
        const bf16* d = p.delta ? p.delta + (size_t)m * p.H : nullptr;
        float ss = 0.f;
        for (int i = tid * 4; i < p.H; i += ST_CONSUMERS * 4) {
            float4 v = *reinterpret_cast<const float4*>(r + i);
            if (d) {
                float dv[4];
                load4(d + i, dv);
                v.x += dv[0]; v.y += dv[1]; v.z += dv[2]; v.w += dv[3];
                *reinterpret_cast<float4*>(r + i) = v;
            }
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            const float4 wv = *reinterpret_cast<const float4*>(w + i);
            const float ov[4] = {v.x * wv.x, v.y * wv.y, v.z * wv.z, v.w * wv.w};
            store4(p.xw + (size_t)m * p.H + i, ov);
        }
        ss = warp_sum(ss);
        if (lane == 0) scratch[warp] = ss;
        consumer_sync();
        if (tid == 0) {
            float t = 0.f;
            for (int wi = 0; wi < ST_WARPS; ++wi) t += scratch[wi];
            p.ss_part[m] = t;
        }
        consumer_sync();
    }
}

// ----------------------------------------------------------------------------- attention from streamed keys and values
// With pages of 16 keys, head size 64 or 128 and no window, a page's keys (or values) of one head come as one box of
// the cache's tensor map: 16 rows, in 64-wide column blocks of [16][64] (one block at head size 64, two at 128), each
// 128-byte swizzled.  The stream warp then brings the keys and values too, between the q/k/v weights and the output
// projection's: the pages of a request are known before the step computes anything (only the newest position's key
// and value are not in them yet; the segment that owns that position puts them into its tile itself).  A 32-key tile
// is [K page 0][K page 1][V page 0][V page 1]; a stage holds two tiles at head size 64 and one at 128.
constexpr int KV_BLOCKS = D / 64;                       // column blocks of a row (streaming wants D % 64 == 0)
constexpr int KV_PAGE_BYTES = (KV_BLOCKS ? KV_BLOCKS : 1) * 2048;  // a page's keys (or values) of one head
constexpr int KV_TILE_BYTES = 4 * KV_PAGE_BYTES;
constexpr bool KV_STREAMABLE = D % 64 == 0 && KV_TILE_BYTES <= ST_STAGE_BYTES;
constexpr int KV_TILES_PER_STAGE = KV_STREAMABLE ? ST_STAGE_BYTES / KV_TILE_BYTES : 1;
constexpr int KV_PAGES_PER_STAGE = 2 * KV_TILES_PER_STAGE;
// byte offset of (key row r of the tile, dim c) from the tile's keys (the values lie 2 * KV_PAGE_BYTES further on)
__device__ __forceinline__ uint32_t kv_off(int r, int c) {
    return (uint32_t)((r >> 4) * KV_PAGE_BYTES + (c >> 6) * 2048 + (r & 15) * 128 + ((((c >> 3) & 7) ^ (r & 7)) << 4) + (c & 7) * 2);
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// S[16 x 32] = Q (fragments) * K^T for a streamed tile at shared-window address `keys`
__device__ __forceinline__ void qk_streamed(float (&sc)[DEC_NK][4], const uint32_t (*qf)[4], const bf16* qtile16, uint32_t keys, int lane) {
#pragma unroll
    for (int n = 0; n < DEC_NK; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        if (ST_Q_IN_REGS) { a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3]; }
        else load_a_frag(a, qtile16, ks, lane);
#pragma unroll
        for (int np = 0; np < DEC_NK / 2; ++np) {  // two n-tiles (16 keys) per ldmatrix.x4
            uint32_t bq[4];
            const int j = lane >> 3;
            ldsm_x4(bq, keys + kv_off(np * 16 + (lane & 7) + (j >> 1) * 8, ks * 16 + (j & 1) * 8));
            mma_bf16(sc[2 * np], a, bq[0], bq[1]);
            mma_bf16(sc[2 * np + 1], a, bq[2], bq[3]);
        }
    }
}
// O[16 x D] += P (from the score accumulators, bfloat16) * V for a streamed tile whose values start at `values`
__device__ __forceinline__ void pv_streamed(float (&o)[DTILES][4], const float (&sc)[DEC_NK][4], uint32_t values, int lane) {
#pragma unroll
    for (int ks = 0; ks < DEC_NK / 2; ++ks) {  // 16 keys per k-step
        const uint32_t a[4] = {pack_bf16(sc[2 * ks][0], sc[2 * ks][1]), pack_bf16(sc[2 * ks][2], sc[2 * ks][3]),
                               pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]), pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3])};
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {  // two n-tiles (16 dims) per ldmatrix.x4.trans
            uint32_t bq[4];
            const int j = lane >> 3;
            ldsm_x4_trans(bq, values + kv_off(ks * 16 + (lane & 7) + (j & 1) * 8, dp * 16 + (j >> 1) * 8));
            mma_bf16(o[2 * dp], a, bq[0], bq[1]);
            mma_bf16(o[2 * dp + 1], a, bq[2], bq[3]);
        }
    }
}

// The key tiles of all requests and head groups are dealt out evenly over the blocks as in flat_attention; a block's
// run is cut into segments at (request, head group) boundaries, a segment's tiles are packed two to a stage, and an
// arithmetic warp takes whole stages (stage i of the segment goes to warp i mod ST_WARPS).
// Which keys a block walks.  With at most as many (request, head group) pairs as blocks, every pair is cut into
// `split` = blocks / pairs parts of equal tile counts and block c takes part c % split of pair c / split: one segment a
// block (a segment costs about as much in staging the queries and merging as its tiles do, so one larger segment
// beats two smaller ones of the same total).  With more pairs than blocks, whole pairs are dealt out in turn.
struct KeySegment {
    int e, kvh, tile0, ntiles, pair, first_block, parts;
};
struct KeyWalk {
    int pairs, split, next;  // next: the next pair this block takes (pairs: none left)
};
__device__ __forceinline__ KeyWalk key_walk(int S, int nkv, int max_split) {
    KeyWalk w;
    w.pairs = S * nkv;
    w.split = w.pairs <= (int)gridDim.x ? min((int)gridDim.x / w.pairs, max_split) : 0;
    w.next = w.split ? ((int)blockIdx.x < w.pairs * w.split ? (int)blockIdx.x / w.split : w.pairs) : (int)blockIdx.x;
    return w;
}
// The block's next segment; false: none left.  A segment may be empty (ntiles <= 0) only when false is returned.
__device__ __forceinline__ bool key_segment(const int* prefix, int nkv, KeyWalk& w, KeySegment& sg) {
    while (w.next < w.pairs) {
        const int pair = w.next;
        w.next = w.split ? w.pairs : pair + (int)gridDim.x;
        sg.pair = pair;
        sg.e = pair / nkv;
        sg.kvh = pair % nkv;
        const int nt = prefix[sg.e + 1] - prefix[sg.e];
        if (nt <= 0) continue;  // a padded row of the batch
        if (w.split) {
            const int per = (nt + w.split - 1) / w.split, part = (int)blockIdx.x % w.split;
            sg.tile0 = part * per;
            sg.ntiles = min(nt, sg.tile0 + per) - sg.tile0;
            sg.first_block = pair * w.split;
            sg.parts = (nt + per - 1) / per;
            if (sg.ntiles <= 0) continue;
        } else {
            sg.tile0 = 0;
            sg.ntiles = nt;
            sg.first_block = (int)blockIdx.x;
            sg.parts = 1;
        }
        return true;
    }
    return false;
}

// This block's weight stages of the whole launch, in order: which box of which matrix comes next.  (Asking the boxes
// 16 to 64 stages further on into L2 as well, so that memory keeps working while the ring is full, was measured: the
// decode step of Llama 3.2 1B at batch 8 went from 1.01 to 1.09-1.13 ms.  The hints compete with the loads the
// arithmetic warps wait for.)
struct WeightWalk {
    int l, phase, tile, c;  // layer, linear of the layer, tile, 512-wide chunk of k
    unsigned deal;
    Linear lin;
    int nchunks;
    bool done;
    __device__ __forceinline__ void start(const StackParams& p) {
        l = 0; phase = -1; tile = 0; c = 0; deal = 0; done = false;
        lin.tiles = 0; lin.N = lin.K = lin.epi = 0; lin.map = nullptr; nchunks = 0;
        next_linear(p);
    }
    // the first tile of the next linear that has one for this block
    __device__ __forceinline__ void next_linear(const StackParams& p) {
        const int ncta = gridDim.x, cta = blockIdx.x;
        for (;;) {
            if (phase >= 0) deal += (unsigned)lin.tiles;
            if (++phase == 4) { phase = 0; ++l; }
            if (l >= p.num_layers) { done = true; return; }
            lin = phase_linear(p, p.layers + l, phase);
            nchunks = (lin.K + ST_KC - 1) / ST_KC;
            tile = (cta + ncta - (int)(deal % (unsigned)ncta)) % ncta;
            c = 0;
            if (tile < lin.tiles) return;
        }
    }
    __device__ __forceinline__ void advance(const StackParams& p) {
        if (++c < nchunks) return;
        c = 0;
        tile += gridDim.x;
        if (tile >= lin.tiles) next_linear(p);
    }
};

// The stream warp's part: this block's key and value pages of one layer into the ring.  All 32 lanes run it: a lane
// looks up a page, lane 0 counts the bytes in, the lanes ask for their pages.  false: given up.
__device__ __forceinline__ bool stream_keys(const StackParams& p, const BlockMem& b, const CUtensorMap* cache_map, const int* prefix,
                                            const int* kvlen, unsigned& count, unsigned& slot, unsigned& free_parity,
                                            unsigned& gate, unsigned& gate_parity, int lane, const Giveup& gu) {
    KeyWalk walk = key_walk(p.S, p.nkv, p.max_split);
    KeySegment sg;
    while (key_segment(prefix, p.nkv, walk, sg)) {
        const int lo = sg.tile0 * DEC_KT, hi = min(kvlen[sg.e], (sg.tile0 + sg.ntiles) * DEC_KT);
        const int page_lo = lo / 16, npages = (hi - lo + 15) / 16;
        const int* bt = p.meta + p.meta[META_BT_OFFSET + p.group] + (size_t)sg.e * p.meta[META_BT_STRIDE + p.group];
        for (int pb = 0; pb < npages; pb += 32) {  // 32 pages = 16 tiles a round
            int page = -1;
            if (pb + lane < npages) {
                page = __ldg(bt + page_lo + pb + lane);
                if (page <= 0 || page >= p.num_pages) {
                    atomicExch(&p.status[STATUS_BAD_PAGE], 1 + (page_lo + pb + lane) * 16);
                    page = -1;
                }
            }
            for (int sb = 0; sb < 32 / KV_PAGES_PER_STAGE && pb + sb * KV_PAGES_PER_STAGE < npages; ++sb) {
                const bool mine = lane / KV_PAGES_PER_STAGE == sb && page >= 0;
                const int landing = __popc(__ballot_sync(0xffffffffu, mine));
                if (!wait_phase(b.empty + slot, free_parity, gu)) return false;
                if (count >= (unsigned)p.inflight) {
                    if (!wait_phase(b.full + gate, gate_parity, gu)) return false;
                    if (++gate == (unsigned)p.stages) { gate = 0; gate_parity ^= 1u; }
                }
                if (lane == 0) mbar_expect_tx(b.full + slot, (uint32_t)landing * 2u * (uint32_t)KV_PAGE_BYTES);
                __syncwarp();
                if (mine) {  // page q of the stage: tile q / 2, page q % 2 of it; keys, then the values two pages further on
                    const int q = lane % KV_PAGES_PER_STAGE;
                    const uint32_t dst = b.ring + slot * ST_STAGE_BYTES + (uint32_t)(q >> 1) * KV_TILE_BYTES + (uint32_t)(q & 1) * KV_PAGE_BYTES;
                    tma_load_3d(dst, cache_map, 0, ((page * 2 + 0) * p.nkv + sg.kvh) * 16, 0, b.full + slot);
                    tma_load_3d(dst + 2u * KV_PAGE_BYTES, cache_map, 0, ((page * 2 + 1) * p.nkv + sg.kvh) * 16, 0, b.full + slot);
                }
                ++count;
                if (++slot == (unsigned)p.stages) { slot = 0; free_parity ^= 1u; }
            }
        }
    }
    return true;
}

// The arithmetic warps' part.  scratch: the region (query tile, the warps' merge buffers, the newest key and value).
__device__ __forceinline__ void streamed_attention(const StackParams& p, const BlockMem& b, const StackLayer* ly, RingCursor& cur,
                                                   unsigned char* region, const int* prefix, const int* kvlen, const float2* rope,
                                                   int* s_last, int tid, const Giveup& gu) {
    const int lane = tid & 31, warp = tid >> 5;
    const int nkv = p.nkv, G = p.nq / nkv, q_stride = (p.nq + 2 * nkv) * D;
    bf16* qtile = reinterpret_cast<bf16*>(region);
    float* mbuf = reinterpret_cast<float*>(region + 16 * LDS * sizeof(bf16));
    bf16* newest = reinterpret_cast<bf16*>(mbuf + ST_WARPS * (32 + 16 * D));  // [2][D]: the newest key (rotated) and value
    const CacheLayout L{nkv, p.page_size, D};
    KeyWalk walk = key_walk(p.S, nkv, p.max_split);
    KeySegment sg;
    unsigned stage0 = 0;  // stages of the phase before the current segment
    while (key_segment(prefix, nkv, walk, sg)) {
        const int row0 = p.cu_tokens[sg.e], kv_len = kvlen[sg.e], kvh = sg.kvh;
        const int lo = sg.tile0 * DEC_KT, hi = min(kv_len, (sg.tile0 + sg.ntiles) * DEC_KT);
        const bool owner = hi == kv_len;  // this segment holds the newest position
        const int half = p.rot / 2, pos = kv_len - 1;
        const bf16* row = p.qkv + (size_t)row0 * q_stride;
        // ---- the group's queries, rotated, into the tile; the newest key (rotated) and value
        const float2* cossin = rope + (size_t)sg.e * (D / 2);
        for (int idx = tid; idx < 16 * (D / 2); idx += ST_CONSUMERS) {
            const int r = idx / (D / 2), i = idx % (D / 2);
            if (r < G) {
                const bf16* x = row + (size_t)(kvh * G + r) * D;
                if (i < half) {
                    float a, c;
                    const float cs = cossin[i].x, sn = cossin[i].y;
                    rotate_pair(__bfloat162float(__ldcg(x + i)), __bfloat162float(__ldcg(x + i + half)), cs, sn, a, c);
                    qtile[toff(r, i)] = __float2bfloat16_rn(a);
                    qtile[toff(r, i + half)] = __float2bfloat16_rn(c);
                } else {  // dims beyond the rotated part, two to a slot
                    const int j = p.rot + 2 * (i - half);
                    qtile[toff(r, j)] = __ldcg(x + j);
                    qtile[toff(r, j + 1)] = __ldcg(x + j + 1);
                }
            } else {
                qtile[toff(r, 2 * i)] = __float2bfloat16_rn(0.f);
                qtile[toff(r, 2 * i + 1)] = __float2bfloat16_rn(0.f);
            }
        }
        if (owner) {
            const bf16* kx = row + (size_t)(p.nq + kvh) * D;
            const bf16* vx = row + (size_t)(p.nq + nkv + kvh) * D;
            for (int i = tid; i < half; i += ST_CONSUMERS) {
                float a, c;
                const float cs = cossin[i].x, sn = cossin[i].y;
                rotate_pair(__bfloat162float(__ldcg(kx + i)), __bfloat162float(__ldcg(kx + i + half)), cs, sn, a, c);
                newest[i] = __float2bfloat16_rn(a);
                newest[i + half] = __float2bfloat16_rn(c);
            }
            for (int i = p.rot + tid; i < D; i += ST_CONSUMERS) newest[i] = __ldcg(kx + i);
            for (int i = tid; i < D; i += ST_CONSUMERS) newest[D + i] = __ldcg(vx + i);
        }
        consumer_sync();
        if (owner && ly->store_kv) {  // to their page, for the steps to come
            const int* bt = p.meta + p.meta[META_BT_OFFSET + p.group] + (size_t)sg.e * p.meta[META_BT_STRIDE + p.group];
            const int page = bt[pos / p.page_size];
            if (page > 0 && page < p.num_pages) {
                for (int i = tid; i < 2 * D; i += ST_CONSUMERS)
                    ly->cache[L.offset(page, i / D, kvh, pos % p.page_size) + (i % D)] = newest[i];
            } else if (tid == 0) {
                atomicExch(&p.status[STATUS_BAD_PAGE], 1 + pos);
            }
        }
        uint32_t qf[ST_Q_IN_REGS ? KSTEPS : 1][4];
        if (ST_Q_IN_REGS) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[ks], qtile, ks, lane);
        }
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[DTILES][4];
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
        const int nstages = (sg.ntiles + KV_TILES_PER_STAGE - 1) / KV_TILES_PER_STAGE;
        // Which warp takes a stage is a matter of the ring slot it lies in (slot mod warps; the ring has a multiple of
        // ST_WARPS slots when keys are streamed): a warp then only ever waits for slots whose earlier contents it has
        // used itself.  A warp that waited for a slot another warp empties could find the slot's barrier a phase
        // behind (that stage still on its way) and, parities being one bit, take it for the phase it wants.
        const int first_si = (int)(((unsigned)warp + (unsigned)ST_WARPS - (cur.slot + stage0) % (unsigned)ST_WARPS) % (unsigned)ST_WARPS);
        for (int si = first_si; si < nstages; si += ST_WARPS) {
            const unsigned n = cur.slot + stage0 + (unsigned)si, slot = n % (unsigned)p.stages;
            wait_phase(b.full + slot, cur.parity ^ ((n / (unsigned)p.stages) & 1u), gu);
            unsigned char* st = b.ring_ptr + (size_t)slot * ST_STAGE_BYTES;
            const uint32_t st_addr = b.ring + slot * ST_STAGE_BYTES;
            bool wrote = false;
            for (int j = 0; j < KV_TILES_PER_STAGE && si * KV_TILES_PER_STAGE + j < sg.ntiles; ++j) {
                unsigned char* keys = st + j * KV_TILE_BYTES;
                unsigned char* values = keys + 2 * KV_PAGE_BYTES;
                const int k0 = lo + (si * KV_TILES_PER_STAGE + j) * DEC_KT;
                if (owner && pos >= k0 && pos < k0 + DEC_KT) {  // the tile with the newest position
                    const int r = pos - k0;  // its row; the rows after it hold nothing: their values must be zeros
                    for (int i = lane; i < D; i += 32) {
                        *reinterpret_cast<bf16*>(keys + kv_off(r, i)) = newest[i];
                        *reinterpret_cast<bf16*>(values + kv_off(r, i)) = newest[D + i];
                    }
                    for (int idx = lane; idx < (DEC_KT - 1 - r) * (D / 8); idx += 32) {
                        const int rr = r + 1 + idx / (D / 8), c8 = (idx % (D / 8)) * 8;
                        *reinterpret_cast<uint4*>(values + kv_off(rr, c8)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    wrote = true;
                    __syncwarp();
                }
                float sc[DEC_NK][4];
                qk_streamed(sc, qf, qtile, st_addr + j * KV_TILE_BYTES, lane);
#pragma unroll
                for (int nn = 0; nn < DEC_NK; ++nn)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int key = k0 + nn * 8 + (lane & 3) * 2 + (c & 1);
                        sc[nn][c] = key < hi ? sc[nn][c] * p.scale_log2 : -INFINITY;
                    }
                softmax_tile<DEC_NK>(sc, m, l, o);
                pv_streamed(o, sc, st_addr + j * KV_TILE_BYTES + 2 * KV_PAGE_BYTES, lane);
            }
            __syncwarp();
            if (wrote) fence_async();  // the copy engine writes this stage next
            if (lane == 0) mbar_arrive_n(b.empty + slot, ST_WARPS);  // this warp alone used the stage
        }
        consumer_sync();  // the queries have been read: their tile and the merge buffer may change
        decode_segment_finish<BAR_CONSUMERS, ST_WARPS>(mbuf, tid, m, l, o, sg.parts, sg.pair, sg.first_block, (int)blockIdx.x, row0, kvh, G, p.nq,
                                                       p.attn_out, p.part_o, p.part_ml, p.counters, s_last);
        stage0 += (unsigned)nstages;
        consumer_sync();
    }
    const unsigned n = cur.slot + stage0;
    cur.parity ^= (n / (unsigned)p.stages) & 1u;
    cur.slot = n % (unsigned)p.stages;
}

size_t stack_region_bytes(int M, int xwidth) {
    const size_t rows_bytes = (size_t)(M <= 8 ? 8 : 16) * (size_t)(((xwidth + 63) / 64 + 7) / 8 * 8) * 128;  // whole chunks of eight groups
    return ((rows_bytes > DEC_MAIN_BYTES ? rows_bytes : DEC_MAIN_BYTES) + 1023) / 1024 * 1024;
}

__global__ void __launch_bounds__(ST_THREADS, 1)
decode_stack_kernel(const StackParams p, const __grid_constant__ CUtensorMap map_xw, const __grid_constant__ CUtensorMap map_attn,
                    const __grid_constant__ CUtensorMap map_act, int region_bytes) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rows = p.M <= 8 ? 8 : 16;
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    BlockMem b;
    b.ring_ptr = smem;
    b.ring = smem_u32(smem);
    unsigned char* region = smem + (size_t)p.stages * ST_STAGE_BYTES;
    b.region_ptr = region;
    b.region = smem_u32(region);
    b.redbuf = reinterpret_cast<float*>(region + region_bytes);
    const int red_floats = 2 * ST_WARPS * 16 * (rows + 1);
    b.inv = b.redbuf + ((red_floats + 3) / 4) * 4;
    b.full = reinterpret_cast<uint64_t*>(b.inv + ST_MAX_ROWS);
    b.empty = b.full + ST_MAX_STAGES;
    b.xfull = b.empty + ST_MAX_STAGES;
    b.xempty = b.xfull + ST_XRING;
    b.xbar = b.xempty + ST_XRING;
    int* prefix = reinterpret_cast<int*>(b.xbar + 1);  // [ST_MAX_ROWS + 1]
    int* kvlen = prefix + ST_MAX_ROWS + 1;             // [ST_MAX_ROWS] keys of every request, the newest included
    int* s_last = kvlen + ST_MAX_ROWS;
    volatile int* gave_up = s_last + 1;
    float2* rope = reinterpret_cast<float2*>(s_last + 3);  // [ST_MAX_ROWS][D / 2] (cos, sin) of the requests' newest positions
    b.xdepth = region_bytes / (rows * 1024);
    if (b.xdepth > ST_XRING) b.xdepth = ST_XRING;
    const Giveup gu{gave_up, p.status, 1 + (int)blockIdx.x};

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(b.full + s, 1);
            mbar_init(b.empty + s, ST_WARPS);
        }
        for (int s = 0; s < ST_XRING; ++s) {
            mbar_init(b.xfull + s, 1);
            mbar_init(b.xempty + s, ST_WARPS);
        }
        mbar_init(b.xbar, 1);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == ST_WARPS) {
        // ---- the stream: this block's tiles of every linear of every layer, in order, and between a layer's q/k/v
        // and output projections its share of the layer's keys and values; lane 0 asks for the weights
        asm volatile("bar.sync %0, %1;" ::"n"(BAR_ALL), "n"(ST_THREADS) : "memory");  // the tile counts of the requests are there
        uint64_t policy;
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        unsigned count = 0;
        unsigned slot = 0, free_parity = 1u;  // the stage that comes next, the parity of its "free" phase
        unsigned gate = 0, gate_parity = 0u;  // the stage `inflight` before it, the parity of its "landed" phase
        WeightWalk at;                         // what the ring gets next
        at.start(p);
        int kv_next = 0;                       // the first layer whose keys and values have not been asked for yet
        bool on = true;
        while (on) {
            // a layer's keys and values come after this block's stages of its q/k/v matrix and before any later stage
            while (p.stream_kv && on && kv_next < p.num_layers && (at.done || 4 * kv_next < 4 * at.l + at.phase)) {
                on = stream_keys(p, b, &p.layers[kv_next].map_cache, prefix, kvlen, count, slot, free_parity, gate, gate_parity, lane, gu);
                ++kv_next;
            }
            if (at.done || !on) break;
            if (!wait_phase(b.empty + slot, free_parity, gu)) { on = false; break; }
            if (count >= (unsigned)p.inflight) {  // not too much on its way at once
                if (!wait_phase(b.full + gate, gate_parity, gu)) { on = false; break; }
                if (++gate == (unsigned)p.stages) { gate = 0; gate_parity ^= 1u; }
            }
            if (lane == 0) {
                const uint32_t dst = b.ring + slot * ST_STAGE_BYTES;
                const int k0 = at.c * (ST_KC / 64);
                mbar_expect_tx(b.full + slot, (uint32_t)ST_STAGE_BYTES);  // rows and k beyond the matrix arrive as zeros
                if (at.lin.epi == 1) {
                    tma_load_3d_hint(dst, at.lin.map, 0, at.tile * 8, k0, b.full + slot, policy);
                    tma_load_3d_hint(dst + ST_STAGE_BYTES / 2, at.lin.map, 0, at.lin.N / 2 + at.tile * 8, k0, b.full + slot, policy);
                } else {
                    tma_load_3d_hint(dst, at.lin.map, 0, at.tile * 16, k0, b.full + slot, policy);
                }
            }
            ++count;
            if (++slot == (unsigned)p.stages) { slot = 0; free_parity ^= 1u; }
            at.advance(p);
        }
        // nothing this warp asked for may still be on its way when the block leaves
        const unsigned issued = count, back = issued < (unsigned)p.stages ? issued : (unsigned)p.stages;
        for (unsigned i = issued - back; i < issued; ++i)
            wait_phase(b.full + i % (unsigned)p.stages, (i / (unsigned)p.stages) & 1u, gu, false);
    } else {
        // ---- the arithmetic
        const int NT = p.M <= 8 ? 1 : 2;
        const CacheLayout L{p.nkv, p.page_size, D};
        bf16* qtile = reinterpret_cast<bf16*>(region);
        bf16* tiles = qtile + 16 * LDS;
        unsigned long long target = 0;
        if (tid == 0) {
            const unsigned long long per_launch = ((unsigned long long)p.num_layers * 5ull + 1ull) * gridDim.x;
            target = ld_acquire(p.arrivals) / per_launch * per_launch;  // what it was when the launch began
        }
        if (warp < DEC_WARPS) flat_prefix<BAR_ATTENTION>(prefix, p.meta, p.cu_tokens, p.positions, p.S, p.window, tid);
        if (tid < ST_MAX_ROWS) kvlen[tid] = tid < min(p.S, p.meta[META_NUM_ENTRIES]) ? p.positions[p.cu_tokens[tid]] + 1 : 0;
        asm volatile("bar.sync %0, %1;" ::"n"(BAR_ALL), "n"(ST_THREADS) : "memory");  // the stream warp reads them
        RingCursor cur{0u, 0u, 0u, 0u, 0u, 0u, 0u, 1u, 0u};
        const int q_stride = (p.nq + 2 * p.nkv) * D;
        const int hidden_tiles = (p.H + 15) / 16;
        const NormFeed none{nullptr, nullptr, nullptr};
        feed_first_norm(p, p.layers[0].norm1, b.redbuf, tid);
        grid_barrier(p, target, tid, gu);
        int np = 1;  // blocks that left a share of the rows' sums of squares
        const float* rope_of = nullptr;  // the frequencies the (cos, sin) table was made from
        for (int l = 0; l < p.num_layers; ++l) {
            const StackLayer* ly = p.layers + l;
            // 1. the normed rows (their scale applied to the products), q/k/v
            rows_to_region(b, &map_xw, rows, p.H, cur, tid, gu);
            row_scales(b.inv, p.ss_part, np, p.M, p.H, p.eps, warp, lane);
            consumer_sync();
            if (NT == 1) linear_phase<1, 0>(p, phase_linear(p, ly, 0), b, cur, nullptr, p.qkv, b.inv, none, tid, gu);
            else linear_phase<2, 0>(p, phase_linear(p, ly, 0), b, cur, nullptr, p.qkv, b.inv, none, tid, gu);
            stamp(p, l, 0, tid);
            grid_barrier(p, target, tid, gu);
            stamp(p, l, 1, tid);
            // 2. attention
            if (p.stream_kv)
                {
                if (ly->inv_freq != rope_of) {  // (cos, sin) of every request's newest position; the same for all layers, as a rule
                    consumer_sync();
                    for (int idx = tid; idx < p.S * (p.rot / 2); idx += ST_CONSUMERS) {
                        const int e = idx / (p.rot / 2), i = idx % (p.rot / 2);
                        float sn, cs;
                        sincosf((float)(kvlen[e] - 1) * ly->inv_freq[i], &sn, &cs);
                        rope[e * (D / 2) + i] = make_float2(cs, sn);
                    }
                    rope_of = ly->inv_freq;
                    consumer_sync();
                }
                streamed_attention(p, b, ly, cur, region, prefix, kvlen, rope, s_last, tid, gu);
            }
            else if (warp < DEC_WARPS)
                flat_attention<BAR_ATTENTION>(blockIdx.x, gridDim.x, tid, qtile, tiles, prefix, s_last, p.qkv, q_stride, ly->cache, L, p.meta,
                                              p.group, p.cu_tokens, p.positions, p.attn_out, p.part_o, p.part_ml, p.counters, ly->inv_freq,
                                              p.rot, ly->store_kv, p.nq, p.window, p.scale_log2, p.num_pages, p.S, p.status);
            stamp(p, l, 2, tid);
            grid_barrier(p, target, tid, gu);
            stamp(p, l, 3, tid);
            // 3. output projection into the residual; feeds the second norm
            {
                const NormFeed feed{ly->norm2, p.xw, p.ss_part};
                rows_to_region(b, &map_attn, rows, p.nq * D, cur, tid, gu);
                if (NT == 1) linear_phase<1, 0>(p, phase_linear(p, ly, 1), b, cur, nullptr, nullptr, nullptr, feed, tid, gu);
                else linear_phase<2, 0>(p, phase_linear(p, ly, 1), b, cur, nullptr, nullptr, nullptr, feed, tid, gu);
                np = hidden_tiles;
            }
            stamp(p, l, 4, tid);
            grid_barrier(p, target, tid, gu);
            stamp(p, l, 5, tid);
            // 4. the normed rows, gate/up with SwiGLU
            rows_to_region(b, &map_xw, rows, p.H, cur, tid, gu);
            row_scales(b.inv, p.ss_part, np, p.M, p.H, p.eps, warp, lane);
            consumer_sync();
            if (NT == 1) linear_phase<1, 0>(p, phase_linear(p, ly, 2), b, cur, nullptr, p.act, b.inv, none, tid, gu);
            else linear_phase<2, 0>(p, phase_linear(p, ly, 2), b, cur, nullptr, p.act, b.inv, none, tid, gu);
            stamp(p, l, 6, tid);
            grid_barrier(p, target, tid, gu);
            stamp(p, l, 7, tid);
            // 5. down projection into the residual; feeds the next layer's first norm
            {
                const NormFeed feed{l + 1 < p.num_layers ? p.layers[l + 1].norm1 : nullptr, p.xw, p.ss_part};
                if (NT == 1) linear_phase<1, 1>(p, phase_linear(p, ly, 3), b, cur, &map_act, nullptr, nullptr, feed, tid, gu);
                else linear_phase<2, 1>(p, phase_linear(p, ly, 3), b, cur, &map_act, nullptr, nullptr, feed, tid, gu);
            }
            stamp(p, l, 8, tid);
            grid_barrier(p, target, tid, gu);
            stamp(p, l, 9, tid);
        }
    }
    asm volatile("bar.sync %0, %1;" ::"n"(BAR_ALL), "n"(ST_THREADS) : "memory");
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(q);
    }
    return fn;
}

// A [rows, K] bfloat16 row-major matrix (K a multiple of 64) seen as [K / 64][rows][64], boxes of `groups` x
// `box_rows` x 64 with the 128-byte swizzle; what lies beyond the matrix arrives as zeros.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows, int groups) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || K % 64 || rows <= 0 || ((uintptr_t)base & 15)) return false;
    alignas(64) CUtensorMap tmp;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)groups};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(map, &tmp, sizeof(tmp));
    return true;
}

// A layer's pages [pages, 2, nkv, 16, D] as rows of D in 64-wide column blocks: one box is a page's keys (or values) of
// one head, landing as D / 64 blocks of [16][64].
bool make_cache_map(CUtensorMap* map, const void* base, long long rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || rows <= 0 || ((uintptr_t)base & 15) || D % 64) return false;
    alignas(64) CUtensorMap tmp;
    cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(D / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, 128};
    cuuint32_t box[3] = {64, 16, (cuuint32_t)(D / 64)};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tmp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    memcpy(map, &tmp, sizeof(tmp));
    return true;
}

size_t stack_fixed_smem(int M, int xwidth) {
    const size_t red = (size_t)((2 * ST_WARPS * 16 * ((M <= 8 ? 8 : 16) + 1) + 3) / 4) * 4 * sizeof(float);
    return stack_region_bytes(M, xwidth) + red + ST_MAX_ROWS * sizeof(float) + (2 * ST_MAX_STAGES + 2 * ST_XRING + 1) * sizeof(uint64_t) +
           (2 * ST_MAX_ROWS + 1 + 2) * sizeof(int) + ST_MAX_ROWS * (D / 2) * sizeof(float2) + 1024 + 64;
}

struct StackPlan { int blocks, stages; size_t smem; };
// Grid and ring depth for M rows of width xwidth (the larger of the model's width and heads x head size) on the
// current device; blocks == 0: this geometry does not fit.
StackPlan stack_plan(int M, int xwidth) {
    StackPlan plan{0, 0, 0};
    int dev = 0, sms = 0, per_sm = 0, smem_max = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return plan;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return plan;
    if (cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return plan;
    const size_t fixed = stack_fixed_smem(M, xwidth);
    if (fixed + (size_t)ST_MIN_STAGES * ST_STAGE_BYTES > (size_t)smem_max) return plan;
    int stages = (int)(((size_t)smem_max - fixed) / ST_STAGE_BYTES);
    if (stages > ST_MAX_STAGES) stages = ST_MAX_STAGES;
    if (stages >= ST_WARPS) stages -= stages % ST_WARPS;  // whole rounds of the warps (see streamed_attention); fewer: keys are not streamed
    const size_t smem = fixed + (size_t)stages * ST_STAGE_BYTES;
    static size_t configured[64] = {};
    if (dev < 0 || dev >= 64) return plan;
    if (smem > configured[dev]) {
        if (cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return plan;
        configured[dev] = smem;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel, ST_THREADS, smem) != cudaSuccess || per_sm < 1) return plan;
    plan.blocks = sms;
    plan.stages = stages;
    plan.smem = smem;
    return plan;
}

}  // namespace

extern "C" int decode_stack_head_dim() { return D; }
extern "C" int decode_stack_layer_bytes() { return (int)sizeof(StackLayer); }
extern "C" int decode_stack_max_rows() { return ST_MAX_ROWS; }

// Writes one layer's descriptor (decode_stack_layer_bytes() bytes, host memory; the table of all layers then goes to
// the device, which must keep it on a 64-byte boundary).  Weights are bfloat16, row-major: w_qkv [(nq + 2 nkv) D, H],
// w_o [H, nq D], w_gate_up [2 I, H] (gate rows, then up rows), w_down [H, I]; H, nq D and I multiples of 64.  cache:
// the layer's pages [num_pages, 2, nkv, page_size, D].
// 0, or an error (the widths, or a tensor map the driver refused).
extern "C" int decode_stack_fill_layer(void* dst, const void* w_qkv, const void* w_o, const void* w_gate_up, const void* w_down,
                                       const float* norm1, const float* norm2, const float* inv_freq, void* cache, int store_kv,
                                       int H, int I, int nq, int nkv, int page_size, int num_pages) {
    StackLayer ly;
    memset(&ly, 0, sizeof(ly));
    if (H % 64 || I % 64 || (nq * D) % 64) return (int)cudaErrorInvalidValue;
    if (!make_map(&ly.map_qkv, w_qkv, (long long)(nq + 2 * nkv) * D, H, 16, ST_KC / 64) || !make_map(&ly.map_o, w_o, H, (long long)nq * D, 16, ST_KC / 64) ||
        !make_map(&ly.map_gate_up, w_gate_up, 2ll * I, H, 8, ST_KC / 64) || !make_map(&ly.map_down, w_down, H, I, 16, ST_KC / 64))
        return (int)cudaErrorInvalidValue;
    if (KV_STREAMABLE && page_size == 16 && !make_cache_map(&ly.map_cache, cache, (long long)num_pages * 2 * nkv * 16)) return (int)cudaErrorInvalidValue;
    ly.norm1 = norm1; ly.norm2 = norm2; ly.inv_freq = inv_freq; ly.cache = (bf16*)cache; ly.store_kv = store_kv;
    memcpy(dst, &ly, sizeof(ly));
    return 0;
}

// For tests and measurements: 0 = the attention fetches keys and values itself (the only way with a window, a head
// size other than 64 or 128, or pages other than 16), 1 (the default) = the stream warp brings them where it can.
extern "C" void decode_stack_set_stream_kv(int on) { g_stack_stream_kv = on; }

// For measurements: the most parts a (request, head group) pair is cut into (one part a pair at batch 8, 64 blocks
// walking 65 tiles each: the slowest block 21 us instead of 15; a block brings keys and values as 2 KB boxes, which
// the copy engine starts at about one per 80 cycles, 30 to 40 GB/s a block).
extern "C" void decode_stack_set_max_split(int parts) { g_stack_max_split = parts > 0 ? parts : 1; }

// For measurements: how many stages a block may have on their way at once (0: the default).
extern "C" void decode_stack_set_inflight(int stages) { g_stack_inflight = stages; }

// For measurements: a device buffer of blocks * layers * 10 64-bit words in which every block leaves the global
// clock after each phase and each barrier of each layer (null: off, the default).  Reading that clock costs a few
// hundred nanoseconds each time.
extern "C" void decode_stack_set_times(long long* buffer) { g_stack_times = buffer; }

// Blocks of the kernel for M rows of width xwidth = max(H, nq * head size) (0: the geometry does not fit this device's
// shared memory).
extern "C" int decode_stack_blocks(int M, int xwidth) { return stack_plan(M, xwidth).blocks; }

// Floats of scratch for the attention's partial results.
extern "C" size_t decode_stack_scratch_floats(int S, int nq, int nkv, int blocks) {
    return (size_t)(blocks + S * nkv) * (nq / nkv) * (D + 2);
}

// Runs `num_layers` layers (descriptors `layers` in device memory, written by decode_stack_fill_layer) on the M = S
// rows of a decode step.  resid [M, H] float32 is updated in place; delta (optional, bfloat16 [M, H]) is added to it
// on the way.  qkv, attn_out, act, xw ([M, H]): bfloat16 workspaces of M rows, 16-byte aligned; ss_part:
// ceil(H / 16) * 16 floats; scratch: decode_stack_scratch_floats(...) floats; counters: S * nkv ints, zero (left zero);
// arrivals: one 64-bit counter that belongs to this (layers, device) pair alone and starts at zero.  all_store_kv: every
// layer writes its own cache (a layer that reads another layer's pages needs what that layer wrote a moment ago, which
// a stream that runs ahead may miss: the attention then fetches keys and values itself).
extern "C" int decode_stack(const void* layers, int num_layers, void* resid, const void* delta, void* qkv, void* attn_out,
                            void* act, void* xw, float* ss_part, float* scratch, int* counters, unsigned long long* arrivals,
                            const int* meta, int group, const int* cu_tokens, const int* positions, int M, int S, int H, int I,
                            int nq, int nkv, int rot, int window, int page_size, int num_pages, float eps, float scale,
                            int all_store_kv, int* status, cudaStream_t stream) {
    if (num_layers <= 0 || M <= 0) return 0;
    if (M > ST_MAX_ROWS || S != M || H % 64 || I % 64 || (nq * D) % 64 || nq % nkv || nq / nkv > 16 || rot % 2 || rot > D || rot <= 0 ||
        ((uintptr_t)layers & 63))
        return (int)cudaErrorInvalidValue;
    const int xwidth = H > nq * D ? H : nq * D;
    const StackPlan plan = stack_plan(M, xwidth);
    if (!plan.blocks) return (int)cudaErrorInvalidConfiguration;
    const int rows = M <= 8 ? 8 : 16;
    CUtensorMap map_xw, map_attn, map_act;
    if (H / 64 > 256 || nq * D / 64 > 256) return (int)cudaErrorInvalidValue;  // a box has at most 256 groups
    if (!make_map(&map_xw, xw, M, H, rows, H / 64) || !make_map(&map_attn, attn_out, M, (long long)nq * D, rows, nq * D / 64) ||
        !make_map(&map_act, act, M, I, rows, ST_KC / 64))
        return (int)cudaErrorInvalidValue;
    StackParams p;
    p.layers = (const StackLayer*)layers;
    p.resid = (float*)resid;
    p.delta = (const bf16*)delta;
    p.qkv = (bf16*)qkv;
    p.attn_out = (bf16*)attn_out;
    p.act = (bf16*)act;
    p.xw = (bf16*)xw;
    p.ss_part = ss_part;
    const size_t slots = (size_t)plan.blocks + (size_t)S * nkv;
    p.part_o = scratch;
    p.part_ml = scratch + slots * (nq / nkv) * D;
    p.counters = counters;
    p.arrivals = arrivals;
    p.meta = meta;
    p.cu_tokens = cu_tokens;
    p.positions = positions;
    p.status = status;
    p.num_layers = num_layers; p.group = group; p.M = M; p.H = H; p.I = I; p.nq = nq; p.nkv = nkv; p.rot = rot;
    p.window = window; p.num_pages = num_pages; p.page_size = page_size; p.S = S; p.stages = plan.stages;
    p.eps = eps; p.scale_log2 = scale * LOG2E;
    p.times = g_stack_times;
    p.max_split = g_stack_max_split;
    p.stream_kv = (g_stack_stream_kv && all_store_kv && KV_STREAMABLE && page_size == 16 && window == 0 && plan.stages % ST_WARPS == 0) ? 1 : 0;
    p.inflight = g_stack_inflight > 0 ? g_stack_inflight : ST_INFLIGHT;
    if (p.inflight > p.stages) p.inflight = p.stages;
    const int region_bytes = (int)stack_region_bytes(M, xwidth);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.blocks, 1, 1);
    cfg.blockDim = dim3(ST_THREADS, 1, 1);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all blocks resident at once: they wait for each other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, decode_stack_kernel, p, map_xw, map_attn, map_act, region_bytes);
    if (err != cudaSuccess) return (int)err;
    LAUNCH_RETURN();
}
