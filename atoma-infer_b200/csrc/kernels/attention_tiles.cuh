// Tile machinery of the bfloat16 attention kernels, specialised by head size (-DHEAD_DIM=...): cp.async loads
// through the block table into padded or swizzled shared-memory tiles, ldmatrix, mma.sync m16n8k16 with float32
// accumulators, online softmax in float32 in base 2; and the body of the decode attention that deals all key tiles
// out evenly over a fixed number of blocks, as device functions, because two kernels run it: the stand-alone one
// and the decode step's persistent layer kernel.
#pragma once
#include <cuda.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
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

namespace {
// The end of a segment of a decode attention: the NW warps' partial results (m, l, o of the rows g and g + 8 of each
// thread's quad) merged in warp order; the segment's result written out if it covers its (request, head group) pair
// alone (parts == 1), else left in scratch slot (block + pair) and counted in, the last segment to arrive for the pair
// merging the pair's slots (first_block + pair ...) in order.  mbuf: NW * (32 + 16 * D) floats of shared memory that
// every warp is done using; the NW * 32 threads meet at hardware barrier BAR.
template <int BAR, int NW> __device__ __forceinline__ void seg_sync() { asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NW * 32) : "memory"); }
template <int BAR, int NW>
__device__ __forceinline__ void decode_segment_finish(float* mbuf, int tid, const float (&m)[2], const float (&l)[2],
                                                      const float (&o)[DTILES][4], int parts, int pair, int first_block, int block,
                                                      int row0, int kvh, int G, int nq, bf16* __restrict__ out,
                                                      float* __restrict__ part_o, float* __restrict__ part_ml,
                                                      int* __restrict__ counters, int* s_last) {
    const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, tig = lane & 3;
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
    seg_sync<BAR, NW>();
    const size_t slot = (size_t)block + pair;
    for (int idx = tid; idx < G * D; idx += NW * 32) {
        int r = idx / D, i = idx % D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mx = fmaxf(mx, mbuf[w * (32 + 16 * D) + r]);
        float lsum = 0.f, acc = 0.f;
        if (mx > -INFINITY) {
#pragma unroll
            for (int w = 0; w < NW; ++w) {
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
        seg_sync<BAR, NW>();
        if (tid == 0) {
            int old = atomicAdd(counters + pair, 1);
            (*s_last) = old == parts - 1;
            if ((*s_last)) counters[pair] = 0;  // as it was found, for the next launch
        }
        seg_sync<BAR, NW>();
        if ((*s_last)) {
            __threadfence();
            const size_t slot0 = (size_t)first_block + pair;
            for (int idx = tid; idx < G * D; idx += NW * 32) {
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
}

}  // namespace

// ----------------------------------------------------------------------------- decode, key tiles dealt out evenly
// The same attention for batches with more (request, head group) pairs than about half the blocks the GPU
// holds: there, one block per pair (or per fixed split of a pair) leaves a last partial wave of blocks that
// run almost alone.  Here the grid is as many blocks as the GPU holds at once and the 32-key tiles of all
// pairs, in (request, head group, key) order, are dealt out evenly: a block takes a contiguous run of
// tiles, which may end one pair and begin the next (a run is cut into segments at pair boundaries).  A
// pair that one block covers alone is written directly; otherwise every segment's partial result goes to
// scratch slot (block index + pair index), a pair's slots being consecutive, and the last block to arrive
// for the pair merges its slots in order.  No block waits for another.
//
// The 128 threads that run these functions meet at hardware barrier BAR (0 in a kernel of 128 threads: the same
// as __syncthreads).  Rows of q, and the newest key and value, are read past the first-level cache: in the
// persistent kernel other blocks wrote them a moment ago, into a buffer this block has read before.
namespace {
template <int BAR> __device__ __forceinline__ void flat_sync() { asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(DEC_WARPS * 32) : "memory"); }

// prefix[e] = 32-key tiles (one head group's worth) of the requests before e, e = 0 .. S; only the step's metadata is read
template <int BAR>
__device__ __forceinline__ void flat_prefix(int* prefix, const int* __restrict__ meta, const int* __restrict__ cu_tokens,
                                            const int* __restrict__ positions, int S, int window, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
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
    flat_sync<BAR>();
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
    flat_sync<BAR>();
}

// Block `block` of `nblocks` walks its run of tiles.  qtile [16][LDS], tiles: the warps' key/value stages (DEC_MAIN_BYTES
// in all, starting at qtile); prefix as flat_prefix left it; s_last: one int of shared memory.
template <int BAR>
__device__ __forceinline__ void flat_attention(int block, int nblocks, int tid, bf16* qtile, bf16* tiles, const int* prefix,
                                               int* s_last, const bf16* __restrict__ q, int q_stride, bf16* __restrict__ cache,
                                               CacheLayout L, const int* __restrict__ meta, int group,
                                               const int* __restrict__ cu_tokens, const int* __restrict__ positions,
                                               bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                                               int* __restrict__ counters, const float* __restrict__ inv_freq, int rot,
                                               int store_kv, int nq, int window, float scale_log2, int num_pages, int S,
                                               int* __restrict__ status) {
    const int lane = tid & 31, warp = tid >> 5;
    const int nkv = L.num_kv_heads, G = nq / nkv;
    const int total = prefix[S] * nkv;
    const int per = (total + nblocks - 1) / nblocks;  // tiles per block
    int t = block * per;
    const int t_end = min(total, t + per);
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
                        rotate_pair(__bfloat162float(__ldcg(x + i)), __bfloat162float(__ldcg(x + i + half)), cs, sn, a, b);
                        qtile[toff(r, i)] = __float2bfloat16_rn(a);
                        qtile[toff(r, i + half)] = __float2bfloat16_rn(b);
                    } else {  // dims beyond the rotated part, two to a slot
                        int j = rot + 2 * (i - half);
                        qtile[toff(r, j)] = __ldcg(x + j);
                        qtile[toff(r, j + 1)] = __ldcg(x + j + 1);
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
                        rotate_pair(__bfloat162float(__ldcg(kx + i)), __bfloat162float(__ldcg(kx + i + half)), cs, sn, a, b);
                        kd[i] = __float2bfloat16_rn(a);
                        kd[i + half] = __float2bfloat16_rn(b);
                    }
                    for (int i = rot + tid; i < D; i += DEC_WARPS * 32) kd[i] = __ldcg(kx + i);
                    for (int i = tid; i < D; i += DEC_WARPS * 32) vd[i] = __ldcg(vx + i);
                    __threadfence();
                }
            }
        } else {
            for (int idx = tid; idx < 16 * (D / 8); idx += DEC_WARPS * 32) {
                int r = idx / (D / 8), c = idx % (D / 8);
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (r < G) v = __ldcg(reinterpret_cast<const uint4*>(q + (size_t)row0 * q_stride + (size_t)(kvh * G + r) * D + c * 8));
                *reinterpret_cast<uint4*>(qtile + toff(r, c * 8)) = v;
            }
        }
        flat_sync<BAR>();
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
        flat_sync<BAR>();  // every warp is done with its tiles: the space becomes the merge buffer
        decode_segment_finish<BAR, DEC_WARPS>(reinterpret_cast<float*>(tiles), tid, m, l, o, parts, pair, first_block, block, row0, kvh, G,
                                              nq, out, part_o, part_ml, counters, s_last);
        t += ntiles;
        flat_sync<BAR>();  // the merge buffer and the query tile are free for the next segment
    }
}
}  // namespace
