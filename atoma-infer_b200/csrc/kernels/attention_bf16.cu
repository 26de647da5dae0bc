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
//    (more loads in flight) and merge at the end; with several splits the partial
//    results go to scratch memory and attn_combine merges them.
//
// The reference does both with FlashAttention-2 for sm80 (csrc/kernels/flash_fwd_kernel.h:
// compute_attn_1rowblock :56-500, compute_attn_1rowblock_splitkv :504-1092, combine
// :1131-1313), one query head per block in the paged case (csrc/src/lib.rs:1576-1602).
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head sizes 16..256 in steps of 16");

namespace {

constexpr int D = HEAD_DIM;
constexpr int LDS = D + 8;            // padded row: consecutive rows shift by 16 bytes, ldmatrix stays conflict-free
constexpr int KSTEPS = D / 16;        // k-steps of Q*K^T
constexpr int DTILES = D / 8;         // n-tiles of the output
constexpr bool Q_IN_REGS = D <= 128;  // larger heads reload Q fragments from shared memory
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

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
        bf16* kd = ktile + r * LDS + c;
        bf16* vd = vtile + r * LDS + c;
        int page = -1, slot = 0;
        if (pos >= lo && pos < hi) {
            int pidx = ps_shift >= 0 ? pos >> ps_shift : pos / ps;
            slot = pos - pidx * ps;
            page = bt_s[pidx - page_lo];
        }
        if (page > 0) {
            const bf16* src = cache + (size_t)page * page_stride + head_off + (size_t)slot * D + c;
            cp_async_16(kd, src);
            cp_async_16(kd + 8, src + 8);
            cp_async_16(vd, src + v_off);
            cp_async_16(vd + 8, src + v_off + 8);
        } else {
            uint4 z = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(kd) = z;
            *reinterpret_cast<uint4*>(kd + 8) = z;
            *reinterpret_cast<uint4*>(vd) = z;
            *reinterpret_cast<uint4*>(vd + 8) = z;
        }
    }
}

// A fragments (16 rows x 16 dims, k-step ks) of a row-major tile [16][LDS]
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const bf16* tile16, int ks, int lane) {
    int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = ks * 16 + (lane >> 4) * 8;
    ldmatrix_x4(a, tile16 + row * LDS + col);
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
            ldmatrix_x4(b, ktile + key * LDS + dim);
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
            ldmatrix_x4_trans(b, vtile + key * LDS + dim);
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
constexpr int DEC_STAGES = D <= 128 ? 2 : 1;
constexpr int DEC_WARP_ELEMS = DEC_STAGES * 2 * DEC_KT * LDS;  // bf16 elements of one warp's K/V stages
constexpr size_t DEC_TILE_BYTES = (size_t)(16 * LDS + DEC_WARPS * DEC_WARP_ELEMS) * sizeof(bf16);
constexpr size_t DEC_MERGE_BYTES = (size_t)DEC_WARPS * (32 + 16 * D) * sizeof(float);
constexpr size_t DEC_SMEM = 16 * LDS * sizeof(bf16) +
    (DEC_WARPS * DEC_WARP_ELEMS * sizeof(bf16) > DEC_MERGE_BYTES ? DEC_WARPS * DEC_WARP_ELEMS * sizeof(bf16) : DEC_MERGE_BYTES);
// + a slice of the block table, sized by the host (bt_cap entries)
}  // namespace

__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache, CacheLayout L,
                   const int* __restrict__ meta, int group, const int* __restrict__ cu_tokens,
                   const int* __restrict__ positions, bf16* __restrict__ out, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int nq, int window, float scale_log2, int num_pages, int splits,
                   int bt_cap, int* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* qtile = reinterpret_cast<bf16*>(smem_raw);
    bf16* tiles = qtile + 16 * LDS;
    int* bt_s = reinterpret_cast<int*>(smem_raw + DEC_SMEM);
    const int split = blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = nq / L.num_kv_heads;
    const int row0 = cu_tokens[e];
    const int kv_len = positions[row0] + 1;
    const int kstart = window > 0 ? max(0, kv_len - window) : 0;
    const int per = (((kv_len - kstart + splits - 1) / splits + DEC_KT - 1) / DEC_KT) * DEC_KT;
    const int lo = kstart + split * per, hi = min(kv_len, lo + per);
    const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)e * meta[META_BT_STRIDE + group];
    const int page_lo = lo / L.page_size;
    int page_cnt = lo < hi ? (hi - 1) / L.page_size - page_lo + 1 : 0;
    if (page_cnt > bt_cap) {  // the host sized the slice for a shorter context than this request has
        if (tid == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + hi);
        page_cnt = bt_cap;
    }
    stage_block_table(bt_s, bt, page_lo, page_cnt, num_pages, tid, DEC_WARPS * 32, status);
    const int hi_s = min(hi, (page_lo + page_cnt) * L.page_size);  // never beyond the staged slice

    for (int idx = tid; idx < 16 * (D / 8); idx += DEC_WARPS * 32) {
        int r = idx / (D / 8), c = idx % (D / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) v = *reinterpret_cast<const uint4*>(q + (size_t)row0 * q_stride + (size_t)(kvh * G + r) * D + c * 8);
        *reinterpret_cast<uint4*>(qtile + r * LDS + c * 8) = v;
    }
    __syncthreads();
    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[ks], qtile, ks, lane);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

    bf16* mine = tiles + warp * DEC_WARP_ELEMS;
    const int ntiles = lo < hi ? (hi - lo + DEC_KT - 1) / DEC_KT : 0;
    auto load_tile = [&](int t, int stage) {
        bf16* k = mine + stage * 2 * DEC_KT * LDS;
        load_kv_tile(k, k + DEC_KT * LDS, cache, L, bt_s, page_lo, kvh, lo + t * DEC_KT, DEC_KT, lo, hi_s, lane, 32);
    };
    if (warp < ntiles) load_tile(warp, 0);
    cp_async_commit();
    for (int t = warp, it = 0; t < ntiles; t += DEC_WARPS, ++it) {
        int stage = 0;
        if (DEC_STAGES == 2) {
            stage = it & 1;
            if (t + DEC_WARPS < ntiles) load_tile(t + DEC_WARPS, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const bf16* ktile = mine + stage * 2 * DEC_KT * LDS;
        const bf16* vtile = ktile + DEC_KT * LDS;
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
            if (t + DEC_WARPS < ntiles) load_tile(t + DEC_WARPS, 0);
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
        } else {
            size_t slot = ((size_t)e * nq + head) * splits + split;
            part_o[slot * D + i] = acc;
            if (i == 0) { part_ml[slot * 2] = mx; part_ml[slot * 2 + 1] = lsum; }
        }
    }
}

// Merges the splits of attn_decode: out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ meta, const int* __restrict__ cu_tokens,
                                    bf16* __restrict__ out, int nq, int splits) {
    const int head = blockIdx.x, e = blockIdx.y;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const size_t base = ((size_t)e * nq + head) * splits;
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float lsum = 0.f, acc = 0.f;
        if (mx > -INFINITY)
            for (int s = 0; s < splits; ++s) {
                float f = fast_exp2(part_ml[(base + s) * 2] - mx);
                lsum += part_ml[(base + s) * 2 + 1] * f;
                acc += part_o[(base + s) * D + i] * f;
            }
        out[((size_t)cu_tokens[e] * nq + head) * D + i] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    }
}

// ----------------------------------------------------------------------------- prefill (and mixed steps)
namespace {
constexpr int PF_KT = 64;    // keys per tile
constexpr int PF_NK = PF_KT / 8;
constexpr int PF_ROWS = 64;  // (token, head) rows per block: 4 warps x 16
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
    const int qt = blockIdx.x, kvh = blockIdx.y, e = blockIdx.z;
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
        *reinterpret_cast<uint4*>(qtile + r * LDS + c * 8) = v;
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
    const bf16* qwarp = qtile + warp * 16 * LDS;
    uint32_t qf[Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) load_a_frag(qf[ks], qwarp, ks, lane);
    }
    // positions of this thread's two rows (-1: a padding row, sees nothing)
    int prow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int tok = (warp * 16 + (lane >> 2) + 8 * h) / G;
        prow[h] = tok < nt ? p_first + tok : -1;
    }
    const int warp_first_tok = (warp * 16) / G, warp_last_tok = min(nt - 1, (warp * 16 + 15) / G);
    const int warp_pmax = warp_first_tok < nt ? p_first + warp_last_tok : -1;
    const int warp_kmin = window > 0 ? max(0, p_first + warp_first_tok - window + 1) : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DTILES][4];
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

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
            float s[PF_NK][4];
            qk_tile<PF_NK>(s, qf, qwarp, ktile, lane);
#pragma unroll
            for (int n = 0; n < PF_NK; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    int key = k0 + n * 8 + (lane & 3) * 2 + (c & 1);
                    int p = prow[c >> 1];
                    bool vis = key <= p && (window <= 0 || p - key < window);
                    s[n][c] = vis ? s[n][c] * scale_log2 : -INFINITY;
                }
            softmax_tile<PF_NK>(s, m, l, o);
            pv_tile<PF_NK>(o, s, vtile, lane);
        }
        __syncthreads();  // the stage may be overwritten by the load of the tile after next
    }
    const int g = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int r = warp * 16 + g + 8 * h;
        int tok = r / G, hd = r % G;
        if (tok >= nt) continue;
        float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        bf16* orow = out + ((size_t)(row0 + t0 + tok) * nq + kvh * G + hd) * D;
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt)
            *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + tig * 2) =
                __floats2bfloat162_rn(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
    }
}

// ----------------------------------------------------------------------------- host side
extern "C" int attn_head_dim() { return D; }

// Float32 words of scratch that attn_decode needs for `splits` > 1: partial outputs and (max, sum) pairs.
extern "C" size_t attn_decode_scratch_floats(int S, int nq, int splits) {
    return splits > 1 ? (size_t)S * nq * splits * (D + 2) : 0;
}

extern "C" int attn_prefill(const void* q, int q_stride, const void* cache, const int* meta, int group,
                            const int* cu_tokens, const int* ctx_lens, void* out, int S, int max_q_len, int nq, int nkv,
                            int page_size, int num_pages, int window, float scale, int max_context, int* status,
                            cudaStream_t stream) {
    if (S <= 0 || max_q_len <= 0) return 0;
    if (nq % nkv || nq / nkv > PF_ROWS) return (int)cudaErrorInvalidValue;
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
    attn_prefill_kernel<<<grid, 128, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)cache, L, meta, group, cu_tokens,
                                                      ctx_lens, (bf16*)out, nq, window, scale * LOG2E, num_pages, bt_cap, status);
    LAUNCH_RETURN();
}

extern "C" int attn_decode(const void* q, int q_stride, const void* cache, const int* meta, int group,
                           const int* cu_tokens, const int* positions, void* out, float* scratch, int S, int nq, int nkv,
                           int page_size, int num_pages, int window, float scale, int splits, int max_context,
                           int* status, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (nq % nkv || nq / nkv > 16 || splits < 1) return (int)cudaErrorInvalidValue;
    if (splits > 1 && !scratch) return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, D};
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)S * nq * splits * D : nullptr;
    int span = window > 0 ? min(max_context, window) : max_context;
    int per = (((span + splits - 1) / splits + DEC_KT - 1) / DEC_KT) * DEC_KT;  // keys of one split at most
    int bt_cap = per / page_size + 2;
    size_t smem = DEC_SMEM + (size_t)bt_cap * sizeof(int);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t err = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
        configured = smem;
    }
    dim3 grid(splits, nkv, S);
    attn_decode_kernel<<<grid, DEC_WARPS * 32, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)cache, L, meta, group,
                                                               cu_tokens, positions, (bf16*)out, part_o, part_ml, nq,
                                                               window, scale * LOG2E, num_pages, splits, bt_cap, status);
    if (splits > 1) {
        dim3 cgrid(nq, S);
        attn_combine_kernel<<<cgrid, D < 128 ? D : 128, 0, stream>>>(part_o, part_ml, meta, cu_tokens, (bf16*)out, nq, splits);
    }
    LAUNCH_RETURN();
}
