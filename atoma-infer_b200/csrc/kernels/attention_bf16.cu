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

#include "attention_tiles.cuh"

namespace cg = cooperative_groups;

int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }


// ----------------------------------------------------------------------------- decode

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
    // Every entry of a decode step brings one token, so entry e is row e; what the block needs of the step's
    // metadata is fetched in one round of independent loads (the block table is the second, the keys the third).
    const int num_entries = meta[META_NUM_ENTRIES], newest = positions[e];
    const int bt_offset = meta[META_BT_OFFSET + group], bt_stride = meta[META_BT_STRIDE + group];
    const bool live = e < num_entries;
    const int G = nq / L.num_kv_heads;
    const int row0 = e;
    const int kv_len = live ? newest + 1 : 0;
    const int kstart = window > 0 ? max(0, kv_len - window) : 0;
    const int per = (((kv_len - kstart + splits - 1) / splits + DEC_KT - 1) / DEC_KT) * DEC_KT;
    const int lo = kstart + split * per, hi = min(kv_len, lo + per);
    const int* bt = meta + bt_offset + (size_t)e * bt_stride;
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
// Decode attention for batches with many (request, head group) pairs: all key tiles dealt out evenly over as many
// blocks as the GPU holds (flat_attention in attention_tiles.cuh says how).
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
    flat_prefix<0>(prefix, meta, cu_tokens, positions, S, window, threadIdx.x);
    pdl_wait();  // q (and, without the fused rotation, the newest key and value) come from the kernels before
    flat_attention<0>(blockIdx.x, gridDim.x, threadIdx.x, qtile, tiles, prefix, &s_last, q, q_stride, cache, L, meta, group,
                      cu_tokens, positions, out, part_o, part_ml, counters, inv_freq, rot, store_kv, nq, window, scale_log2,
                      num_pages, S, status);
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
