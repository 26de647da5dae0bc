// Core kernels, for float32 and bfloat16 storage alike; all arithmetic is float32.
//
// These are the plain kernels of the engine: the whole float32 path runs on them,
// and the bfloat16 path uses them wherever no faster kernel exists for a size.
// Every reduction runs in an order that depends only on the element it belongs to
// (never on the batch, the portioning of a prompt, or the pages used), so float32
// logits are bit-identical however the work is cut.
//
// What they stand for in the reference: candle's embedding, RmsNorm, rope, silu and
// mul (models/src/llama.rs:470, 402-408, 218-251, 362-366), reshape_and_cache_flash
// (csrc/kernels/cache_manager.cu:139-170) and the paged attention kernels
// (csrc/kernels/flash_fwd_kernel.h).
#include "common.cuh"

int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

// ----------------------------------------------------------------------------- embedding
// resid[t, :] = scale * table[tokens[t], :], widened to float32 (the residual stream is float32).
// A negative token id -1 - s stands for "the token last sampled into slot s" (last_tokens[s]):
// a decode step can be launched before the host has read the previous step's tokens.
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                  float* __restrict__ resid, const int* __restrict__ meta, int H, int V, float scale,
                                  const int* __restrict__ last_tokens, int num_slots, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    int tok = tokens[t];
    // a slot beyond the array leaves the id negative, which is reported as a bad token below
    if (tok < 0 && last_tokens && -(long long)tok - 1 < num_slots) tok = last_tokens[-tok - 1];
    bool bad = tok < 0 || tok >= V;
    if (bad && threadIdx.x == 0) atomicExch(&status[STATUS_BAD_TOKEN], 1 + t);
    const T* row = table + (size_t)(bad ? 0 : tok) * H;
    float* out = resid + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = bad ? 0.f : scale * to_float(row[i]);
}

extern "C" int embed_rows(const int* tokens, const void* table, int table_dtype, float* resid, const int* meta,
                          int T, int H, int V, float scale, const int* last_tokens, int num_slots, int* status,
                          cudaStream_t stream) {
    if (T <= 0) return 0;
    int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == DT_F32)
        return (int)launch_kernel(embed_rows_kernel<float>, T, threads, 0, stream, tokens, (const float*)table, resid, meta, H, V, scale,
                                  last_tokens, num_slots, status);
    return (int)launch_kernel(embed_rows_kernel<__nv_bfloat16>, T, threads, 0, stream, tokens, (const __nv_bfloat16*)table, resid,
                              meta, H, V, scale, last_tokens, num_slots, status);
}

// ----------------------------------------------------------------------------- RMSNorm
// resid[t] += delta[t] (if delta), out[t] = resid[t] * rsqrt(mean(resid[t]^2) + eps) * w.
// With `rows`: works on rows[r] of resid/delta, writes out[r], leaves resid untouched.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const int* __restrict__ rows,
                   const float* __restrict__ w, float eps, TO* __restrict__ out, const int* __restrict__ meta, int H,
                   int aligned) {
    __shared__ float red[33];
    constexpr int MAXV = 4;  // up to 4 x 4 values per thread stay in registers (H <= 16 * blockDim)
    // four values per access: rows start on multiples of four elements and the buffers on 16 bytes
    const bool in_regs = aligned && (H % 4 == 0) && H <= 4 * MAXV * (int)blockDim.x;
    float4 wv[MAXV];
    if (in_regs) {  // the norm weight depends on no earlier kernel: fetched before the wait
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < H) wv[j] = *reinterpret_cast<const float4*>(w + i);
        }
    }
    pdl_wait();
    // The kernels after this one may start now, not earlier: they fetch their weights and then wait for this
    // kernel, and blocks that wait through the whole of the kernel before this one slow it down.
    pdl_launch_dependents();
    int r = blockIdx.x;
    int limit = rows ? meta[META_NUM_ROWS] : meta[META_NUM_TOKENS];
    if (r >= limit) return;
    size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* x = resid + src * H;
    const TD* dl = delta ? delta + src * H : nullptr;
    TO* o = out + (size_t)r * H;
    float ss = 0.f;
    if (in_regs) {
        float4 v[MAXV];
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < H) {
                v[j] = *reinterpret_cast<const float4*>(x + i);
                if (dl) {
                    float dv[4];
                    load4(dl + i, dv);
                    v[j].x += dv[0]; v[j].y += dv[1]; v[j].z += dv[2]; v[j].w += dv[3];
                    if (!rows) *reinterpret_cast<float4*>(x + i) = v[j];
                }
                ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
                ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
            }
        }
        ss = block_sum(ss, red);
        float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < H) {
                const float ov[4] = {v[j].x * inv * wv[j].x, v[j].y * inv * wv[j].y, v[j].z * inv * wv[j].z, v[j].w * inv * wv[j].w};
                store4(o + i, ov);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl) {
            v += to_float(dl[i]);
            if (!rows) x[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = x[i];
        if (dl && rows) v += to_float(dl[i]);
        o[i] = from_float<TO>(v * inv * w[i]);
    }
}

// The same for a thousand rows and more of bfloat16 activations (fewer would leave multiprocessors idle): one warp per row, the row's values in registers (NV float4
// per lane), no block barrier; every lane has all its loads in flight at once.  The sum of squares is taken
// in another order than above, which bfloat16 results do not show (float32 rows always take the kernel
// above, whose order never changes).
template <int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ delta, const float* __restrict__ w,
                        float eps, __nv_bfloat16* __restrict__ out, const int* __restrict__ meta) {
    constexpr int H = NV * 128;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= meta[META_NUM_TOKENS]) return;
    float* x = resid + (size_t)r * H;
    const __nv_bfloat16* dl = delta ? delta + (size_t)r * H : nullptr;
    float4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) v[j] = *reinterpret_cast<const float4*>(x + (j * 32 + lane) * 4);
    float ss = 0.f;
    if (dl) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float dv[4];
            load4(dl + (j * 32 + lane) * 4, dv);
            v[j].x += dv[0]; v[j].y += dv[1]; v[j].z += dv[2]; v[j].w += dv[3];
            *reinterpret_cast<float4*>(x + (j * 32 + lane) * 4) = v[j];
        }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = rsqrtf(ss / (float)H + eps);
    __nv_bfloat16* o = out + (size_t)r * H;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const float4 wv = *reinterpret_cast<const float4*>(w + (j * 32 + lane) * 4);
        const float ov[4] = {v[j].x * inv * wv.x, v[j].y * inv * wv.y, v[j].z * inv * wv.z, v[j].w * inv * wv.w};
        store4(o + (j * 32 + lane) * 4, ov);
    }
}

extern "C" int add_rmsnorm(float* resid, const void* delta, int delta_dtype, const int* rows, const float* w,
                           float eps, void* out, int out_dtype, const int* meta, int n, int H,
                           cudaStream_t stream) {
    if (n <= 0) return 0;
    int threads = H >= 1024 ? 256 : 128;
    const int aligned = (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
    if (n >= 1024 && !rows && aligned && out_dtype == DT_BF16 && (!delta || delta_dtype == DT_BF16) && H % 128 == 0 && H <= 4096) {
#define ROWS_CASE(NV) \
    if (H == NV * 128) \
        return (int)launch_kernel(add_rmsnorm_rows_kernel<NV>, (n + 7) / 8, 256, 0, stream, resid, (const __nv_bfloat16*)delta, w, \
                                  eps, (__nv_bfloat16*)out, meta)
        ROWS_CASE(8); ROWS_CASE(16); ROWS_CASE(24); ROWS_CASE(32);
#undef ROWS_CASE
    }
#define NORM_CASE(TD, TO) \
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, add_rmsnorm_kernel<TD, TO>, n, threads, 0, stream, resid, (const TD*)delta, \
                                  rows, w, eps, (TO*)out, meta, H, aligned)
    if (delta_dtype == DT_F32 && out_dtype == DT_F32) NORM_CASE(float, float);
    else if (delta_dtype == DT_BF16 && out_dtype == DT_BF16) NORM_CASE(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == DT_F32 && out_dtype == DT_BF16) NORM_CASE(float, __nv_bfloat16);
    else NORM_CASE(__nv_bfloat16, float);
#undef NORM_CASE
}

// ----------------------------------------------------------------------------- float32 GEMM
// y[M, N] = x[M, K] * w[N, K]^T, plain FFMA.  Each output element is one accumulator
// running over k = 0..K-1 in order, so its value does not depend on M or on the tile
// it falls in.  No tensor cores, no TF32.
#define GB 64
#define GK 16
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       float* __restrict__ y, int M, int N, int K) {
    __shared__ float xs[GK][GB + 4];
    __shared__ float ws[GK][GB + 4];
    pdl_launch_dependents();
    pdl_wait();
    int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
    int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int idx = threadIdx.x + i * 256;  // 0..1023 over a 64 x 16 tile
            int r = idx / GK, c = idx % GK;
            int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            xs[c][r] = (gm < M && gk < K) ? x[(size_t)gm * K + gk] : 0.f;
            ws[c][r] = (gn < N && gk < K) ? w[(size_t)gn * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn < N) y[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

extern "C" int gemm_f32(const float* x, const float* w, float* y, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GB - 1) / GB, (M + GB - 1) / GB);
    return (int)launch_kernel(gemm_f32_kernel, grid, 256, 0, stream, x, w, y, M, N, K);
}

// ----------------------------------------------------------------------------- rotation + cache write
// One row of the fused projection per token: [q (nq heads) | k (nkv heads) | v (nkv heads)].
// Rotates q in place and writes rotated k and plain v to the token's slot of its page.
// angle = position * inv_freq[i] in float32; pairs are (x[i], x[i + rot/2]) within the
// first `rot` dims of a head (models/src/llama.rs:189-198, :250).  With store_kv = 0
// (a layer that reads another layer's cache) only q is rotated.
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_entry, const int* __restrict__ meta, int group,
                                     const float* __restrict__ inv_freq, T* __restrict__ cache, CacheLayout L,
                                     int nq, int rot, int store_kv, int num_pages, int* __restrict__ status) {
    // one row of threads (threadIdx.y) per (token, head of the fused row): q heads, then k heads, then v heads
    pdl_launch_dependents();
    const int d = L.head_dim, nkv = L.num_kv_heads, half = rot / 2;
    const int t = blockIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y;
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    float freq = 0.f;
    if ((is_q || is_k) && (int)threadIdx.x < half) freq = inv_freq[threadIdx.x];  // a constant: before the wait
    pdl_wait();
    if (h >= nq + 2 * nkv || t >= meta[META_NUM_TOKENS]) return;
    if (!is_q && !store_kv) return;
    const int pos = positions[t];
    T* x = qkv + ((size_t)t * (nq + 2 * nkv) + h) * d;
    T* dst = x;  // q is rotated in place
    if (!is_q) {
        const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group];
        int page = bt[pos / L.page_size];
        if (page <= 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
            return;
        }
        dst = cache + L.offset(page, is_k ? 0 : 1, is_k ? h - nq : h - nq - nkv, pos % L.page_size);
    }
    if (is_q || is_k) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float f = i == (int)threadIdx.x ? freq : inv_freq[i];
            float sn, cs;
            sincosf((float)pos * f, &sn, &cs);
            float lo, hi;
            rotate_pair(to_float(x[i]), to_float(x[i + half]), cs, sn, lo, hi);
            dst[i] = from_float<T>(lo);
            dst[i + half] = from_float<T>(hi);
        }
        if (is_k)
            for (int i = rot + threadIdx.x; i < d; i += blockDim.x) dst[i] = x[i];  // dims beyond the rotated part
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = x[i];
    }
}

// The same for many tokens: one block per token.  The token's cosines and sines are computed once (not once
// per head) and every thread moves 16 bytes at a time: a pair of chunks (the same dims of a head's two
// halves) for the heads that rotate, single chunks for the values and for dims beyond the rotated part.
// Needs rot / 2 and the head size to be multiples of a chunk (8 bfloat16 or 4 float32 values).
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_store_rows_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_entry,
                          const int* __restrict__ meta, int group, const float* __restrict__ inv_freq,
                          T* __restrict__ cache, CacheLayout L, int nq, int rot, int store_kv, int num_pages,
                          int* __restrict__ status) {
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ float trig[];  // cos[half], sin[half]
    pdl_launch_dependents();
    pdl_wait();
    const int d = L.head_dim, nkv = L.num_kv_heads, half = rot / 2;
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &trig[half + i], &trig[i]);
    int page = 0;
    if (store_kv) {
        const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group];
        page = bt[pos / L.page_size];
        if (page <= 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
            page = 0;  // keys and values are dropped; the queries are still rotated
        }
    }
    __syncthreads();
    T* row = qkv + (size_t)t * (nq + 2 * nkv) * d;
    const int slot = pos % L.page_size;
    // items: for each rotating head (q, then k if stored) half/VEC pairs of chunks and (d - rot)/VEC single
    // chunks (k only: q stays where it is); for each value head d/VEC single chunks
    const int rot_heads = nq + (page > 0 ? nkv : 0);
    const int pairs = half / VEC, tail = (d - rot) / VEC, per_rot = pairs + tail;
    const int items = rot_heads * per_rot + (page > 0 ? nkv * (d / VEC) : 0);
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
        if (it < rot_heads * per_rot) {
            const int h = it / per_rot, j = it % per_rot;
            const bool is_q = h < nq;
            const T* x = row + (size_t)h * d;
            T* dst = is_q ? row + (size_t)h * d : cache + L.offset(page, 0, h - nq, slot);
            if (j < pairs) {
                float a[VEC], b[VEC], lo[VEC], hi[VEC];
#pragma unroll
                for (int c = 0; c < VEC; c += 4) {
                    float ta[4], tb[4];
                    load4(x + j * VEC + c, ta);
                    load4(x + half + j * VEC + c, tb);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { a[c + i] = ta[i]; b[c + i] = tb[i]; }
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) rotate_pair(a[i], b[i], trig[j * VEC + i], trig[half + j * VEC + i], lo[i], hi[i]);
#pragma unroll
                for (int c = 0; c < VEC; c += 4) {
                    const float tl[4] = {lo[c], lo[c + 1], lo[c + 2], lo[c + 3]}, th[4] = {hi[c], hi[c + 1], hi[c + 2], hi[c + 3]};
                    store4(dst + j * VEC + c, tl);
                    store4(dst + half + j * VEC + c, th);
                }
            } else if (!is_q) {  // dims beyond the rotated part travel unchanged
                const int off = rot + (j - pairs) * VEC;
                *reinterpret_cast<uint4*>(dst + off) = *reinterpret_cast<const uint4*>(x + off);
            }
        } else {
            const int iv = it - rot_heads * per_rot, h = iv / (d / VEC), j = iv % (d / VEC);
            const T* x = row + (size_t)(nq + nkv + h) * d + j * VEC;
            *reinterpret_cast<uint4*>(cache + L.offset(page, 1, h, slot) + j * VEC) = *reinterpret_cast<const uint4*>(x);
        }
    }
}

extern "C" int rope_kv_store(void* qkv, int dtype, const int* positions, const int* token_entry, const int* meta,
                             int group, const float* inv_freq, void* cache, int num_pages, int T, int nq, int nkv,
                             int d, int rot, int page_size, int store_kv, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    CacheLayout L{nkv, page_size, d};
    // hundreds of tokens: one block per token with 16-byte accesses, where the sizes and addresses allow it
    const int vec = dtype == DT_F32 ? 4 : 8;
    if (T >= 256 && rot % (2 * vec) == 0 && d % vec == 0 && rot <= 512 && (((uintptr_t)qkv | (uintptr_t)cache) & 15) == 0) {
        const size_t smem = (size_t)rot * sizeof(float);
        if (dtype == DT_F32)
            return (int)launch_kernel(rope_kv_store_rows_kernel<float>, T, 256, smem, stream, (float*)qkv, positions, token_entry,
                                      meta, group, inv_freq, (float*)cache, L, nq, rot, store_kv, num_pages, status);
        return (int)launch_kernel(rope_kv_store_rows_kernel<__nv_bfloat16>, T, 256, smem, stream, (__nv_bfloat16*)qkv, positions,
                                  token_entry, meta, group, inv_freq, (__nv_bfloat16*)cache, L, nq, rot, store_kv,
                                  num_pages, status);
    }
    // few tokens: one head per block (many small blocks, short latency); else eight heads per block
    int heads = nq + 2 * nkv, hpb = T >= 64 ? 8 : 1;
    dim3 threads(d >= 128 ? 64 : 32, hpb);
    dim3 grid(T, (heads + hpb - 1) / hpb);
    if (dtype == DT_F32)
        return (int)launch_kernel(rope_kv_store_kernel<float>, grid, threads, 0, stream, (float*)qkv, positions, token_entry,
                                  meta, group, inv_freq, (float*)cache, L, nq, rot, store_kv, num_pages, status);
    return (int)launch_kernel(rope_kv_store_kernel<__nv_bfloat16>, grid, threads, 0, stream, (__nv_bfloat16*)qkv, positions,
                              token_entry, meta, group, inv_freq, (__nv_bfloat16*)cache, L, nq, rot, store_kv, num_pages,
                              status);
}

// ----------------------------------------------------------------------------- attention over the cache
// One block per (token, query head).  The query at position p reads the keys at
// positions kstart..p of its request through the block table (kstart = 0, or
// p - window + 1 for a windowed layer), 64 at a time in position order, with a
// running maximum and sum (softmax in float32).  The order of every sum depends on
// p and the window only, so the result is the same whether the token came alone,
// in a portion of a prompt, or beside other requests.
#define ATTN_KT 64
#define ATTN_THREADS 128
template <typename T>
__global__ void __launch_bounds__(ATTN_THREADS)
attn_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache, CacheLayout L,
                    const int* __restrict__ meta, int group, const int* __restrict__ token_entry,
                    const int* __restrict__ positions, T* __restrict__ out, int nq, int window, float scale,
                    int num_pages, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x, h = blockIdx.y;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int d = L.head_dim, ps = L.page_size, tid = threadIdx.x;
    const int p = positions[t];
    const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group];
    const int kvh = h / (nq / L.num_kv_heads);
    extern __shared__ float sm[];
    float* qs = sm;                // d
    float* prob = qs + d;          // ATTN_KT
    float* red = prob + ATTN_KT;   // 40
    float* tile = red + 40;        // ATTN_KT * (d + 1)
    const int ld = d + 1;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
    for (int i = tid; i < d; i += ATTN_THREADS) qs[i] = to_float(qrow[i]);
    float m = -INFINITY, l = 0.f;
    float acc[2] = {0.f, 0.f};  // head sizes up to 2 * ATTN_THREADS
    const int kstart = window > 0 ? max(0, p - window + 1) : 0;
    for (int k0 = kstart; k0 <= p; k0 += ATTN_KT) {
        const int n = min(ATTN_KT, p - k0 + 1);
        __syncthreads();  // the previous tile's values are no longer read
        for (int idx = tid; idx < n * d; idx += ATTN_THREADS) {
            int j = idx / d, i = idx % d, pos = k0 + j;
            int page = bt[pos / ps];
            if (page <= 0 || page >= num_pages) {
                atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
                tile[j * ld + i] = 0.f;
            } else {
                tile[j * ld + i] = to_float(cache[L.offset(page, 0, kvh, pos % ps) + i]);
            }
        }
        __syncthreads();
        float s = -INFINITY;
        if (tid < n) {
            float dot = 0.f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], tile[tid * ld + i], dot);
            s = dot * scale;
        }
        float m_new = fmaxf(m, block_max(s, red));
        float pj = tid < n ? expf(s - m_new) : 0.f;
        if (tid < ATTN_KT) prob[tid] = pj;
        float tsum = block_sum(pj, red);  // its barriers also order the key reads before the value writes
        float corr = expf(m - m_new);
        l = l * corr + tsum;
        m = m_new;
        for (int idx = tid; idx < n * d; idx += ATTN_THREADS) {
            int j = idx / d, i = idx % d, pos = k0 + j;
            int page = bt[pos / ps];
            bool ok = page > 0 && page < num_pages;
            tile[j * ld + i] = ok ? to_float(cache[L.offset(page, 1, kvh, pos % ps) + i]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < 2; ++a) {
            int i = tid + a * ATTN_THREADS;
            if (i < d) {
                float o = acc[a] * corr;
                for (int j = 0; j < n; ++j) o = fmaf(prob[j], tile[j * ld + i], o);
                acc[a] = o;
            }
        }
    }
    T* orow = out + ((size_t)t * nq + h) * d;
    float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        int i = tid + a * ATTN_THREADS;
        if (i < d) orow[i] = from_float<T>(acc[a] * inv);
    }
}

extern "C" int attn_generic(const void* q, int q_stride, const void* cache, int dtype, const int* meta, int group,
                            const int* token_entry, const int* positions, void* out, int T, int nq, int nkv, int d,
                            int page_size, int num_pages, int window, float scale, int* status,
                            cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d > 2 * ATTN_THREADS) return (int)cudaErrorInvalidValue;
    CacheLayout L{nkv, page_size, d};
    size_t smem = (size_t)(d + ATTN_KT + 40 + ATTN_KT * (d + 1)) * sizeof(float);
    dim3 grid(T, nq);
    cudaError_t e;
    // the attribute only ever grows, and is not set again inside a stream capture once it is large enough
    static size_t configured_f32 = 0, configured_bf16 = 0;
    if (dtype == DT_F32) {
        if (smem > configured_f32) {
            e = cudaFuncSetAttribute(attn_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured_f32 = smem;
        }
        return (int)launch_kernel(attn_generic_kernel<float>, grid, ATTN_THREADS, smem, stream, (const float*)q, q_stride,
                                  (const float*)cache, L, meta, group, token_entry, positions, (float*)out, nq, window, scale,
                                  num_pages, status);
    } else {
        if (smem > configured_bf16) {
            e = cudaFuncSetAttribute(attn_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured_bf16 = smem;
        }
        return (int)launch_kernel(attn_generic_kernel<__nv_bfloat16>, grid, ATTN_THREADS, smem, stream,
                                  (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)cache, L, meta, group, token_entry,
                                  positions, (__nv_bfloat16*)out, nq, window, scale, num_pages, status);
    }
}

// ----------------------------------------------------------------------------- SwiGLU gate
// out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(z) = z / (1 + exp(-z))  (models/src/llama.rs:364).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, const int* __restrict__ meta, int I) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.y;
    if (meta && t >= meta[META_NUM_TOKENS]) return;  // without step metadata every launched row is a real one
    constexpr int V = 16 / sizeof(T);  // elements of a 16-byte access
    const T* g = gu + (size_t)t * 2 * I;
    T* o = out + (size_t)t * I;
    int i = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (I % V == 0) {  // rows stay 16-byte aligned
        if (i >= I) return;
        uint4 gv = *reinterpret_cast<const uint4*>(g + i), uv = *reinterpret_cast<const uint4*>(g + I + i), ov;
        const T* gp = reinterpret_cast<const T*>(&gv);
        const T* up = reinterpret_cast<const T*>(&uv);
        T* op = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            float x = to_float(gp[j]);
            op[j] = from_float<T>(x / (1.f + expf(-x)) * to_float(up[j]));
        }
        *reinterpret_cast<uint4*>(o + i) = ov;
    } else {
        for (int j = i; j < min(i + V, I); ++j) {
            float x = to_float(g[j]);
            o[j] = from_float<T>(x / (1.f + expf(-x)) * to_float(g[I + j]));
        }
    }
}

extern "C" int silu_mul(const void* gu, void* out, int dtype, const int* meta, int T, int I, cudaStream_t stream) {
    if (T <= 0) return 0;
    int per_block = 256 * (dtype == DT_F32 ? 4 : 8);
    dim3 grid((I + per_block - 1) / per_block, T);
    if (dtype == DT_F32) return (int)launch_kernel(silu_mul_kernel<float>, grid, 256, 0, stream, (const float*)gu, (float*)out, meta, I);
    return (int)launch_kernel(silu_mul_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                              meta, I);
}

// ----------------------------------------------------------------------------- weights ahead of time
// A kernel of its own that only asks byte ranges into L2 (see PrefetchRanges).  It reads and writes nothing of
// the step, yet it waits for the kernel before it like every other one: a dependent launch waits only for the
// grid directly ahead of it, so a link of the chain that ended early would let the kernel behind it (the
// attention) run ahead of the projection whose rows it reads.
__global__ void l2_prefetch_kernel(const PrefetchRanges r) {
    pdl_launch_dependents();
    prefetch_ranges_l2(r, (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x, (unsigned long long)gridDim.x * blockDim.x);
    pdl_wait();
}
extern "C" int l2_prefetch(int n, const void* const* ptrs, const unsigned long long* bytes, cudaStream_t stream) {
    const PrefetchRanges r = make_prefetch_ranges(n, ptrs, bytes);
    if (!(r.bytes[0] | r.bytes[1] | r.bytes[2] | r.bytes[3])) return 0;
    return (int)launch_kernel(l2_prefetch_kernel, 64, 128, 0, stream, r);
}
// The same on a stream of its own, beside the step's chain of dependent launches: an ordinary launch.
extern "C" int l2_prefetch_aside(int n, const void* const* ptrs, const unsigned long long* bytes, cudaStream_t stream) {
    const PrefetchRanges r = make_prefetch_ranges(n, ptrs, bytes);
    if (!(r.bytes[0] | r.bytes[1] | r.bytes[2] | r.bytes[3])) return 0;
    return (int)launch_kernel_pdl(false, l2_prefetch_kernel, 64, 128, 0, stream, r);
}

// ----------------------------------------------------------------------------- casts
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(to_float(in[i]));
}
extern "C" int cast_f32_bf16(const float* in, void* out, size_t n, cudaStream_t stream) {
    if (!n) return 0;
    cast_kernel<float, __nv_bfloat16><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(in, (__nv_bfloat16*)out, n);
    LAUNCH_RETURN();
}
extern "C" int cast_bf16_f32(const void* in, float* out, size_t n, cudaStream_t stream) {
    if (!n) return 0;
    cast_kernel<__nv_bfloat16, float><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)in, out, n);
    LAUNCH_RETURN();
}
