// Weight-streaming linear layer for few rows: y[M, N] = x[M, K] * w[N, K]^T, bfloat16 in,
// float32 accumulate, bfloat16 or float32 out.
//
// A decode step multiplies a handful of rows by every weight matrix: the time is the
// time to read the weights once.  Each warp owns COLS rows of w (output columns) and
// streams them with 16-byte loads, 32 lanes side by side; the few rows of x come from
// L1/L2.  A 128-row tensor-core tile would be nearly all padding here.  The reference
// calls cuBLAS for these (models/src/llama.rs:269-271, 311, 364-365, 476).
//
// Optional epilogues: silu(gate) * up for a fused [gate; up] weight (out has N/2
// columns), and float32 output for the logits.
#include "common.cuh"

#define SK_ROWS 8   // rows of x per pass
#define SK_COLS 2   // output columns per warp
#define SK_WARPS 8

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

template <typename TO, int EPI>  // EPI 0: plain, 1: silu(gate)*up with gate rows [0, N/2), up rows [N/2, N)
__global__ void __launch_bounds__(SK_WARPS * 32)
linear_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, TO* __restrict__ y,
                     const int* __restrict__ meta, int use_rows, int M, int N, int K) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m0 = blockIdx.y * SK_ROWS;
    int m_live = use_rows ? meta[META_NUM_ROWS] : (meta ? meta[META_NUM_TOKENS] : M);
    m_live = min(m_live, M);
    if (m0 >= m_live) return;
    const int rows = min(SK_ROWS, m_live - m0);
    const int n_out = EPI == 1 ? N / 2 : N;
    const int c0 = (blockIdx.x * SK_WARPS + warp) * SK_COLS;  // first output column of this warp
    if (c0 >= n_out) return;
    // weight rows this warp reads: for EPI 1 column c needs gate row c and up row n_out + c
    constexpr int WR = EPI == 1 ? 2 * SK_COLS : SK_COLS;
    const __nv_bfloat16* wrow[WR];
#pragma unroll
    for (int c = 0; c < SK_COLS; ++c) {
        int col = min(c0 + c, n_out - 1);
        wrow[c] = w + (size_t)col * K;
        if (EPI == 1) wrow[SK_COLS + c] = w + (size_t)(n_out + col) * K;
    }
    float acc[WR][SK_ROWS];
#pragma unroll
    for (int c = 0; c < WR; ++c)
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) acc[c][r] = 0.f;

    const int kvec = (K / 8) * 8;
    for (int k = lane * 8; k < kvec; k += 32 * 8) {
        bf16x8 wv[WR];
#pragma unroll
        for (int c = 0; c < WR; ++c) wv[c] = *reinterpret_cast<const bf16x8*>(wrow[c] + k);
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
            if (r < rows) {
                bf16x8 xv = *reinterpret_cast<const bf16x8*>(x + (size_t)(m0 + r) * K + k);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 xf = __bfloat1622float2(xv.v[i]);
#pragma unroll
                    for (int c = 0; c < WR; ++c) {
                        float2 wf = __bfloat1622float2(wv[c].v[i]);
                        acc[c][r] = fmaf(xf.x, wf.x, acc[c][r]);
                        acc[c][r] = fmaf(xf.y, wf.y, acc[c][r]);
                    }
                }
            }
        }
    }
    for (int k = kvec + lane; k < K; k += 32) {  // K not a multiple of 8
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r)
            if (r < rows) {
                float xf = __bfloat162float(x[(size_t)(m0 + r) * K + k]);
#pragma unroll
                for (int c = 0; c < WR; ++c) acc[c][r] = fmaf(xf, __bfloat162float(wrow[c][k]), acc[c][r]);
            }
    }
#pragma unroll
    for (int c = 0; c < WR; ++c)
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) acc[c][r] = warp_sum(acc[c][r]);
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < SK_COLS; ++c) {
            int col = c0 + c;
            if (col >= n_out) break;
#pragma unroll
            for (int r = 0; r < SK_ROWS; ++r) {
                if (r >= rows) break;
                float v = acc[c][r];
                if (EPI == 1) {
                    // the gate and up products are rounded to bfloat16 first, as separate
                    // GEMMs with bfloat16 outputs would leave them
                    float g = __bfloat162float(__float2bfloat16_rn(v));
                    float u = __bfloat162float(__float2bfloat16_rn(acc[SK_COLS + c][r]));
                    v = g / (1.f + expf(-g)) * u;
                }
                y[(size_t)(m0 + r) * n_out + col] = from_float<TO>(v);
            }
        }
    }
}

// x, w: bfloat16; K-rows of x and w must start 16-byte aligned when K % 8 == 0 is used
// for vector loads (K % 8 != 0 falls to scalar loads for the tail only if rows stay aligned).
extern "C" int linear_skinny(const void* x, const void* w, void* y, int out_dtype, int epilogue, const int* meta,
                             int use_rows, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 != 0) return (int)cudaErrorInvalidValue;  // rows would lose 16-byte alignment
    if (epilogue == 1 && (N % 2)) return (int)cudaErrorInvalidValue;
    int n_out = epilogue == 1 ? N / 2 : N;
    dim3 grid((n_out + SK_WARPS * SK_COLS - 1) / (SK_WARPS * SK_COLS), (M + SK_ROWS - 1) / SK_ROWS);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
    const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
    if (epilogue == 1) {
        if (out_dtype != DT_BF16) return (int)cudaErrorInvalidValue;
        linear_skinny_kernel<__nv_bfloat16, 1><<<grid, SK_WARPS * 32, 0, stream>>>(xb, wb, (__nv_bfloat16*)y, meta, use_rows, M, N, K);
    } else if (out_dtype == DT_F32) {
        linear_skinny_kernel<float, 0><<<grid, SK_WARPS * 32, 0, stream>>>(xb, wb, (float*)y, meta, use_rows, M, N, K);
    } else {
        linear_skinny_kernel<__nv_bfloat16, 0><<<grid, SK_WARPS * 32, 0, stream>>>(xb, wb, (__nv_bfloat16*)y, meta, use_rows, M, N, K);
    }
    LAUNCH_RETURN();
}
