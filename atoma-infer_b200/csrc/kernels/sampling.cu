// Sampling on the device: argmax, temperature, top-k, top-p, repetition penalty.
//
// The reference samples on the host, one row at a time, after copying the whole row
// of logits off the device (backends/vllm/src/model_executor.rs:193-262): ArgMax when
// sampling is off or the temperature is 1, else All / TopK / TopP / TopKThenTopP
// (backends/vllm/src/llm_service.rs:346-369), each request with a generator of its
// own seeded at admission (:371-372).  Here one block samples one row, and only the
// token id leaves the device.  The random number of a request's n-th token is
// Philox-4x32-10 of (seed, n): it does not depend on who shares the batch.
//
// Per row: s = logits / T; p = exp(s - max s).  top-k keeps p >= the k-th largest p;
// top-p then keeps the most likely tokens whose mass reaches top_p of what top-k
// kept (ties at either edge are kept).  The token is the first, in index order, at
// which the running sum of kept p exceeds u * (their total).  Greedy (T == 0) is the
// largest logit, the lowest index among equals.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    uint32_t n0 = hi1 ^ c[1] ^ k[0], n2 = hi0 ^ c[3] ^ k[1];
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u;
}

__device__ float philox_uniform(uint64_t seed, uint64_t step) {
    uint32_t c[4] = {(uint32_t)step, (uint32_t)(step >> 32), 0u, 0u};
    uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
#pragma unroll
    for (int r = 0; r < 10; ++r) philox_round(c, k);
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// p_i of the row, or 0 when dropped by the thresholds
__device__ __forceinline__ float prob_of(float logit, float T, float m) { return expf(logit / T - m); }

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p,
                   const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ step,
                   int* __restrict__ out, const int* __restrict__ num_rows, const int* __restrict__ slots,
                   int* __restrict__ last_tokens) {
    __shared__ float red[33];
    __shared__ float fsum[SAMPLE_THREADS];
    __shared__ ArgMax amax[32];
    __shared__ int found, last_kept;
    __shared__ float target_s;
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (num_rows && r >= *num_rows) return;
    const float* row = logits + (size_t)r * V;
    const float T = temperature ? temperature[r] : 0.f;

    // argmax of the logits, lowest index among equals
    ArgMax best{-INFINITY, 0x7fffffff};
    if (V % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {  // four logits a load
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i = tid; i < V / 4; i += SAMPLE_THREADS) {
            const float4 v = row4[i];
            best = better(best, ArgMax{v.x, 4 * i});
            best = better(best, ArgMax{v.y, 4 * i + 1});
            best = better(best, ArgMax{v.z, 4 * i + 2});
            best = better(best, ArgMax{v.w, 4 * i + 3});
        }
    } else {
        for (int i = tid; i < V; i += SAMPLE_THREADS) best = better(best, ArgMax{row[i], i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) amax[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = amax[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0) amax[0] = best;
    }
    __syncthreads();
    best = amax[0];
    if (!(T > 0.f)) {
        if (tid == 0) {
            int tok = best.i == 0x7fffffff ? 0 : best.i;
            out[r] = tok;
            if (slots) last_tokens[slots[r]] = tok;  // where the next step's embedding can find it
        }
        return;
    }
    const float m = best.v / T;

    // thresholds on p, as bit patterns (p >= 0, so the unsigned order is the float order)
    uint32_t kth = 0u;
    const int k = top_k ? top_k[r] : 0;
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {  // largest v with count(p >= v) >= k
            uint32_t cand = kth | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) cnt += __float_as_uint(prob_of(row[i], T, m)) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)k) kth = cand;
        }
    }
    uint32_t cut = kth;
    const float tp = top_p ? top_p[r] : 1.f;
    if (tp < 1.f) {
        float mass = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            float p = prob_of(row[i], T, m);
            mass += __float_as_uint(p) >= kth ? p : 0.f;
        }
        mass = block_sum(mass, red);
        const float want = tp * mass;
        uint32_t v = 0u;
        for (int bit = 31; bit >= 0; --bit) {  // largest v with mass(p >= v) >= top_p * mass
            uint32_t cand = v | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                float p = prob_of(row[i], T, m);
                uint32_t b = __float_as_uint(p);
                s += (b >= cand && b >= kth) ? p : 0.f;
            }
            s = block_sum(s, red);
            if (s >= want) v = cand;
        }
        cut = max(cut, v);
    }

    // ordered scan: thread t owns the indices [t*chunk, (t+1)*chunk)
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = tid * chunk, hi = min(V, lo + chunk);
    float mine = 0.f;
    int my_last = -1;
    for (int i = lo; i < hi; ++i) {
        float p = prob_of(row[i], T, m);
        if (__float_as_uint(p) >= cut) { mine += p; my_last = i; }
    }
    fsum[tid] = mine;
    if (tid == 0) { found = V; last_kept = -1; }
    __syncthreads();
    atomicMax(&last_kept, my_last);
    if (tid == 0) {
        float run = 0.f;
        for (int t = 0; t < SAMPLE_THREADS; ++t) { float s = fsum[t]; fsum[t] = run; run += s; }  // exclusive prefix
        target_s = philox_uniform(seed[r], step[r]) * run;
    }
    __syncthreads();
    const float target = target_s;
    float run = fsum[tid];
    if (run <= target && run + mine > target) {
        for (int i = lo; i < hi; ++i) {
            float p = prob_of(row[i], T, m);
            if (__float_as_uint(p) >= cut) {
                run += p;
                if (run > target) { atomicMin(&found, i); break; }
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int tok = found < V ? found : max(last_kept, 0);
        out[r] = tok;
        if (slots) last_tokens[slots[r]] = tok;
    }
}

extern "C" int sample_rows(const float* logits, int R, int V, const float* temperature, const int* top_k,
                           const float* top_p, const unsigned long long* seed, const unsigned long long* step,
                           int* out, const int* num_rows, const int* slots, int* last_tokens, cudaStream_t stream) {
    if (R <= 0) return 0;
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, sample_rows_kernel, R, SAMPLE_THREADS, 0, stream, logits, V, temperature, top_k, top_p, seed,
                              step, out, num_rows, slots, last_tokens);
}

// Repetition penalty on one row: every distinct token id of `context` once; a
// non-negative logit is divided by the penalty, a negative one multiplied
// (backends/vllm/src/model_executor.rs:211-225).
__global__ void repeat_penalty_kernel(float* __restrict__ row, int V, float penalty, const int* __restrict__ context, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int tok = context[i];
    if (tok < 0 || tok >= V) return;
    for (int j = 0; j < i; ++j)
        if (context[j] == tok) return;  // an earlier thread owns this token
    float l = row[tok];
    row[tok] = l >= 0.f ? l / penalty : l * penalty;
}

extern "C" int repeat_penalty(float* row, int V, float penalty, const int* context, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    repeat_penalty_kernel<<<(n + 127) / 128, 128, 0, stream>>>(row, V, penalty, context, n);
    LAUNCH_RETURN();
}
