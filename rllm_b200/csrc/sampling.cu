// On-device token sampling: one block per logits row, the row never leaves the GPU.
//   temperature <= 0 : argmax, lowest index on ties, NaNs never win (no candidate: id 0);
//   otherwise        : x = logit / T; candidates x >= threshold, where the threshold is found by
//                      40 bisection steps on the value (top_k: largest t with count(x >= t) >= k;
//                      top_p: largest t whose candidates hold >= top_p of the mass of the top_k
//                      set); the token is argmax(x + g), g = -ln(-ln(u)) Gumbel noise with
//                      u = hash(seed, counter, token) in (0,1): an exact draw from softmax(x)
//                      that is reproducible whatever else is in the batch.
// Semantics and hash constants: crates/rllm-core/src/sample.rs:19-109 of AxiomOperator/rllm;
// its device counterpart is sample_rows (crates/rllm-cuda/kernels/kernels.cu:885-954).
#include "common.cuh"
#include <math.h>

#define SAMPLE_THREADS 1024
#define BISECT_STEPS 40

__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long counter,
                                              unsigned int token) {
    unsigned long long z = seed ^ (counter * 0x9E3779B97F4A7C15ull) ^
                           ((unsigned long long)token * 0xD1B54A32D192ED03ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

struct KeyIdx { float key; int idx; };
__device__ __forceinline__ KeyIdx better(KeyIdx a, KeyIdx b) {
    // larger key wins; equal keys: lower index; idx < 0 means "no candidate"
    if (b.idx < 0) return a;
    if (a.idx < 0) return b;
    if (b.key > a.key || (b.key == a.key && b.idx < a.idx)) return b;
    return a;
}
__device__ KeyIdx block_best(KeyIdx v, KeyIdx* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        KeyIdx other;
        other.key = __shfl_xor_sync(0xffffffffu, v.key, o);
        other.idx = __shfl_xor_sync(0xffffffffu, v.idx, o);
        v = better(v, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        KeyIdx t = sh[0];
        for (int i = 1; i < nw; ++i) t = better(t, sh[i]);
        sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* logits, long long row_stride, int vocab,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                   const unsigned long long* __restrict__ counter, int* __restrict__ out) {
    __shared__ float red[33];
    __shared__ KeyIdx best_sh[33];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)r * row_stride;
    const float T = temperature ? temperature[r] : 0.f;

    if (!(T > 0.f)) {
        KeyIdx b; b.key = -INFINITY; b.idx = -1;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const float v = x[i];
            if (v > b.key) { b.key = v; b.idx = i; }     // NaN compares false
        }
        b = block_best(b, best_sh);
        if (tid == 0) out[r] = b.idx < 0 ? 0 : b.idx;
        return;
    }
    const float inv_t = 1.0f / T;
    float lo = INFINITY, hi = -INFINITY;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i] * inv_t;
        lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    hi = block_max(hi, red);
    lo = -block_max(-lo, red);
    const float vmax = hi;
    float thr = -INFINITY;
    const int k = top_k ? top_k[r] : 0;
    const float p = top_p ? top_p[r] : 1.0f;
    if (k > 0 && k < vocab) {
        float a = lo, b = hi;
        for (int s = 0; s < BISECT_STEPS; ++s) {
            const float mid = 0.5f * (a + b);
            float c = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) c += (x[i] * inv_t >= mid) ? 1.f : 0.f;
            c = block_sum(c, red);                       // counts < 2^24 are exact in float
            if (c >= (float)k) a = mid; else b = mid;
        }
        thr = a; lo = a;
    }
    if (p < 1.0f) {
        float total = 0.f;
        for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
            const float v = x[i] * inv_t;
            if (v >= thr) total += expf(v - vmax);
        }
        total = block_sum(total, red);
        float a = lo, b = hi;
        for (int s = 0; s < BISECT_STEPS; ++s) {
            const float mid = 0.5f * (a + b);
            float ms = 0.f;
            for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
                const float v = x[i] * inv_t;
                if (v >= mid) ms += expf(v - vmax);
            }
            ms = block_sum(ms, red);
            if (ms >= p * total) a = mid; else b = mid;
        }
        thr = a;
    }
    const unsigned long long sd = seed ? seed[r] : 0ull, ct = counter ? counter[r] : 0ull;
    KeyIdx b; b.key = -INFINITY; b.idx = -1;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i] * inv_t;
        if (v >= thr) {
            const float u = hash_uniform(sd, ct, (unsigned)i);
            const float key = v + (-logf(-logf(u)));
            if (key > b.key) { b.key = key; b.idx = i; }
        }
    }
    b = block_best(b, best_sh);
    if (tid == 0) out[r] = b.idx < 0 ? 0 : b.idx;
}

// logits[index[i]] += delta[i] (logit bias, frequency and presence penalties): index is the flat
// position row * row_stride + token; the caller has summed the deltas of equal positions, so no
// two threads touch one value (crates/rllm-cuda/kernels/kernels.cu:875-880).
__global__ void logit_adjust_kernel(float* __restrict__ logits, const long long* __restrict__ index,
                                    const float* __restrict__ delta, int n) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) logits[index[i]] += delta[i];
}

RLLM_API int rllm_logit_adjust(float* logits, const long long* index, const float* delta, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return rllm_launch(logit_adjust_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, logits, index, delta, n);
}

RLLM_API int rllm_sample_rows(const float* logits, long long row_stride, int rows, int vocab,
                              const float* temperature, const int* top_k, const float* top_p,
                              const unsigned long long* seed, const unsigned long long* counter,
                              int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || vocab >= (1 << 24)) return (int)cudaErrorInvalidValue;
    return rllm_launch(sample_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, vocab,
                       temperature, top_k, top_p, seed, counter, out);
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_logit_adjust)
RLLM_PACKED(rllm_sample_rows)
