// Paged causal attention, plain form: one block per (token, query head), float32
// arithmetic, any head size that is a multiple of 2 up to 512, any page size, any
// number of heads and groups, optional sliding window.  It is the float32 path of
// the engine and the reference the tensor-core kernels are tested against.
//
// Token t of request r = seq_ids[t] at absolute position pos sees keys p with
// max(0, pos+1-window) <= p <= pos (window 0: all keys); the keys of the step's own
// tokens are already in the cache.  Key p lives in page block_table[r][p / bs] at
// offset p % bs; cache layout [page][kv_head][bs][hd].
//
// Formula: crates/rllm-cpu/src/lib.rs:389-425 of AxiomOperator/rllm; its device
// counterpart is paged_attention (crates/rllm-cuda/kernels/kernels.cu:1634-1690).
// Keys are consumed in chunks of 128 in ascending order with an online softmax, so
// the result for a token depends only on its own keys, never on the batch around it.
#include "common.cuh"
#include <math.h>

#define ATT_THREADS 128
#define ATT_MAX_ACC 4   // hd <= ATT_THREADS * ATT_MAX_ACC

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_generic_kernel(const TQ* q, const TC* k_cache,
                               const TC* v_cache, TO* out,
                               const int* __restrict__ positions, const int* __restrict__ seq_ids,
                               const int* __restrict__ block_table, int table_stride, int H, int K,
                               int hd, int bs, float scale, int window, int n_pages, int* err) {
    extern __shared__ float smem[];
    pdl_wait();
    pdl_launch_dependents();
    float* qs = smem;                    // [hd]
    float* pr = smem + hd;               // [ATT_THREADS] probabilities of the chunk
    int* rowoff = (int*)(pr + ATT_THREADS);  // [ATT_THREADS] element offset / hd of each key row
    __shared__ float red[33];

    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (H / K);
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_ids[t] * table_stride;
    const int first = (window > 0 && pos + 1 - window > 0) ? pos + 1 - window : 0;
    const int tid = threadIdx.x;

    const TQ* qrow = q + ((size_t)t * H + h) * hd;
    for (int i = tid; i < hd; i += ATT_THREADS) qs[i] = to_f<TQ>(qrow[i]);
    __syncthreads();

    float acc[ATT_MAX_ACC];
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) acc[a] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int c0 = first; c0 <= pos; c0 += ATT_THREADS) {
        const int p = c0 + tid;
        float s = -INFINITY;
        if (p <= pos) {
            int page = table[p / bs];
            if (page < 0 || page >= n_pages) {        // refused: read page 0, report
                if (err) atomicExch(err, RLLM_ERR_PAGE);
                page = 0;
            }
            const size_t row = ((size_t)page * K + kvh) * bs + (p % bs);
            rowoff[tid] = (int)row;
            const TC* kr = k_cache + row * hd;
            float dot = 0.f;
            for (int i = 0; i < hd; ++i) dot += qs[i] * to_f<TC>(kr[i]);
            s = dot * scale;
        }
        const float cmax = block_max(s, red);
        const float m_new = fmaxf(m_run, cmax);
        const float e = (p <= pos) ? expf(s - m_new) : 0.f;
        pr[tid] = e;
        const float csum = block_sum(e, red);          // also orders pr/rowoff writes before reads
        const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * alpha + csum;
        m_run = m_new;
        const int cn = min(ATT_THREADS, pos + 1 - c0);
#pragma unroll
        for (int a = 0; a < ATT_MAX_ACC; ++a) {
            const int d = tid + a * ATT_THREADS;
            if (d < hd) {
                float v = acc[a] * alpha;
                for (int j = 0; j < cn; ++j) v += pr[j] * to_f<TC>(v_cache[(size_t)rowoff[j] * hd + d]);
                acc[a] = v;
            }
        }
        __syncthreads();
    }
    TO* orow = out + ((size_t)t * H + h) * hd;
    const float inv = 1.0f / l_run;
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) {
        const int d = tid + a * ATT_THREADS;
        if (d < hd) orow[d] = from_f<TO>(acc[a] * inv);
    }
}

RLLM_API int rllm_paged_attention_generic(const void* q, int q_dtype, const void* k_cache,
                                          const void* v_cache, int cache_dtype, void* out,
                                          int out_dtype, const int* positions, const int* seq_ids,
                                          const int* block_table, int table_stride, int n, int H,
                                          int K, int hd, int bs, float scale, int window, int n_pages, int* err,
                                          cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hd > ATT_THREADS * ATT_MAX_ACC || K <= 0 || H % K != 0 || bs <= 0) return (int)cudaErrorInvalidValue;
    if (q_dtype != cache_dtype || q_dtype != out_dtype) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)(hd + 2 * ATT_THREADS) * sizeof(float);
    dim3 grid(n, H);
    if (q_dtype == RLLM_F32)
        return rllm_launch(paged_attention_generic_kernel<float, float, float>, grid, dim3(ATT_THREADS), smem,
                           stream, (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out,
                           positions, seq_ids, block_table, table_stride, H, K, hd, bs, scale, window, n_pages, err);
    return rllm_launch(paged_attention_generic_kernel<bf16, bf16, bf16>, grid, dim3(ATT_THREADS), smem, stream,
                       (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions,
                       seq_ids, block_table, table_stride, H, K, hd, bs, scale, window, n_pages, err);
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_paged_attention_generic)
