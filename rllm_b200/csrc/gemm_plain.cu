// Plain matrix product C[m,n] (+)= A[m,k] . W[n,k]^T on the CUDA cores with float32
// multiply-add: the true 32-bit path of the engine (no tensor cores, no reduced
// precision mode) and the reference the fast bf16 products are tested against.
//
// Every output element is accumulated by one thread over k in ascending order, so
// its value does not depend on m, on the other rows of the batch or on the grid.
// Any m, n, k >= 1.  A and W may be float32 or bfloat16 (converted on load);
// C is float32 or bfloat16.  accumulate != 0 adds the product to C (C must be
// float32 then): the residual stream takes the output projections that way.
//
// AxiomOperator/rllm computes this with 8 running sums on the CPU
// (crates/rllm-cpu/src/lib.rs:202-239) and through cuBLAS on the GPU
// (crates/rllm-cuda/src/gpu.rs:238-268).
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* A, const TW* __restrict__ W, TC* C, int m,
                  int n, int k, int lda, int ldw, int ldc, int accumulate) {
    __shared__ float As[TK][TM + 1];
    __shared__ float Ws[TK][TN + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;        // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < k; k0 += TK) {
        // 64 rows x 16 k-values per operand; 256 threads load 4 elements each
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int idx = tid + l * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < m && gk < k) ? to_f<TA>(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < n && gk < k) ? to_f<TW>(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            TC* c = C + (size_t)gm * ldc + gn;
            float v = acc[i][j];
            if (accumulate) v += to_f<TC>(*c);
            *c = from_f<TC>(v);
        }
    }
}

RLLM_API int rllm_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C,
                             int c_dtype, int m, int n, int k, int lda, int ldw, int ldc,
                             int accumulate, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return (int)cudaErrorInvalidValue;
    if (accumulate && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    dim3 grid((n + TN - 1) / TN, (m + TM - 1) / TM);
#define LAUNCH(TA, TW, TC)                                                                        \
    return rllm_launch(gemm_plain_kernel<TA, TW, TC>, grid, dim3(256), 0, stream, (const TA*)A,    \
                       (const TW*)W, (TC*)C, m, n, k, lda, ldw, ldc, accumulate)
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (key) {
        case 0: LAUNCH(float, float, float); break;
        case 1: LAUNCH(float, float, bf16); break;
        case 2: LAUNCH(float, bf16, float); break;
        case 3: LAUNCH(float, bf16, bf16); break;
        case 4: LAUNCH(bf16, float, float); break;
        case 5: LAUNCH(bf16, float, bf16); break;
        case 6: LAUNCH(bf16, bf16, float); break;
        case 7: LAUNCH(bf16, bf16, bf16); break;
        default: return (int)cudaErrorInvalidValue;
    }
#undef LAUNCH
    return 0;
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_gemm_plain)
