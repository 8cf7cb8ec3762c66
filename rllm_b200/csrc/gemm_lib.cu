// Library matrix product C[m,n] (+)= A[m,k] . W[n,k]^T through cuBLAS, bfloat16 operands with
// float32 accumulation, C float32 or bfloat16.  It stands where AxiomOperator/rllm's engine calls
// cuBLAS too: every dense product of more than 8 rows (crates/rllm-cuda/src/gpu.rs:238-268,
// Blas::gemm_tn; dispatch in crates/rllm-cuda/src/backend.rs:1198-1249).  accumulate != 0
// adds into a float32 C (beta = 1): the residual stream takes output projections that way.
//
// One handle and one 32 MiB workspace per device, made at the first call on that device
// (before any stream capture); the workspace is set explicitly so that a captured call
// allocates nothing.
#include "common.cuh"
#include <cublas_v2.h>

#define MAX_DEVICES 16
static cublasHandle_t g_handle[MAX_DEVICES];
static void* g_workspace[MAX_DEVICES];
static const size_t kWorkspaceBytes = 32u << 20;

static int get_handle(cublasHandle_t* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (!g_handle[dev]) {
        if (cublasCreate(&g_handle[dev]) != CUBLAS_STATUS_SUCCESS) return 10001;
        e = cudaMalloc(&g_workspace[dev], kWorkspaceBytes);
        if (e != cudaSuccess) return (int)e;
        if (cublasSetWorkspace(g_handle[dev], g_workspace[dev], kWorkspaceBytes) != CUBLAS_STATUS_SUCCESS)
            return 10002;
    }
    *out = g_handle[dev];
    return 0;
}

// Returns 0, a cudaError_t, or 10000 + cublasStatus_t.
RLLM_API int rllm_gemm_lib(const void* A, const void* W, void* C, int c_dtype, int m, int n, int k,
                           int lda, int ldw, int ldc, int accumulate, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (k <= 0) return (int)cudaErrorInvalidValue;
    if (accumulate && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    cublasHandle_t h;
    int st = get_handle(&h);
    if (st) return st;
    if (cublasSetStream(h, stream) != CUBLAS_STATUS_SUCCESS) return 10003;
    const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
    // row-major C[m,n] = A . W^T  ==  column-major C^T[n,m] = W^T(op T) . A(op N)
    cublasStatus_t s = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, n, m, k, &alpha, W, CUDA_R_16BF, ldw, A,
                                    CUDA_R_16BF, lda, &beta, C, c_dtype == RLLM_F32 ? CUDA_R_32F : CUDA_R_16BF,
                                    ldc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    return s == CUBLAS_STATUS_SUCCESS ? 0 : 10000 + (int)s;
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_gemm_lib)
