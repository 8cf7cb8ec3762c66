// Weight-streaming product for decode: C[m,n] = X[m,k] . W[n,k]^T with few rows (m <= 64),
// bfloat16 operands, float32 accumulation on the tensor cores (mma.sync m16n8k16).
// The step is bound by reading W once from HBM, so the kernel is organised around the weight
// stream: a CTA owns 16 weight rows (32 for the fused SwiGLU form: 16 gate rows and the 16 up
// rows with the same index), its 8 warps interleave over k in steps of 32 elements, every thread
// fetches 16 contiguous bytes of two weight rows straight from global memory into the
// registers the MMA wants, and the batch rows X come through L1.  Partial sums of the 8 warps
// are added in warp order, so a column's value never depends on the other columns (requests)
// of the batch.
//
// Trick: for D = A.B the k index may be permuted as long as A and B use the same permutation.
// Lane (g = lane/4, t = lane%4) holds elements [8t, 8t+8) of a 32-wide k step of row g for both
// operands; elements 0-3 feed one MMA (as its k slots 2t,2t+1,2t+8,2t+9), elements 4-7 the next.
//
// Epilogues: store (float32 / bfloat16), accumulate into a float32 C (residual stream), or
// SwiGLU: C[b, j] = silu(gate_j) * up_j.
//
// Counterparts in AxiomOperator/rllm: matvec_f (crates/rllm-cuda/kernels/kernels.cu:608-651) and
// matvec_glu_f (1288-1356), CUDA-core kernels for m <= 8; above that it calls cuBLAS.
#include "common.cuh"

#define SG_WARPS 8
#define SG_THREADS (SG_WARPS * 32)

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// The batch rows are written by the kernel before this one, which may still run when this kernel
// starts (programmatic dependent launch).  They are therefore read with an ordinary, volatile load
// that stays behind griddepcontrol.wait: a read-only load (__ldg, or a const __restrict__ pointer,
// which the compiler turns into ld.global.nc) is "invariant" to the compiler, which may move it
// above the wait, where it sees the values of the step before.
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

enum { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

// An RMSNorm whose kernel this product saves (the contract of gemv_stream.cu's SvNorm).  Producer
// side, accumulate epilogue: beside the sums x it leaves in C, the launch writes bfloat16(x * w_next)
// and, per CTA, the sums of squares of its 16 columns of x: ssq_out [CTAs][16 or 64] (16 up to 16
// batch rows), batch row b in column b.  Consumer side, other epilogues: the rows that came in are
// such x * w; the result rows are multiplied by 1 / sqrt(sum of the parts / d + eps), the parts
// ssq_in [n_parts][stride] added in a fixed order that does not depend on the batch.
struct SgNorm {
    bf16* xw_out;
    const float* w_next;
    float* ssq_out;
    int ld_xw;
    const float* ssq_in;
    int n_parts, stride;
    float inv_d, eps;
};


// NT: batch columns / 8.  RT: weight row tiles per CTA (2 for SwiGLU).  U: k steps fetched ahead.
template <int NT, int EPI, typename TC, int U>
__global__ void __launch_bounds__(SG_THREADS)
skinny_gemm_kernel(const bf16* __restrict__ W, const bf16* X, TC* C, int m,
                   int n, int k, int ldw, int ldx, int ldc, int up_row_offset, const SgNorm nm) {
    constexpr int RT = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int NCOL = NT <= 2 ? 16 : 64;             // columns of a part of sums of squares
    constexpr int NPG = 16;                             // groups that share the parts (part p belongs to group p % 16):
                                                        // the same for every batch size, so that a row's sum is
                                                        // added in one order
    constexpr int TG = SG_THREADS / NCOL;               // thread groups (16 or 4), each takes NPG / TG groups of parts
    constexpr int GPT = NPG / TG;
    extern __shared__ float red[];          // [SG_WARPS][RT][16][NT*8]
    __shared__ float nred[NPG][NCOL];       // consumer side of a deferred norm: partial sums [group][batch row]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * 16;
    const bool norm_out = EPI == EPI_ACCUM && nm.ssq_out != nullptr;
    const bool norm_in = EPI != EPI_ACCUM && nm.ssq_in != nullptr;
    // the following norm's weight at the output column this thread writes (a weight: no need to wait for it)
    const float wn = (norm_out && r0 + (threadIdx.x & 15) < n) ? nm.w_next[r0 + (threadIdx.x & 15)] : 0.f;
    float nsum[GPT];
#pragma unroll
    for (int j = 0; j < GPT; ++j) nsum[j] = 0.f;
    bool norm_loaded = false;
    // the parts of the rows' sums of squares, left by the kernel before (so: after the wait): thread
    // (thread group, column) adds the parts of its groups, four loads in flight per group
    auto load_norm = [&]() {
        if (!norm_in || norm_loaded) return;
        norm_loaded = true;
        const int col = threadIdx.x % NCOL, tg = threadIdx.x / NCOL;
        if (col >= nm.stride) return;
        for (int p0 = 0; p0 < nm.n_parts; p0 += 4 * NPG) {
            float f[GPT][4];
#pragma unroll
            for (int j = 0; j < GPT; ++j)
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int p = p0 + u * NPG + tg * GPT + j;
                    f[j][u] = p < nm.n_parts ? __ldcg(nm.ssq_in + (size_t)p * nm.stride + col) : 0.f;
                }
#pragma unroll
            for (int j = 0; j < GPT; ++j)
#pragma unroll
                for (int u = 0; u < 4; ++u) nsum[j] += f[j][u];
        }
    };
    // rows beyond n are clamped for loading and dropped at the store
    const bf16* wrow[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
        const int base = r0 + rt * up_row_offset;
        const int lim = (rt == 0 ? n : n + up_row_offset) - 1;
        wrow[rt][0] = W + (size_t)min(base + g, lim) * ldw + 8 * t;
        wrow[rt][1] = W + (size_t)min(base + g + 8, lim) * ldw + 8 * t;
    }
    const bf16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = 8 * j + g < m;
        xrow[j] = X + (size_t)(xok[j] ? 8 * j + g : 0) * ldx + 8 * t;
    }
    float acc[RT][NT][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rt][j][e] = 0.f;

    const int steps = (k + 31) >> 5;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int s0 = warp; s0 < steps; s0 += SG_WARPS * U) {
        uint4 a[U][RT][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = (s0 + u * SG_WARPS) << 5;
            const bool ok = kk + 8 * t + 8 <= k;       // k % 8 == 0: a 16-byte chunk is whole or absent
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                a[u][rt][0] = ok ? ldg_stream(wrow[rt][0] + kk) : zero;
                a[u][rt][1] = ok ? ldg_stream(wrow[rt][1] + kk) : zero;
            }
        }
        // The weights do not depend on the kernel before this one, the activations do: with a
        // programmatic dependent launch the first weight loads are already in flight while the
        // previous kernel drains.  (Without that launch attribute the wait returns at once.)
        if (s0 == warp) {
            pdl_wait();
            load_norm();               // beside the batch rows' loads, while the weights arrive
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = (s0 + u * SG_WARPS) << 5;
            const bool ok = kk + 8 * t + 8 <= k;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 b = (ok && xok[j]) ? ldg_cached(xrow[j] + kk) : zero;
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    mma16816(acc[rt][j], a[u][rt][0].x, a[u][rt][1].x, a[u][rt][0].y, a[u][rt][1].y, b.x, b.y);
                    mma16816(acc[rt][j], a[u][rt][0].z, a[u][rt][1].z, a[u][rt][0].w, a[u][rt][1].w, b.z, b.w);
                }
            }
        }
    }
    pdl_wait();                 // warps that had no k step still have to wait before they write
    pdl_launch_dependents();    // the next kernel may start to fill the SMs that this one leaves
    load_norm();
    if (norm_in) {
#pragma unroll
        for (int j = 0; j < GPT; ++j) nred[(threadIdx.x / NCOL) * GPT + j][threadIdx.x % NCOL] = nsum[j];
    }
    // partial sums -> shared memory [warp][rt][row 0..15][batch 0..NT*8)
    constexpr int NB = NT * 8;
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float* base = red + ((size_t)(warp * RT + rt) * 16) * NB;
            base[(g)*NB + 8 * j + 2 * t] = acc[rt][j][0];
            base[(g)*NB + 8 * j + 2 * t + 1] = acc[rt][j][1];
            base[(g + 8) * NB + 8 * j + 2 * t] = acc[rt][j][2];
            base[(g + 8) * NB + 8 * j + 2 * t + 1] = acc[rt][j][3];
        }
    __syncthreads();
    // outputs: 16 rows x NB batch columns; consecutive threads take consecutive rows (contiguous in C)
    // (16 * NB is a multiple of 32: a warp is in the loop with all its lanes or not at all)
    for (int o = threadIdx.x; o < 16 * NB; o += SG_THREADS) {
        const int row = o & 15, b = o >> 4;
        const bool ok = b < m && r0 + row < n;
        float v[RT];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < SG_WARPS; ++w) s += red[((size_t)(w * RT + rt) * 16 + row) * NB + b];
            v[rt] = s;
        }
        if (norm_in) {
            float tot = 0.f;
#pragma unroll
            for (int pg = 0; pg < NPG; ++pg) tot += nred[pg][b];
            const float rs = 1.0f / sqrtf(tot * nm.inv_d + nm.eps);
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) v[rt] *= rs;
        }
        TC* c = C + (size_t)(ok ? b : 0) * ldc + (ok ? r0 + row : 0);
        float x_new = 0.f;
        if (ok) {
            if (EPI == EPI_STORE) *c = from_f<TC>(v[0]);
            else if (EPI == EPI_ACCUM) { x_new = to_f<TC>(*c) + v[0]; *c = from_f<TC>(x_new); }
            else *c = from_f<TC>(v[0] / (1.0f + expf(-v[0])) * v[RT - 1]);
        }
        if (norm_out) {
            if (ok) nm.xw_out[(size_t)b * nm.ld_xw + r0 + row] = __float2bfloat16(x_new * wn);
            // the 16 lanes of a half-warp hold the 16 rows of batch column b
            float sq = x_new * x_new;
            sq += __shfl_xor_sync(0xffffffffu, sq, 8);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            if (row == 0) nm.ssq_out[(size_t)blockIdx.x * NCOL + b] = sq;
        }
    }
}

template <int NT, int EPI, typename TC>
static int launch_sg(const bf16* W, const bf16* X, void* C, int m, int n, int k, int ldw, int ldx, int ldc,
                     int up_row_offset, const SgNorm& nm, cudaStream_t stream) {
    constexpr int RT = (EPI == EPI_SWIGLU) ? 2 : 1;
    // k steps fetched ahead: 16 weight loads of 16 bytes in flight per thread where registers allow
    constexpr int U = (NT * RT >= 8) ? 2 : (NT >= 2 ? 4 : 8 / RT);
    const size_t smem = (size_t)SG_WARPS * RT * 16 * NT * 8 * sizeof(float);
    auto kern = skinny_gemm_kernel<NT, EPI, TC, U>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return rllm_launch(kern, dim3((n + 15) / 16), dim3(SG_THREADS), smem, stream, W, X, (TC*)C, m, n, k, ldw, ldx,
                       ldc, up_row_offset, nm);
}

template <int EPI, typename TC>
static int dispatch_nt(const bf16* W, const bf16* X, void* C, int m, int n, int k, int ldw, int ldx, int ldc,
                       int up, const SgNorm& nm, cudaStream_t s) {
    if (m <= 8) return launch_sg<1, EPI, TC>(W, X, C, m, n, k, ldw, ldx, ldc, up, nm, s);
    if (m <= 16) return launch_sg<2, EPI, TC>(W, X, C, m, n, k, ldw, ldx, ldc, up, nm, s);
    if (m <= 32) return launch_sg<4, EPI, TC>(W, X, C, m, n, k, ldw, ldx, ldc, up, nm, s);
    return launch_sg<8, EPI, TC>(W, X, C, m, n, k, ldw, ldx, ldc, up, nm, s);
}

// epilogue: 0 store, 1 accumulate into float32 C, 2 SwiGLU (W holds n gate rows then, from row
// up_row_offset on, n up rows; C is [m, n]).  Requires m <= 64, k % 8 == 0, ldw % 8 == 0,
// ldx % 8 == 0 and 16-byte aligned W and X; returns cudaErrorInvalidValue otherwise.
// A deferred RMSNorm (SgNorm above).  Producer, accumulate epilogue, xw_out != null: xw_out [m, ld_xw]
// bfloat16, w_next [n] float32, ssq_out [ceil(n / 16)][m <= 16 ? 16 : 64] float32.  Consumer, other
// epilogues, ssq_in != null: n_parts_in parts of ssq_stride_in (>= m) columns, norm_d the length of the
// rows that were squared, norm_eps.
RLLM_API int rllm_skinny_gemm(const void* W, const void* X, void* C, int c_dtype, int m, int n, int k,
                              int ldw, int ldx, int ldc, int epilogue, int up_row_offset,
                              void* xw_out, int ld_xw, const float* w_next, float* ssq_out, const float* ssq_in,
                              int n_parts_in, int ssq_stride_in, int norm_d, float norm_eps, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 64 || k <= 0 || (k & 7) || (ldw & 7) || (ldx & 7) || ((uintptr_t)W & 15) || ((uintptr_t)X & 15))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_ACCUM && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    SgNorm nm = {};
    if (xw_out) {
        if (epilogue != EPI_ACCUM || !w_next || !ssq_out || ld_xw < n) return (int)cudaErrorInvalidValue;
        nm.xw_out = (bf16*)xw_out; nm.w_next = w_next; nm.ssq_out = ssq_out; nm.ld_xw = ld_xw;
    }
    if (ssq_in) {
        if (epilogue == EPI_ACCUM || n_parts_in <= 0 || norm_d <= 0 || ssq_stride_in < m)
            return (int)cudaErrorInvalidValue;
        nm.ssq_in = ssq_in; nm.n_parts = n_parts_in; nm.stride = ssq_stride_in; nm.inv_d = 1.0f / (float)norm_d;
        nm.eps = norm_eps;
    }
    const bf16* w = (const bf16*)W;
    const bf16* x = (const bf16*)X;
    if (epilogue == EPI_STORE) {
        return c_dtype == RLLM_F32 ? dispatch_nt<EPI_STORE, float>(w, x, C, m, n, k, ldw, ldx, ldc, 0, nm, stream)
                                   : dispatch_nt<EPI_STORE, bf16>(w, x, C, m, n, k, ldw, ldx, ldc, 0, nm, stream);
    } else if (epilogue == EPI_ACCUM) {
        return dispatch_nt<EPI_ACCUM, float>(w, x, C, m, n, k, ldw, ldx, ldc, 0, nm, stream);
    } else if (epilogue == EPI_SWIGLU) {
        return c_dtype == RLLM_F32
                   ? dispatch_nt<EPI_SWIGLU, float>(w, x, C, m, n, k, ldw, ldx, ldc, up_row_offset, nm, stream)
                   : dispatch_nt<EPI_SWIGLU, bf16>(w, x, C, m, n, k, ldw, ldx, ldc, up_row_offset, nm, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_skinny_gemm)
