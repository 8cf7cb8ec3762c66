// Blackwell tensor-core product for many rows: D[M,N] = A[M,K] . B[N,K]^T, bfloat16 operands,
// float32 accumulation in tensor memory (TMEM), operands staged in shared memory by TMA.
//
//   * persistent CTAs (one per SM) walk over 128 x 256 output tiles; K is walked in blocks of 64
//     elements through a ring of shared-memory stages, each holding a [128 x 64] A tile and a
//     [256 x 64] B tile in the 128-byte-swizzled K-major layout that both TMA writes and
//     tcgen05.mma reads; two accumulators in TMEM let one tile's epilogue overlap the next tile's MMAs;
//   * warp 0 (one elected lane) issues the TMA loads (cp.async.bulk.tensor.2d) and arms the
//     stage's "full" mbarrier with the byte count; warp 1 (one elected lane) issues
//     tcgen05.mma.cta_group::1.kind::f16 (M = 128, N = BN, K = 16, four per stage) and releases
//     the stage with tcgen05.commit on its "empty" mbarrier; after the last block a commit on the
//     "accumulator full" mbarrier hands the tile to the epilogue;
//   * warps 2..5 are the epilogue: each owns 32 TMEM lanes (= 32 rows of the tile), reads its row
//     with tcgen05.ld 32 columns at a time and writes it out: store (float32 or bfloat16),
//     accumulate into a float32 C (the residual stream), or SwiGLU (the B tile holds 128 gate rows
//     and the 128 up rows of the same index; out = silu(gate) * up).
//   Rows beyond M and columns beyond N come in as zeros from TMA and are dropped at the store.
//
// Every wait on an mbarrier is bounded: when the limit is hit the thread records a code in the
// error word, raises the CTA's abort flag, every role leaves its loop, copies still in flight are
// waited for (bounded again), TMEM is freed and the kernel returns; the host reads the error word.
//
// AxiomOperator/rllm hands these products to cuBLAS (crates/rllm-cuda/src/gpu.rs:238-268) and
// follows gate/up with a separate silu_mul kernel (crates/rllm-cuda/kernels/kernels.cu:1212-1219).
#include "tcgen05.cuh"
#include <math.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

enum { TC_EPI_STORE = 0, TC_EPI_ACCUM = 1, TC_EPI_SWIGLU = 2 };
enum { TC_ERR_FULL = 1, TC_ERR_EMPTY = 2, TC_ERR_ACC = 3 };

// ---------------------------------------------------------------- the kernel
template <typename TC> __device__ __forceinline__ void store_row32(TC* dst, const float (&v)[32], int n_valid);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int n_valid) {
    if (n_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < n_valid) dst[j] = v[j];
    }
}
template <> __device__ __forceinline__ void store_row32<bf16>(bf16* dst, const float (&v)[32], int n_valid) {
    if (n_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 u;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
            u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
            u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
            reinterpret_cast<uint4*>(dst)[j] = u;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < n_valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

// Persistent: the grid is one CTA per SM; CTA c takes tiles c, c + grid, c + 2 grid, ... (m fastest, so
// the CTAs running together share few weight rows and the whole of A stays in L2).  Two accumulator
// buffers in TMEM (2 x BN columns): the epilogue of one tile overlaps the MMAs of the next, and the
// operand ring never drains between tiles.
template <int BN, int EPI, typename TC, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, TC* __restrict__ C,
               int ldc, int M, int N, int K, int up_row_offset, int* __restrict__ err) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2;
    constexpr int B_BYTES = BN * TC_BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BN_OUT = (EPI == TC_EPI_SWIGLU) ? BN / 2 : BN;        // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + BN_OUT - 1) / BN_OUT;
    const int total_tiles = m_tiles * n_tiles;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();                                    // the A operand is written by the kernel before

    if (warp == 0 && lane == 0) {
        // ---- TMA producer: one continuous ring over all of this CTA's tiles
        int it = 0, issued = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN_OUT;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag)) {
                    if (!abort_flag) { atomicExch(err, TC_ERR_EMPTY); abort_flag = 1; }
                    ok = false;
                    break;
                }
                unsigned char* a_s = smem + (size_t)s * STAGE_BYTES;
                unsigned char* b_s = a_s + A_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a_s, &tmA, kb * TC_BK, m0, &full_bar[s]);
                if (EPI == TC_EPI_SWIGLU) {
                    tma_load_2d(b_s, &tmB, kb * TC_BK, n0, &full_bar[s]);
                    tma_load_2d(b_s + B_BYTES / 2, &tmB, kb * TC_BK, up_row_offset + n0, &full_bar[s]);
                } else {
                    tma_load_2d(b_s, &tmB, kb * TC_BK, n0, &full_bar[s]);
                }
                issued = it + 1;
            }
        }
        if (abort_flag) {
            // copies already issued must land before the CTA's shared memory goes away
            volatile int no_abort = 0;
            for (int i = max(0, issued - STAGES); i < issued; ++i)
                mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1, &no_abort);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = idesc_bf16(TC_BM, BN);
        int it = 0, local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            // the epilogue of the tile that used this buffer two tiles ago must have read it
            if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, TC_ERR_ACC); abort_flag = 1; }
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph, &abort_flag)) {
                    if (!abort_flag) { atomicExch(err, TC_ERR_FULL); abort_flag = 1; }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = s_addr(smem + (size_t)s * STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)       // 16 elements = 32 bytes along K: +2 in 16-byte units
                    umma_bf16(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb | kk) != 0);
                umma_commit(&empty_bar[s]);                  // arrives when these MMAs have read the stage
            }
            if (ok) umma_commit(&acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        int local = 0;
        bool first = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN_OUT;
            const int gm = m0 + row;
            bool ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, &abort_flag);
            if (!ok && !abort_flag) { atomicExch(err, TC_ERR_ACC); abort_flag = 1; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (first && tile + (int)gridDim.x >= total_tiles) { pdl_launch_dependents(); first = false; }
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < BN_OUT; c0 += 32) {
                uint32_t r[32];
                float v[32];
                tmem_ld32(taddr + c0, r);
                if (EPI == TC_EPI_SWIGLU) {
                    uint32_t u[32];
                    tmem_ld32(taddr + BN / 2 + c0, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g = __uint_as_float(r[j]);
                        v[j] = g / (1.0f + __expf(-g)) * __uint_as_float(u[j]);
                    }
                } else {
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                }
                if (c0 + 32 >= BN_OUT) {                     // all of this thread's TMEM reads of the tile are done
                    tc_fence_before();
                    mbar_arrive(&acc_empty[buf]);
                }
                const int gn = n0 + c0;
                if (gm < M && gn < N) {
                    TC* dst = C + (size_t)gm * ldc + gn;
                    const int n_valid = min(32, N - gn);
                    if (EPI == TC_EPI_ACCUM) {
                        if (sizeof(TC) == 4 && n_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 c4 = reinterpret_cast<const float4*>(dst)[j];
                                v[4 * j] += c4.x; v[4 * j + 1] += c4.y; v[4 * j + 2] += c4.z; v[4 * j + 3] += c4.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (j < n_valid) v[j] += to_f<TC>(dst[j]);
                        }
                    }
                    store_row32<TC>(dst, v, n_valid);
                }
            }
        }
    }
    __syncwarp();          // the lanes that had no role meet the elected one: the barrier below wants whole warps
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ---------------------------------------------------------------- host side
// Tensor map of a row-major bfloat16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zero fill outside.  Needs a 16-byte aligned base and
// ld a multiple of 8.
static int make_tmap(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    TmapEncodeFn enc = tmap_encoder();
    if (!enc) return 30001;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 30000 + (int)r;
}

template <int BN, int EPI, typename TC, int STAGES>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int ldc, int M, int N, int K, int up,
                     int* err, cudaStream_t stream) {
    constexpr int BN_OUT = (EPI == TC_EPI_SWIGLU) ? BN / 2 : BN;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    auto kern = gemm_tc_kernel<BN, EPI, TC, STAGES>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        if (n_sm <= 0) n_sm = 148;
    }
    const int tiles = ((M + TC_BM - 1) / TC_BM) * ((N + BN_OUT - 1) / BN_OUT);
    dim3 grid(tiles < n_sm ? tiles : n_sm);
    return rllm_launch(kern, grid, dim3(TC_THREADS), smem, stream, ta, tb, (TC*)C, ldc, M, N, K, up, err);
}

// C[M,N] (+)= A[M,K] . B[N,K]^T on the tcgen05 tensor cores.  epilogue 0 store, 1 accumulate into a
// float32 C, 2 SwiGLU (B holds N gate rows and, from row up_row_offset, N up rows; C[M,N] =
// silu(gate) * up).  A, B bfloat16 row-major with 16-byte aligned bases and lda, ldb multiples of 8;
// K a multiple of 8.  `err` is a device int that receives a code if a bounded wait ran out.
// Returns 0, a cudaError_t, 30000 + CUresult of the tensor-map encoder, or cudaErrorInvalidValue.
RLLM_API int rllm_gemm_tc(const void* A, const void* B, void* C, int c_dtype, int M, int N, int K, int lda, int ldb,
                          int ldc, int epilogue, int up_row_offset, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || !err)
        return (int)cudaErrorInvalidValue;
    if (epilogue == TC_EPI_ACCUM && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    CUtensorMap ta, tb;
    int st = make_tmap(&ta, A, M, K, lda, TC_BM);
    if (st) return st;
    const int b_rows = epilogue == TC_EPI_SWIGLU ? up_row_offset + N : N;
    const int b_box = epilogue == TC_EPI_SWIGLU ? 128 : 256;
    st = make_tmap(&tb, B, b_rows, K, ldb, b_box);
    if (st) return st;
    if (epilogue == TC_EPI_STORE) {
        return c_dtype == RLLM_F32 ? launch_tc<256, TC_EPI_STORE, float, 4>(ta, tb, C, ldc, M, N, K, 0, err, stream)
                                   : launch_tc<256, TC_EPI_STORE, bf16, 4>(ta, tb, C, ldc, M, N, K, 0, err, stream);
    } else if (epilogue == TC_EPI_ACCUM) {
        return launch_tc<256, TC_EPI_ACCUM, float, 4>(ta, tb, C, ldc, M, N, K, 0, err, stream);
    } else if (epilogue == TC_EPI_SWIGLU) {
        return c_dtype == RLLM_F32
                   ? launch_tc<256, TC_EPI_SWIGLU, float, 4>(ta, tb, C, ldc, M, N, K, up_row_offset, err, stream)
                   : launch_tc<256, TC_EPI_SWIGLU, bf16, 4>(ta, tb, C, ldc, M, N, K, up_row_offset, err, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// =====================================================================================================
// Few rows (decode): the same machinery with the operands swapped.  The weight matrix W[n,k] is the
// M side (128 weight rows per CTA, streamed once from HBM through a deep TMA ring), the m <= 64
// batch rows X[m,k] are the N side, so the accumulator D[weight row, batch row] is C transposed.
// The K range may be split over the grid.y CTAs of a thread-block cluster to fill the machine when
// n/128 is small: each CTA accumulates its K slice and parks its sums in its own shared memory.
// With 2, 4 or 8 CTAs every CTA of the cluster then takes its share of the tile's weight rows,
// reads those rows' sums from all CTAs through distributed shared memory (mapa / ld.shared::cluster)
// in rank order, which is ascending k, and writes its share of C; the old values of an
// accumulating C are fetched while the MMAs still run.  (With the leader alone adding and writing,
// the kernel's last 6 us were a chain of round trips: 192 loads through distributed shared memory
// per thread, then 64 loads of C, then 64 stores; spread over four CTAs they take 2.)  Other split
// counts, and SwiGLU, leave the additions to the cluster's leader.  No global scratch, no atomics,
// a fixed order of addition.  SwiGLU: a CTA takes 64 gate rows and the 64 up rows of the same
// index; the up rows' sums reach the gate rows' threads through shared memory.
// =====================================================================================================
// The sums of one weight row for BN / S batch columns, parked by the S CTAs of a cluster in their
// shared memory as [batch column][weight row]: all loads are issued before the first addition (a
// round trip through distributed shared memory takes about 200 ns), the additions run in rank order.
template <int BN, int S>
__device__ __forceinline__ void cluster_row_sums(uint32_t red_addr, uint32_t elem_offset, float (&acc)[BN / 2]) {
    constexpr int COLS = BN / S;
    float f[S][COLS];
#pragma unroll
    for (int z = 0; z < S; ++z) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr), "r"(z));
        remote += elem_offset * 4;
#pragma unroll
        for (int i = 0; i < COLS; ++i)
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(f[z][i]) : "r"(remote + (uint32_t)(i * TC_BM) * 4) : "memory");
    }
#pragma unroll
    for (int i = 0; i < COLS; ++i) {
        float a = f[0][i];
#pragma unroll
        for (int z = 1; z < S; ++z) a += f[z][i];
        acc[i] = a;
    }
}

// An RMSNorm whose kernel this product saves (the contract of gemv_stream.cu's SvNorm, with 64
// columns per part).  Producer side, accumulate epilogue: beside the sums x it writes into C, the
// launch writes bfloat16(x * w_next) and, per CTA, the sums of squares of the x it wrote (row b of
// the batch in column b of part tile * splits + split; a CTA that writes nothing writes zeros).
// Consumer side, store and SwiGLU epilogues: the rows that came in are such x * w; the result rows
// are multiplied by 1 / sqrt(sum of the parts / d + eps).  The parts are added in a fixed order.
struct SwapNorm {
    bf16* xw_out;
    const float* w_next;
    float* ssq_out;
    int ld_xw;
    const float* ssq_in;
    int n_parts, stride;      // parts of `stride` columns: 64 from this kernel, 16 from gemv_stream and skinny_gemm
    float inv_d, eps;
};
#define SWAP_NORM_COLS 64

template <int BN, int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(TC_THREADS, STAGES > 4 ? 1 : 2)
gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    TC* __restrict__ C, int ldc, int m, int n, int K, int up_row_offset, int* __restrict__ err,
                    const SwapNorm nrm) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2;          // 128 weight rows x 64 k
    constexpr int B_BYTES = BN * TC_BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int ROWS_OUT = (EPI == TC_EPI_SWIGLU) ? TC_BM / 2 : TC_BM;     // output columns of C per CTA
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float norm_part[8][SWAP_NORM_COLS];          // consumer side of a deferred norm: partial sums,
    __shared__ float norm_rs[SWAP_NORM_COLS];               // and 1 / rms per batch row
    float* red = reinterpret_cast<float*>(smem);            // exchange buffer: the stages are free once the MMAs are done
    float* sq = red + BN * TC_BM;                           // producer side: squares [weight row][BN + 1]
    const bool norm_out = EPI == TC_EPI_ACCUM && nrm.ssq_out != nullptr;
    const bool norm_in = EPI != TC_EPI_ACCUM && nrm.ssq_in != nullptr;
    float wn = 0.f;                                         // the following norm's weight at this thread's column
    float v[BN];                                            // this thread's accumulator row (epilogue warps)
    float c_old[EPI == TC_EPI_ACCUM ? BN : 1];              // and the values of C it adds to
#pragma unroll
    for (int j = 0; j < BN; ++j) v[j] = 0.f;
#pragma unroll
    for (int j = 0; j < (EPI == TC_EPI_ACCUM ? BN : 1); ++j) c_old[j] = 0.f;
    bool ep_ok = true;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int n0 = tile * ROWS_OUT;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    const int kb_per = (nkb + n_splits - 1) / n_splits;
    const int kb0 = split * kb_per, kb1 = min(nkb, kb0 + kb_per);
    const int my_kb = max(0, kb1 - kb0);
    // With 2, 4 or 8 CTAs on a tile the sums are added and written by all of them, each taking its
    // share of the tile's weight rows (`scatter`): thread t of the 128 epilogue threads takes row
    // split * R + t % R (R = 128 / n_splits rows per CTA) and the batch columns of group t / R.
    const bool scatter = EPI != TC_EPI_SWIGLU && (n_splits == 2 || n_splits == 4 || n_splits == 8);
    const int sc_rows = TC_BM / n_splits, sc_cols = BN / n_splits;
    const int sc_t = (warp & 3) * 32 + lane;
    const int sc_row = scatter ? split * sc_rows + (sc_t & (sc_rows - 1)) : 0;
    const int sc_b0 = scatter ? (sc_t / sc_rows) * sc_cols : 0;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, BN < 32 ? 32 : BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer.  The weights do not depend on the kernel before: their loads start at once;
        // the activations are loaded only after the wait.
        int issued = 0;
        bool waited = false;
        for (int i = 0; i < my_kb; ++i) {
            const int kb = kb0 + i, s = i % STAGES;
            const uint32_t ph = (i / STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, TC_ERR_EMPTY); abort_flag = 1; }
                break;
            }
            unsigned char* a_s = smem + (size_t)s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            if (EPI == TC_EPI_SWIGLU) {
                tma_load_2d(a_s, &tmW, kb * TC_BK, n0, &full_bar[s]);
                tma_load_2d(a_s + A_BYTES / 2, &tmW, kb * TC_BK, up_row_offset + n0, &full_bar[s]);
            } else {
                tma_load_2d(a_s, &tmW, kb * TC_BK, n0, &full_bar[s]);
            }
            if (!waited) { pdl_wait(); waited = true; }
            tma_load_2d(a_s + A_BYTES, &tmX, kb * TC_BK, 0, &full_bar[s]);
            issued = i + 1;
        }
        if (abort_flag) {
            for (int i = max(0, issued - STAGES); i < issued; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                { volatile int no_abort = 0; mbar_wait(&full_bar[s], ph, &no_abort); }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = idesc_bf16(TC_BM, BN);
        bool ok = true;
        for (int i = 0; i < my_kb && ok; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (i / STAGES) & 1;
            if (!mbar_wait(&full_bar[s], ph, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, TC_ERR_FULL); abort_flag = 1; }
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t a_addr = s_addr(smem + (size_t)s * STAGE_BYTES);
            const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
            for (int kk = 0; kk < TC_BK / 16; ++kk)
                umma_bf16(tmem_base, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (i | kk) != 0);
            umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_bar);
    } else if (warp >= 2) {
        // ---- epilogue, first half: accumulator -> registers (thread = weight row, registers = batch columns)
        pdl_wait();                                     // C may be touched from here on
        const int quarter = warp & 3;
        if (EPI == TC_EPI_ACCUM && scatter) {
            // the old values of C: fetched while the MMAs run, so that the end of the kernel does not wait for them
            if (n0 + sc_row < n) {
#pragma unroll
                for (int i = 0; i < BN / 2; ++i)
                    if (i < sc_cols && sc_b0 + i < m) c_old[i] = to_f<TC>(C[(size_t)(sc_b0 + i) * ldc + n0 + sc_row]);
                if (norm_out) wn = nrm.w_next[n0 + sc_row];
            }
        } else if (EPI == TC_EPI_ACCUM && split == 0) {
            const int out_col = n0 + quarter * 32 + lane;
            if (out_col < n) {
#pragma unroll
                for (int b = 0; b < BN; ++b)
                    if (b < m) c_old[b] = to_f<TC>(C[(size_t)b * ldc + out_col]);
                if (norm_out) wn = nrm.w_next[out_col];
            }
        }
        if (norm_in) {
            // 1 / rms of the rows that came in, from the parts the kernel before left (ordinary loads:
            // they are its output), also while the MMAs run: 16 threads take the 64 columns four at a
            // time, 8 such groups share the parts, four loads in flight each
            const int t = quarter * 32 + lane, c4 = (t & 15) * 4, g = t >> 4;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c4 < BN && c4 < nrm.stride) {
                for (int p0 = g; p0 < nrm.n_parts; p0 += 32) {
                    float4 f[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int p = p0 + 8 * u;
                        f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (p < nrm.n_parts)
                            asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(f[u].x), "=f"(f[u].y), "=f"(f[u].z), "=f"(f[u].w)
                                         : "l"(nrm.ssq_in + (size_t)p * nrm.stride + c4) : "memory");
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) { a.x += f[u].x; a.y += f[u].y; a.z += f[u].z; a.w += f[u].w; }
                }
            }
            norm_part[g][c4] = a.x; norm_part[g][c4 + 1] = a.y; norm_part[g][c4 + 2] = a.z; norm_part[g][c4 + 3] = a.w;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (t < SWAP_NORM_COLS) {
                float tot = 0.f;
#pragma unroll
                for (int gg = 0; gg < 8; ++gg) tot += norm_part[gg][t];
                norm_rs[t] = 1.0f / sqrtf(tot * nrm.inv_d + nrm.eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (my_kb > 0) {
            ep_ok = mbar_wait(&acc_bar, 0, &abort_flag);
            if (!ep_ok && !abort_flag) { atomicExch(err, TC_ERR_ACC); abort_flag = 1; }
        }
        ep_ok = __all_sync(0xffffffffu, ep_ok);
        if (ep_ok && my_kb > 0) {
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) v[c0 + j] = __uint_as_float(r[j]);
            }
        }
        pdl_launch_dependents();
        if (n_splits > 1 && (split > 0 || scatter)) {
            // park the partial sums in this CTA's own shared memory for the CTAs that add them
            // (the stages are free: all MMAs that read them have completed)
            const int row = quarter * 32 + lane;
#pragma unroll
            for (int b = 0; b < BN; ++b) red[b * TC_BM + row] = v[b];
        }
    }
    __syncwarp();          // the lanes that had no role meet the elected one: the barriers below want whole warps
    tc_fence_before();
    __syncthreads();
    if (n_splits > 1) {
        // Every thread of every CTA of the cluster comes here, whatever happened before: the
        // cluster barrier has no time-out.  #1: the followers' partial sums are in place.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp >= 2 && scatter) {
        // ---- epilogue, second half, shared by the cluster: this thread's row and columns from every
        // CTA's parked sums (its own among them), in rank order, which is ascending k
        float acc[BN / 2];
#pragma unroll
        for (int i = 0; i < BN / 2; ++i) acc[i] = 0.f;
        const uint32_t off = (uint32_t)(sc_b0 * TC_BM + sc_row);
        if (n_splits == 2) cluster_row_sums<BN, 2>(s_addr(red), off, acc);
        else if (n_splits == 4) cluster_row_sums<BN, 4>(s_addr(red), off, acc);
        else cluster_row_sums<BN, 8>(s_addr(red), off, acc);
        const int out_col = n0 + sc_row;
        const bool row_ok = ep_ok && out_col < n;
        const int rl = sc_t & (sc_rows - 1);
#pragma unroll
        for (int i = 0; i < BN / 2; ++i)
            if (i < sc_cols) {
                const int b = sc_b0 + i;
                const bool ok = row_ok && b < m;
                float o = (EPI == TC_EPI_ACCUM) ? acc[i] + c_old[i] : acc[i];
                if (norm_in) o *= norm_rs[b];
                if (ok) C[(size_t)b * ldc + out_col] = from_f<TC>(o);
                if (norm_out) {
                    if (ok) nrm.xw_out[(size_t)b * nrm.ld_xw + out_col] = __float2bfloat16(o * wn);
                    sq[rl * (BN + 1) + b] = ok ? o * o : 0.f;
                }
            }
        if (norm_out) {
            // this CTA's part: for every batch row the squares of its sc_rows weight rows, in row order
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (sc_t < BN) {
                float tot = 0.f;
                for (int r = 0; r < sc_rows; ++r) tot += sq[r * (BN + 1) + sc_t];
                nrm.ssq_out[(size_t)(tile * n_splits + split) * SWAP_NORM_COLS + sc_t] = tot;
            }
        }
    } else if (warp >= 2 && split == 0) {
        // ---- epilogue, second half (the cluster's leader): add the followers' sums in rank order, write out
        const int row = (warp & 3) * 32 + lane;
        for (int z = 1; z < n_splits; ++z) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(s_addr(red)), "r"(z));
            // 16 loads in flight at a time: issued one by one with the addition between them, each
            // would wait for the round trip of the one before
#pragma unroll
            for (int b0 = 0; b0 < BN; b0 += 16) {
                float f[16];
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(f[i]) : "r"(remote + (uint32_t)((b0 + i) * TC_BM + row) * 4) : "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) v[b0 + i] += f[i];
            }
        }
        // global weight row of this thread (SwiGLU: rows 0..63 gate j, rows 64..127 up j)
        const int out_col = (EPI == TC_EPI_SWIGLU) ? n0 + (row & 63) : n0 + row;
        const bool col_ok = out_col < n;
        if (EPI == TC_EPI_SWIGLU) {
            if (ep_ok && row >= 64) {
#pragma unroll
                for (int b = 0; b < BN; ++b) red[b * 64 + (row - 64)] = v[b];      // consecutive rows, consecutive banks
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps
            if (ep_ok && row < 64 && col_ok) {
#pragma unroll
                for (int b = 0; b < BN; ++b)
                    if (b < m) {
                        const float rs = norm_in ? norm_rs[b] : 1.0f;
                        const float g = v[b] * rs;
                        C[(size_t)b * ldc + out_col] = from_f<TC>(__fdividef(g, 1.0f + __expf(-g)) * (red[b * 64 + row] * rs));
                    }
            }
        } else {
            const bool row_ok = ep_ok && col_ok;
            if (EPI == TC_EPI_ACCUM) {
#pragma unroll
                for (int b = 0; b < BN; ++b) v[b] += c_old[b];
            }
#pragma unroll
            for (int b = 0; b < BN; ++b) {
                const bool ok = row_ok && b < m;
                if (norm_in) v[b] *= norm_rs[b];
                if (ok) C[(size_t)b * ldc + out_col] = from_f<TC>(v[b]);
                if (norm_out) {
                    if (ok) nrm.xw_out[(size_t)b * nrm.ld_xw + out_col] = __float2bfloat16(v[b] * wn);
                    sq[row * (BN + 1) + b] = ok ? v[b] * v[b] : 0.f;
                }
            }
            if (norm_out) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (row < BN) {
                    float tot = 0.f;
                    for (int r = 0; r < TC_BM; ++r) tot += sq[r * (BN + 1) + row];
                    nrm.ssq_out[(size_t)(tile * n_splits + split) * SWAP_NORM_COLS + row] = tot;
                }
            }
        }
    } else if (warp >= 2 && norm_out) {
        // a follower of a cluster whose leader writes everything: its part is empty
        const int t = (warp & 3) * 32 + lane;
        if (t < BN) nrm.ssq_out[(size_t)(tile * n_splits + split) * SWAP_NORM_COLS + t] = 0.f;
    }
    if (n_splits > 1) {
        // #2: the leader has read the followers' shared memory; they may exit
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    if (warp == 1) tmem_dealloc(tmem_base, BN < 32 ? 32 : BN);
}

template <int BN, int EPI, typename TC, int STAGES>
static int launch_swap_stages(const CUtensorMap& tw, const CUtensorMap& tx, void* C, int ldc, int m, int n, int K, int up,
                              int n_splits, int* err, const SwapNorm& nrm, cudaStream_t stream) {
    constexpr int ROWS_OUT = (EPI == TC_EPI_SWIGLU) ? TC_BM / 2 : TC_BM;
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    auto kern = gemm_tc_swap_kernel<BN, STAGES, EPI, TC>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid((n + ROWS_OUT - 1) / ROWS_OUT, n_splits);
    return rllm_launch_cluster(kern, grid, dim3(TC_THREADS), smem, stream, n_splits, tw, tx, (TC*)C, ldc, m, n, K, up,
                               err, nrm);
}

// At most one CTA per SM: a ring of 8 stages, so that a single CTA keeps 190 KB in flight.  More
// CTAs than SMs: 4 stages, two CTAs share an SM and one streams while the other starts or ends.
template <int BN, int EPI, typename TC>
static int launch_swap(const CUtensorMap& tw, const CUtensorMap& tx, void* C, int ldc, int m, int n, int K, int up,
                       int n_splits, int* err, const SwapNorm& nrm, cudaStream_t stream) {
    constexpr int ROWS_OUT = (EPI == TC_EPI_SWIGLU) ? TC_BM / 2 : TC_BM;
    const int ctas = ((n + ROWS_OUT - 1) / ROWS_OUT) * n_splits;
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n_sm = 148;
    }
    if (ctas <= n_sm)
        return launch_swap_stages<BN, EPI, TC, 8>(tw, tx, C, ldc, m, n, K, up, n_splits, err, nrm, stream);
    return launch_swap_stages<BN, EPI, TC, 4>(tw, tx, C, ldc, m, n, K, up, n_splits, err, nrm, stream);
}

// C[m,n] (+)= X[m,k] . W[n,k]^T for m <= 64 with W as the streamed operand (see above).
// n_splits (1..8) CTAs of a cluster share each tile's K range.
// A deferred RMSNorm (SwapNorm above).  Producer, accumulate epilogue, xw_out != null: xw_out
// [m, ld_xw] bfloat16, w_next [n] float32, ssq_out [ceil(n / 128) * n_splits, 64] float32.
// Consumer, other epilogues, ssq_in != null: n_parts_in parts of ssq_stride_in columns (>= m, a
// multiple of 4), norm_d the length of the rows that were squared, norm_eps.
RLLM_API int rllm_gemm_tc_swap(const void* W, const void* X, void* C, int c_dtype, int m, int n, int K, int ldw,
                               int ldx, int ldc, int epilogue, int up_row_offset, int n_splits, int* err,
                               void* xw_out, int ld_xw, const float* w_next, float* ssq_out, const float* ssq_in,
                               int n_parts_in, int ssq_stride_in, int norm_d, float norm_eps, cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 64 || K <= 0 || (K & 7) || (ldw & 7) || (ldx & 7) || ((uintptr_t)W & 15) || ((uintptr_t)X & 15) || !err ||
        n_splits < 1 || n_splits > 8)
        return (int)cudaErrorInvalidValue;
    if (epilogue == TC_EPI_ACCUM && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    CUtensorMap tw, tx;
    const int w_rows = epilogue == TC_EPI_SWIGLU ? up_row_offset + n : n;
    int st = make_tmap(&tw, W, w_rows, K, ldw, epilogue == TC_EPI_SWIGLU ? 64 : 128);
    if (st) return st;
    const int bn = m <= 32 ? 32 : 64;
    st = make_tmap(&tx, X, m, K, ldx, bn);
    if (st) return st;
    SwapNorm nrm = {};
    if (xw_out) {
        if (epilogue != TC_EPI_ACCUM || !w_next || !ssq_out || ld_xw < n) return (int)cudaErrorInvalidValue;
        nrm.xw_out = (bf16*)xw_out; nrm.w_next = w_next; nrm.ssq_out = ssq_out; nrm.ld_xw = ld_xw;
    }
    if (ssq_in) {
        // the rows' columns are read four at a time: parts of a multiple of 4 columns, all of the batch's
        if (epilogue == TC_EPI_ACCUM || n_parts_in <= 0 || norm_d <= 0 || ((uintptr_t)ssq_in & 15) ||
            (ssq_stride_in & 3) || ssq_stride_in < m)
            return (int)cudaErrorInvalidValue;
        nrm.ssq_in = ssq_in; nrm.n_parts = n_parts_in; nrm.stride = ssq_stride_in; nrm.inv_d = 1.0f / (float)norm_d;
        nrm.eps = norm_eps;
    }
#define SWAP(BN_, EPI_, TC_) \
    return launch_swap<BN_, EPI_, TC_>(tw, tx, C, ldc, m, n, K, up_row_offset, n_splits, err, nrm, stream)
    if (epilogue == TC_EPI_STORE) {
        if (c_dtype == RLLM_F32) { if (bn == 32) { SWAP(32, TC_EPI_STORE, float); } SWAP(64, TC_EPI_STORE, float); }
        if (bn == 32) { SWAP(32, TC_EPI_STORE, bf16); }
        SWAP(64, TC_EPI_STORE, bf16);
    } else if (epilogue == TC_EPI_ACCUM) {
        if (bn == 32) { SWAP(32, TC_EPI_ACCUM, float); }
        SWAP(64, TC_EPI_ACCUM, float);
    } else if (epilogue == TC_EPI_SWIGLU) {
        if (c_dtype == RLLM_F32) { if (bn == 32) { SWAP(32, TC_EPI_SWIGLU, float); } SWAP(64, TC_EPI_SWIGLU, float); }
        if (bn == 32) { SWAP(32, TC_EPI_SWIGLU, bf16); }
        SWAP(64, TC_EPI_SWIGLU, bf16);
    }
#undef SWAP
    return (int)cudaErrorInvalidValue;
}

TC_DEFINE_WAIT_CONTROLS(rllm_tc)

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_gemm_tc)
RLLM_PACKED(rllm_gemm_tc_swap)
