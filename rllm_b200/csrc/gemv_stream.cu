// Weight-streaming product for decode steps, C[m,n] (+)= X[m,k] . W[n,k]^T with m <= 16, as a few
// persistent CTAs per SM fed by TMA.
//
// The product is bound by reading W once from HBM, and the matrices of one layer are small (34 to
// 200 MB): a grid of short-lived CTAs spends a good part of its time filling and draining the
// machine.  Here the grid is two or three CTAs per SM, all resident from the start.  The weight
// rows are cut into granules of 8 rows and every CTA takes an equal share of consecutive granules
// (the shares differ by at most one).  A producer thread streams the CTA's share through a ring of
// shared-memory stages with TMA: a stage is 16 KB of weights, 128 / ATOMS rows of ATOMS * 64
// k-columns (128-byte swizzle), and the same k-columns of the batch rows; the shape is chosen by
// the launcher so that a share of a few rows still fills whole stages.  Four consumer warps split
// the k16 steps of a stage, read their fragments with ldmatrix and multiply with mma.sync m16n8k16
// (float32 accumulators in registers), release the stage, and add their partial sums in warp order
// through shared memory when the K range of a chunk of rows is done, while the producer is already
// filling the ring with the next rows.  Nothing waits on another CTA; the sum over k runs in one
// fixed order, so a row's result does not depend on the batch or on the grid.
//
// With a programmatic dependent launch the kernel starts while the one before it is still running:
// the weights do not depend on that kernel, so the ring is filled with weights at once, and only
// the batch rows are loaded after griddepcontrol.wait.  The ring is sized so that the CTAs of two
// such kernels fit one SM (the running one and the next, already holding its first weights).
//
// Epilogues as in the other products: store, accumulate into a float32 C, and SwiGLU (W holds n
// gate rows and, from row up_row_offset on, n up rows; a granule is then 8 gate rows and the 8 up
// rows of the same features, so that silu(gate) * up is formed in registers).
//
// Replaces, for these sizes, the reference's matvec_bf16 / matvec_glu_silu_bf16
// (crates/rllm-cuda/src/kernels.cu, "matvec"; dispatch in crates/rllm-cuda/src/backend.rs:1697-1729).
#include "tcgen05.cuh"
#include <cuda_bf16.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

enum { SV_EPI_STORE = 0, SV_EPI_ACCUM = 1, SV_EPI_SWIGLU = 2 };
enum { SV_ERR_FULL = 1, SV_ERR_EMPTY = 2 };          // the codes of the other TMA kernels

constexpr int SV_ATOM = 64;               // k columns per TMA box: 128 bytes per row, one swizzle row
constexpr int SV_GRAN = 8;                // weight rows per granule
constexpr int SV_WARPS = 4;               // consumer warps
constexpr int SV_THREADS = (SV_WARPS + 1) * 32;
constexpr int SV_GRAN_BYTES = SV_GRAN * SV_ATOM * 2;      // 1024: 8 rows of one atom
constexpr int SV_W_BYTES = 16384;                          // weight bytes of a stage: ROWS rows x ATOMS atoms

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(SV_WARPS * 32) : "memory"); }

// Tensor maps: the weights with boxes of 64, 32, 16 and 8 rows (a chunk of the share is loaded with
// the fewest boxes that cover exactly its rows), and the batch rows.
struct SvMaps {
    CUtensorMap w[4];
    CUtensorMap x;
};

// An RMSNorm that stands between two products of a decode step, without a kernel of its own:
//
//   the product BEFORE the norm (accumulating into the float32 residual stream C) also writes, for
//   every element it produces, xw = bfloat16(c * norm_weight[column]) and adds c^2 to a sum of
//   squares per batch row; every CTA stores its sums in ssq_out[CTA][16] (fixed order inside the CTA);
//
//   the product AFTER the norm takes xw as its X operand, adds the n_parts partial sums of each batch
//   row in a fixed order, and multiplies its result rows by r = 1 / sqrt(sum / d + eps) before they
//   are stored or go through SwiGLU:  (x * w * r) . W^T  =  r * ((x * w) . W^T).
//
// The sums do not depend on the batch (a row's partials come from its own elements only).
struct SvNorm {
    // producer side (null: none)
    bf16* xw_out;
    const float* w_next;
    float* ssq_out;
    int ld_xw;
    // consumer side (null: none)
    const float* ssq_in;
    int n_parts, stride;      // parts of `stride` columns (16 from this kernel and skinny_gemm, 64 from gemm_tc_swap)
    float inv_d, eps;
};

// The share of CTA `c` of `G`: granules [first, last).
__device__ __forceinline__ void sv_share(int n_gran, int c, int G, int& first, int& last) {
    first = (int)(((long long)n_gran * c) / G);
    last = (int)(((long long)n_gran * (c + 1)) / G);
}

// NT: batch rows / 8 (1 or 2).  ATOMS (2, 4 or 8): boxes of 64 k-columns side by side in a stage;
// a stage holds 128 / ATOMS weight rows of ATOMS * 64 k-columns, 16 KB whatever the shape, so that
// a CTA whose share is a few rows still has whole stages in flight.  The rows of a stage are
// "slots" of 16.  Without SwiGLU a slot is two consecutive granules; with SwiGLU a slot is one
// granule of 8 features, rows 0-7 its gate rows (first half of each atom), rows 8-15 its up rows
// (second half).  The four consumer warps split the k16 steps of an atom (warp w takes step w of
// every atom) and every warp works on all slots, so that the warps are busy whatever the number of
// rows; at the end of a chunk the four partial sums of a slot are added in warp order through
// shared memory by the warp of that number, which writes the slot's rows.
template <int NT, int EPI, typename TC, int ATOMS, int STAGES>
__global__ void __launch_bounds__(SV_THREADS)
gemv_stream_kernel(const __grid_constant__ SvMaps maps, TC* __restrict__ C, int ldc, int m, int n, int K,
                   int up_row_offset, int* err, const SvNorm nm) {
    constexpr int ROWS = 128 / ATOMS;
    constexpr int SLOTS = ROWS / 16;
    constexpr int BK = ATOMS * SV_ATOM;
    constexpr int WATOM_BYTES = ROWS * 128;
    constexpr int XATOM_BYTES = NT * SV_GRAN_BYTES;
    constexpr int STAGE_BYTES = SV_W_BYTES + ATOMS * XATOM_BYTES;
    constexpr int HALVES = (EPI == SV_EPI_SWIGLU) ? 2 : 1;
    constexpr int GRAN_PER_CHUNK = ROWS / (SV_GRAN * HALVES);
    constexpr int RED_FLOATS = SV_WARPS * SLOTS * NT * 32 * 4;          // [source warp][slot][j][lane][4]
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* red = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);     // two buffers
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ volatile int abort_flag;
    __shared__ float norm_red[8][16];         // partial sums of squares: [segment or warp][batch row]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_gran = (n + SV_GRAN - 1) / SV_GRAN;
    int g_first, g_last;
    sv_share(n_gran, blockIdx.x, gridDim.x, g_first, g_last);
    const int nkb = (K + BK - 1) / BK;
    const int n_chunks = (g_last - g_first + GRAN_PER_CHUNK - 1) / GRAN_PER_CHUNK;
    const int total = n_chunks * nkb;                     // stages this CTA streams

    // Every thread signals at once that the next kernel of the stream may be scheduled: all CTAs of
    // this grid are resident from the start, so the next kernel takes nothing from this one; it
    // comes to rest beside it (a ring of three stages is about 60 KB, so the CTAs of two grids fit
    // the SM's shared memory) with its first weights in flight, and waits in its own griddepcontrol.wait for this grid to complete.
    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.w[i]) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.x) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], SV_WARPS); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == SV_WARPS) {
        // ---- TMA producer (one thread).  A copy costs about 70 ns whatever its size, so a stage is
        // fetched with as few copies as possible: three-dimensional boxes (64 k-columns, rows, ATOMS atoms)
        // that arrive as [atom][row][128 bytes]; one per power of two in the chunk's granule count
        // (one in all for a whole chunk), twice that with SwiGLU, and one for the batch rows.
        auto issue_w = [&](int it) {
            const int s = it % STAGES, chunk = it / nkb, kb = it - chunk * nkb;
            const int g0 = g_first + chunk * GRAN_PER_CHUNK;
            const int ng = min(GRAN_PER_CHUNK, g_last - g0);
            unsigned char* st = smem + (size_t)s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], ATOMS * (HALVES * ng * SV_GRAN_BYTES + XATOM_BYTES));
#pragma unroll
            for (int half = 0; half < HALVES; ++half) {
                int done = 0;
#pragma unroll
                for (int lvl = 0; lvl < 4; ++lvl) {
                    const int gr = 8 >> lvl;
                    if (gr <= GRAN_PER_CHUNK && (ng & gr)) {
                        tma_load_3d(st + half * (SV_W_BYTES / 2) + ATOMS * done * SV_GRAN_BYTES, &maps.w[lvl], 0,
                                    (half ? up_row_offset : 0) + (g0 + done) * SV_GRAN, kb * ATOMS, &full_bar[s]);
                        done += gr;
                    }
                }
            }
        };
        auto issue_x = [&](int it) {
            const int s = it % STAGES, kb = it % nkb;
            tma_load_3d(smem + (size_t)s * STAGE_BYTES + SV_W_BYTES, &maps.x, 0, 0, kb * ATOMS, &full_bar[s]);
        };
        if (lane != 0) return;
        const int head = min(STAGES, total);
        for (int it = 0; it < head; ++it) issue_w(it);       // weights: no dependence on the kernel before
        pdl_wait();
        for (int it = 0; it < head; ++it) issue_x(it);
        int issued = head;
        for (int it = head; it < total; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, SV_ERR_EMPTY); abort_flag = 1; }
                break;
            }
            issue_w(it);
            issue_x(it);
            issued = it + 1;
        }
        if (abort_flag) {
            // the copies in flight still write into this CTA's shared memory: wait for them (bounded)
            for (int it = max(0, issued - STAGES); it < issued; ++it) {
                volatile int no_abort = 0;
                mbar_wait(&full_bar[it % STAGES], (it / STAGES) & 1, &no_abort);
            }
        }
        return;
    }

    // ---- consumers
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix x4 of an A fragment (16 rows x 16 k): lane l gives the row address of matrix l>>3:
    // matrices 0/1 are rows 0-7 / 8-15 of k 0-7, matrices 2/3 the same rows of k 8-15.
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;          // row within the slot's 16
    const int a_chunk = ((2 * warp + (lane >> 4)) ^ (a_row & 7)) << 4;       // swizzled 16-byte chunk of this warp's k16 step
    const uint32_t a_off = (EPI == SV_EPI_SWIGLU)
        ? (uint32_t)((a_row >> 3) * (SV_W_BYTES / 2) + (a_row & 7) * 128 + a_chunk)
        : (uint32_t)(a_row * 128 + a_chunk);
    // ldmatrix x2 of the B fragment (8 batch rows x 16 k): lanes 0-15 give the addresses
    const int b_row = lane & 7;
    const uint32_t b_off = (uint32_t)(b_row * 128 + (((2 * warp + ((lane >> 3) & 1)) ^ b_row) << 4));

    // The rows' 1/rms for a deferred norm: thread (segment = tid / 16, b = tid % 16) adds every eighth
    // partial sum of batch row b into shared memory here, while the first stages arrive; the eight
    // segment sums are added in order at the end of the first chunk, behind that chunk's barrier.
    float rscale[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) rscale[j][0] = rscale[j][1] = 1.f;
    bool waited = false, scaled = nm.ssq_in == nullptr;
    if (nm.ssq_in) {
        pdl_wait();                       // the sums come from the kernel before
        waited = true;
        const int b = tid & 15, seg = tid >> 4;
        float ssum = 0.f;
        // eight loads in flight at a time, added in the order of the parts (one after the other, each
        // load would wait for the round trip of the one before)
        for (int p0 = seg; p0 < nm.n_parts; p0 += 64) {
            float f[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int p = p0 + 8 * u;
                f[u] = p < nm.n_parts ? __ldcg(nm.ssq_in + (size_t)p * nm.stride + b) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) ssum += f[u];
        }
        norm_red[seg][b] = ssum;
    }
    float ssq[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) ssq[j][0] = ssq[j][1] = 0.f;

    float acc[SLOTS][NT][4];
    int it = 0;
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        const int g0 = g_first + chunk * GRAN_PER_CHUNK;
        const int ng = min(GRAN_PER_CHUNK, g_last - g0);
        const int n_slots = (EPI == SV_EPI_SWIGLU) ? ng : (ng + 1) >> 1;
        // where slot sl lies in a stage: the chunk's boxes follow one another, largest first, each as
        // [atom][rows of the box]; a slot lies in one box (an odd last granule is a box of its own)
        uint32_t slot_off[SLOTS], slot_astride[SLOTS];
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl) {
            const int q = (EPI == SV_EPI_SWIGLU) ? sl : 2 * sl;       // first granule of the slot
            int done = 0;
            slot_off[sl] = 0;
            slot_astride[sl] = SV_GRAN_BYTES;
#pragma unroll
            for (int lvl = 0; lvl < 4; ++lvl) {
                const int gr = 8 >> lvl;
                if (gr <= GRAN_PER_CHUNK && (ng & gr)) {
                    if (q >= done && q < done + gr) {
                        slot_off[sl] = (uint32_t)(ATOMS * done * SV_GRAN_BYTES + (q - done) * SV_GRAN_BYTES);
                        slot_astride[sl] = (uint32_t)(gr * SV_GRAN_BYTES);
                    }
                    done += gr;
                }
            }
        }
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[sl][j][e] = 0.f;
        // Accumulating: the old values of the rows this thread will write are fetched now and arrive
        // while the chunk streams (read at the chunk's end they cost a round trip to L2 each, one
        // after the other, at the end of the kernel).
        float c_old[NT][4];
        float wn[2] = {0.f, 0.f};         // norm weights of this thread's two rows (deferred norm)
        if (EPI == SV_EPI_ACCUM) {
            if (!waited) { pdl_wait(); waited = true; }      // C belongs to the kernels before until here
            if (warp < n_slots) {
                const int row_end = min(n, g_last * SV_GRAN);
                const int r_lo = (g0 + 2 * warp) * SV_GRAN + g;
                if (nm.w_next) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) wn[h] = r_lo + 8 * h < row_end ? nm.w_next[r_lo + 8 * h] : 0.f;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int b = 8 * j + 2 * t + e, row = r_lo + 8 * h;
                            c_old[j][2 * h + e] = (row < row_end && b < m) ? to_f<TC>(C[(size_t)b * ldc + row]) : 0.f;
                        }
            }
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&full_bar[s], ph, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, SV_ERR_FULL); abort_flag = 1; }
                break;
            }
            const uint32_t st = s_addr(smem + (size_t)s * STAGE_BYTES);
            const uint32_t xs = st + SV_W_BYTES;
#pragma unroll
            for (int at = 0; at < ATOMS; ++at) {
                uint32_t b[NT][2];
#pragma unroll
                for (int j = 0; j < NT; ++j) ldsm_x2(xs + at * XATOM_BYTES + j * SV_GRAN_BYTES + b_off, b[j][0], b[j][1]);
#pragma unroll
                for (int sl = 0; sl < SLOTS; ++sl) {
                    if (sl < n_slots) {
                        uint32_t a0, a1, a2, a3;
                        ldsm_x4(st + slot_off[sl] + at * slot_astride[sl] + a_off, a0, a1, a2, a3);
#pragma unroll
                        for (int j = 0; j < NT; ++j) mma_16816(acc[sl][j], a0, a1, a2, a3, b[j][0], b[j][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
        }
        // the four warps' partial sums of each slot -> shared memory, added in warp order
        float* buf = red + (chunk & 1) * RED_FLOATS;
#pragma unroll
        for (int sl = 0; sl < SLOTS; ++sl)
#pragma unroll
            for (int j = 0; j < NT; ++j)
                *reinterpret_cast<float4*>(buf + ((((size_t)warp * SLOTS + sl) * NT + j) * 32 + lane) * 4) =
                    make_float4(acc[sl][j][0], acc[sl][j][1], acc[sl][j][2], acc[sl][j][3]);
        consumer_sync();               // every consumer warp comes here, also after a wait that ran out
        if (abort_flag) break;
        if (!scaled) {
            scaled = true;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float tot = 0.f;
#pragma unroll
                    for (int sg = 0; sg < 8; ++sg) tot += norm_red[sg][8 * j + 2 * t + e];
                    rscale[j][e] = 1.0f / sqrtf(tot * nm.inv_d + nm.eps);
                }
        }
        if (warp >= n_slots) continue;
        float v[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int src = 0; src < SV_WARPS; ++src) {
                const float4 p = *reinterpret_cast<const float4*>(buf + ((((size_t)src * SLOTS + warp) * NT + j) * 32 + lane) * 4);
                sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
            }
            v[j][0] = sum.x * rscale[j][0]; v[j][1] = sum.y * rscale[j][1];
            v[j][2] = sum.z * rscale[j][0]; v[j][3] = sum.w * rscale[j][1];
        }
        if (!waited) { pdl_wait(); waited = true; }      // C belongs to the kernels before until here
        // rows of this lane in slot `warp`: row g (sums 0, 1) and row g + 8 (sums 2, 3); batch columns 8j + 2t, + 1
        const int row_end = min(n, g_last * SV_GRAN);
        if (EPI == SV_EPI_SWIGLU) {
            const int f = (g0 + warp) * SV_GRAN + g;
            if (f < row_end) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int b = 8 * j + 2 * t + e;
                        if (b < m) {
                            const float gate = v[j][e], up = v[j][2 + e];
                            C[(size_t)b * ldc + f] = from_f<TC>(gate / (1.0f + expf(-gate)) * up);
                        }
                    }
            }
        } else {
            const int r_lo = (g0 + 2 * warp) * SV_GRAN + g;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = r_lo + 8 * h;
                if (row >= row_end) continue;
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int b = 8 * j + 2 * t + e;
                        if (b < m) {
                            TC* c = C + (size_t)b * ldc + row;
                            const float val = v[j][2 * h + e];
                            if (EPI == SV_EPI_ACCUM) {
                                const float sum = c_old[j][2 * h + e] + val;
                                *c = from_f<TC>(sum);
                                if (nm.xw_out) {
                                    nm.xw_out[(size_t)b * nm.ld_xw + row] = from_f<bf16>(sum * wn[h]);
                                    ssq[j][e] += sum * sum;
                                }
                            } else *c = from_f<TC>(val);
                        }
                    }
            }
        }
    }
    if (EPI == SV_EPI_ACCUM && nm.ssq_out) {
        // this thread's sums -> the 8 lanes with equal t -> the four warps, in warp order
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float sq = ssq[j][e];
                sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                sq += __shfl_xor_sync(0xffffffffu, sq, 16);
                if (g == 0) norm_red[warp][8 * j + 2 * t + e] = sq;
                else if (NT == 1 && g == 1) norm_red[warp][8 + 2 * t + e] = 0.f;
            }
        consumer_sync();
        if (tid < 16) {
            if (!waited) pdl_wait();
            nm.ssq_out[(size_t)blockIdx.x * 16 + tid] =
                norm_red[0][tid] + norm_red[1][tid] + norm_red[2][tid] + norm_red[3][tid];
        }
    }
}

// Three-dimensional view of a row-major [rows, cols] bfloat16 matrix: (64 columns of an atom, rows,
// atoms), box (64, box_rows, atoms).
static int sv_tmap(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows, int atoms) {
    cuuint64_t dims[3] = {SV_ATOM, (cuuint64_t)rows, (cuuint64_t)(cols / SV_ATOM)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, SV_ATOM * 2};
    cuuint32_t box[3] = {SV_ATOM, (cuuint32_t)box_rows, (cuuint32_t)atoms};
    return tmap_encode_bf16(map, base, 3, dims, strides, box);
}

struct SvProblem {
    const void *W, *X;
    void* C;
    int m, n, K, ldw, ldx, ldc, up, grid, nt, w_rows, stages;
    int* err;
    SvNorm nm;
};

template <int NT, int EPI, typename TC, int ATOMS, int STAGES>
static int launch_sv_stages(const SvMaps& maps, void* C, int ldc, int m, int n, int K, int up, int grid, int* err,
                            const SvNorm& nm, cudaStream_t stream) {
    constexpr int SLOTS = 128 / ATOMS / 16;
    constexpr size_t smem = (size_t)STAGES * (SV_W_BYTES + ATOMS * NT * SV_GRAN_BYTES) +
                            2 * (SV_WARPS * SLOTS * NT * 32 * 4) * sizeof(float) + 1024;
    auto kern = gemv_stream_kernel<NT, EPI, TC, ATOMS, STAGES>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    return rllm_launch(kern, dim3(grid), dim3(SV_THREADS), smem, stream, maps, (TC*)C, ldc, m, n, K, up, err, nm);
}

template <int NT, int EPI, typename TC, int ATOMS>
static int launch_sv_atoms(const SvProblem& p, cudaStream_t stream) {
    SvMaps maps;
    for (int lvl = 0; lvl < 4; ++lvl) {
        int st = sv_tmap(&maps.w[lvl], p.W, p.w_rows, p.K, p.ldw, (8 >> lvl) * SV_GRAN, ATOMS);
        if (st) return st;
    }
    int st = sv_tmap(&maps.x, p.X, p.m, p.K, p.ldx, 8 * NT, ATOMS);
    if (st) return st;
    if (p.stages == 10 && ATOMS * NT <= 4)           // ten stages of the widest shapes do not fit; they get five
        return launch_sv_stages<NT, EPI, TC, ATOMS, 10>(maps, p.C, p.ldc, p.m, p.n, p.K, p.up, p.grid, p.err, p.nm, stream);
    if (p.stages == 3)
        return launch_sv_stages<NT, EPI, TC, ATOMS, 3>(maps, p.C, p.ldc, p.m, p.n, p.K, p.up, p.grid, p.err, p.nm, stream);
    return launch_sv_stages<NT, EPI, TC, ATOMS, 5>(maps, p.C, p.ldc, p.m, p.n, p.K, p.up, p.grid, p.err, p.nm, stream);
}

// The stage shape follows the share of a CTA: few rows, more k-columns per stage.
template <int NT, int EPI, typename TC>
static int launch_sv(const SvProblem& p, cudaStream_t stream) {
    const int n_gran = (p.n + SV_GRAN - 1) / SV_GRAN;
    const int share = (n_gran + p.grid - 1) / p.grid * (EPI == SV_EPI_SWIGLU ? 2 : 1);   // granule boxes of the largest share
    if (share <= 2) return launch_sv_atoms<NT, EPI, TC, 8>(p, stream);
    if (share <= 4) return launch_sv_atoms<NT, EPI, TC, 4>(p, stream);
    return launch_sv_atoms<NT, EPI, TC, 2>(p, stream);
}

// C[m,n] (+)= X[m,k] . W[n,k]^T for m <= 16.  epilogue: 0 store, 1 accumulate into float32 C,
// 2 SwiGLU (W holds n gate rows and, from row up_row_offset on, n up rows; C is [m, n]).
// grid: number of CTAs (0: one per SM).  stages: depth of the ring, 3, 5 or 10 stages of 18 to 24 KB
// (3 CTAs of 3 stages, or 2 of 5, fit one SM; 10 falls back to 5 where it does not fit).  Requires k % 64 == 0, ldw % 8 == 0, ldx % 8 == 0 and
// 16-byte aligned W and X; returns cudaErrorInvalidValue otherwise.  err: device int that receives
// a code when a bounded wait runs out.
// Deferred norm (see SvNorm), both optional.  Producing side, accumulate epilogue only: xw_out [m, ld_xw]
// bfloat16, w_next [n] float32, ssq_out [CTAs of this launch][16] float32 (the launcher returns the
// number of CTAs in *n_parts_out).  Consuming side, store and SwiGLU epilogues: ssq_in [n_parts_in][16],
// norm_d the row length the sums run over, norm_eps.
RLLM_API int rllm_gemv_stream(const void* W, const void* X, void* C, int c_dtype, int m, int n, int K, int ldw,
                              int ldx, int ldc, int epilogue, int up_row_offset, int grid, int stages, int* err,
                              void* xw_out, int ld_xw, const float* w_next, float* ssq_out, int* n_parts_out,
                              const float* ssq_in, int n_parts_in, int ssq_stride_in, int norm_d, float norm_eps,
                              cudaStream_t stream) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 16 || K <= 0 || (K % SV_ATOM) || (ldw & 7) || (ldx & 7) || ((uintptr_t)W & 15) || ((uintptr_t)X & 15) ||
        !err || grid < 0 || (stages != 3 && stages != 5 && stages != 10))
        return (int)cudaErrorInvalidValue;
    if (epilogue == SV_EPI_ACCUM && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    if (grid == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&grid, cudaDevAttrMultiProcessorCount, dev);
    }
    const int n_gran = (n + SV_GRAN - 1) / SV_GRAN;
    if (grid > n_gran) grid = n_gran;
    SvProblem p;
    p.W = W; p.X = X; p.C = C; p.m = m; p.n = n; p.K = K; p.ldw = ldw; p.ldx = ldx; p.ldc = ldc;
    p.up = up_row_offset; p.grid = grid; p.stages = stages; p.nt = m <= 8 ? 1 : 2; p.err = err;
    p.w_rows = epilogue == SV_EPI_SWIGLU ? up_row_offset + n : n;
    p.nm = SvNorm{};
    if (xw_out || ssq_out || w_next) {
        if (epilogue != SV_EPI_ACCUM || !xw_out || !ssq_out || !w_next) return (int)cudaErrorInvalidValue;
        p.nm.xw_out = (bf16*)xw_out; p.nm.w_next = w_next; p.nm.ssq_out = ssq_out; p.nm.ld_xw = ld_xw;
        if (n_parts_out) *n_parts_out = grid;
    }
    if (ssq_in) {
        if (epilogue == SV_EPI_ACCUM || n_parts_in <= 0 || norm_d <= 0 || ssq_stride_in < 16) return (int)cudaErrorInvalidValue;
        p.nm.ssq_in = ssq_in; p.nm.n_parts = n_parts_in; p.nm.stride = ssq_stride_in; p.nm.inv_d = 1.0f / (float)norm_d;
        p.nm.eps = norm_eps;
    }
    const int nt = p.nt;
#define SV(NT_, EPI_, TC_) return launch_sv<NT_, EPI_, TC_>(p, stream)
    if (epilogue == SV_EPI_STORE) {
        if (c_dtype == RLLM_F32) { if (nt == 1) { SV(1, SV_EPI_STORE, float); } SV(2, SV_EPI_STORE, float); }
        if (nt == 1) { SV(1, SV_EPI_STORE, bf16); }
        SV(2, SV_EPI_STORE, bf16);
    } else if (epilogue == SV_EPI_ACCUM) {
        if (nt == 1) { SV(1, SV_EPI_ACCUM, float); }
        SV(2, SV_EPI_ACCUM, float);
    } else if (epilogue == SV_EPI_SWIGLU) {
        if (c_dtype == RLLM_F32) { if (nt == 1) { SV(1, SV_EPI_SWIGLU, float); } SV(2, SV_EPI_SWIGLU, float); }
        if (nt == 1) { SV(1, SV_EPI_SWIGLU, bf16); }
        SV(2, SV_EPI_SWIGLU, bf16);
    }
#undef SV
    return (int)cudaErrorInvalidValue;
}

TC_DEFINE_WAIT_CONTROLS(rllm_stream)

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_gemv_stream)
