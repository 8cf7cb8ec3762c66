// The many-row tcgen05 product with two SMs on one tile (tcgen05.mma.cta_group::2): a pair of CTAs
// (a thread-block cluster of two) computes a 256 x 256 tile of D[M,N] = A[M,K] . B[N,K]^T.  Each CTA
// stages its own 128 rows of A and its own half of the B tile (128 of the 256 rows of B) per block
// of 64 along K, and holds the accumulator of its own 128 rows of D (all 256 columns) in its tensor
// memory; the MMA, issued by one thread of the pair's first CTA (the leader), reads A from each SM's
// own shared memory and B from both.  Per 128 x 256 x 64 of multiply-adds a CTA thus fills 32 KB of
// shared memory where the one-CTA kernel (gemm_tc.cu) fills 48 KB.  A stage holds 128 elements
// along K (two swizzled tiles of 64 per operand): eight MMAs per barrier round and commit, where
// four left the issuing thread as busy as the tensor pipe (2,048 x 24,576 x 4,096 with SwiGLU: 291 us
// with stages of 64, as the one-CTA kernel; 270 us with stages of 128).
//
//   * persistent pairs (one per two SMs) walk over the tiles; a ring of stages per CTA; two
//     accumulator buffers in TMEM (2 x 256 columns) so that a tile's epilogue overlaps the next
//     tile's MMAs;
//   * warp 0 of each CTA (one lane) issues its TMA loads; every load of the pair completes bytes on
//     the LEADER's "full" mbarrier of the stage (cp.async.bulk.tensor with .cta_group::2 may signal
//     a barrier of the peer CTA); the leader's producer arms that barrier with the pair's byte count;
//   * warp 1 of the leader (one lane) issues the MMAs and commits with
//     tcgen05.commit.cta_group::2 ... .multicast::cluster: the arrival lands on the barrier at the
//     same offset in both CTAs ("empty" per stage, "accumulator full" per buffer);
//   * warps 2..5 of each CTA are its epilogue (as in gemm_tc.cu); one lane per warp reports the
//     buffer free on the leader's "accumulator empty" barrier (a remote arrive for the peer).
//   SwiGLU: the leader's half of B holds 128 gate rows, the peer's the 128 up rows of the same
//   index, so that a thread finds gate and up of an output column in its own accumulator row.
//
// A fourth epilogue (T2_EPI_QKV) ends the fused q/k/v projection of a prompt step: a thread owns a
// token's row of the tile, 256 columns = whole heads (head size 64 or 128), and does for each head
// what qk_norm_rope_store (elementwise.cu) does in a kernel of its own: RMSNorm over the head with
// the q or k norm weight, rotate-half rotary with the (cos, sin) of the token's angles, queries out
// as bfloat16, keys and values into their page of the cache.  The float32 projection never goes
// to memory.
//
// The last, partial wave: when the tiles left over after the full waves would keep at most half (a
// quarter) of the pairs busy, each of them is cut into two (four) slices of columns (MMAs of N = 128
// or 64), so that the wave takes half (a quarter) of a tile's time; a product with fewer tiles than
// pairs is cut the same way.  A work item is a tile or a slice of one.
//
// No TMA load is multicast.  Every wait on an mbarrier is bounded (tcgen05.cuh); the two barriers
// that have no limit are the cluster barriers at the start and the end, which every thread of both
// CTAs reaches whatever happened between them.
#include "tcgen05.cuh"
#include <math.h>

#define T2_BM 128            // rows of A per CTA (256 per pair)
#define T2_BN 256            // columns of the accumulator
#define T2_BK 64
#define T2_THREADS 192
#define T2_HALF_BYTES (128 * T2_BK * 2)          // one [128 x 64] operand tile: 16 KB
#define T2_KH 2                                  // blocks of 64 along K per stage (one barrier round, 4 * T2_KH MMAs)
#define T2_STAGE_BYTES (2 * T2_KH * T2_HALF_BYTES)   // per CTA: T2_KH A tiles, then T2_KH tiles of its half of B

enum { T2_EPI_STORE = 0, T2_EPI_ACCUM = 1, T2_EPI_SWIGLU = 2, T2_EPI_QKV = 3 };
enum { T2_ERR_FULL = 1, T2_ERR_EMPTY = 2, T2_ERR_ACC = 3 };

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of `p` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(s_addr(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose bytes complete on a barrier given by its cluster address (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(s_addr(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t z = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
}
// the arrival lands on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(s_addr(bar)), "h"(both) : "memory");
}

template <typename TC> __device__ __forceinline__ void t2_store_row32(TC* dst, const float (&v)[32], int n_valid);
template <> __device__ __forceinline__ void t2_store_row32<float>(float* dst, const float (&v)[32], int n_valid) {
    if (n_valid >= 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (j < n_valid) dst[j] = v[j];
    }
}
template <> __device__ __forceinline__ void t2_store_row32<bf16>(bf16* dst, const float (&v)[32], int n_valid) {
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

struct T2Qkv {
    bf16* q_out;                 // [M, H * hd]
    bf16* k_cache;               // [pages, K, bs, hd]
    bf16* v_cache;
    const int* slots;            // [M]: page * bs + offset of the token's place, < 0: keep nothing
    const float2* cs_table;      // [M, hd / 2] (cos, sin), null: no rotation
    const float* q_norm_w;       // [hd], null: no norm
    const float* k_norm_w;
    int H, K, bs, write_kv, n_slots;
    float eps;
};

struct T2Maps {
    CUtensorMap a;          // boxes of 64 x 128 rows
    CUtensorMap b[3];       // boxes of 64 x 128, 64 and 32 rows: a CTA's half of a whole, half and quarter B tile
};

// Work item -> (tile, slice, log2 of the slices its tile is cut into): the first `head` items are
// whole tiles, the others the slices of the `tail` tiles behind them.
__device__ __forceinline__ void t2_item(int item, int head, int tail_log2, int& tile, int& slice, int& sl_log2) {
    if (item < head) { tile = item; slice = 0; sl_log2 = 0; return; }
    const int j = item - head;
    tile = head + (j >> tail_log2);
    slice = j & ((1 << tail_log2) - 1);
    sl_log2 = tail_log2;
}

// grid (2 * pairs), clusters of two along x (a kernel with cta_group::2 instructions is refused with
// "invalid cluster size" when its clusters are not even along x): CTAs 2p and 2p + 1 are pair p,
// which takes tiles p, p + pairs, ... (m fastest, as in gemm_tc.cu).
template <int EPI, typename TC, int STAGES, int HD = 128>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ T2Maps maps, TC* __restrict__ C, int ldc, int M, int N, int K,
                int up_row_offset, int* __restrict__ err, int tail_tiles, int tail_log2, const T2Qkv qk) {
    constexpr int BN_OUT = (EPI == T2_EPI_SWIGLU) ? T2_BN / 2 : T2_BN;      // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES];      // used in the leader: bytes of both CTAs
    __shared__ __align__(8) uint64_t empty_bar[STAGES];     // in each CTA: the MMAs have read the stage
    __shared__ __align__(8) uint64_t acc_full[2];           // in each CTA: the accumulator buffer is complete
    __shared__ __align__(8) uint64_t acc_empty[2];          // used in the leader: both epilogues have read the buffer
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();                   // 0: the leader
    const int nkb = (K + T2_KH * T2_BK - 1) / (T2_KH * T2_BK);      // stages along K
    const int m_tiles = (M + 2 * T2_BM - 1) / (2 * T2_BM), n_tiles = (N + BN_OUT - 1) / BN_OUT;
    const int total_tiles = m_tiles * n_tiles;
    const int head = total_tiles - tail_tiles;                   // whole tiles; then the slices of the others
    const int total_items = head + (tail_tiles << tail_log2);
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.b[0]) : "memory");
        if (tail_tiles) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.b[tail_log2]) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 warps of 2 CTAs
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(&tmem_base_slot, 2 * T2_BN);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                            // the peer's barriers exist before anything arrives at them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_wait();                                    // the A operand is written by the kernel before

    if (warp == 0 && lane == 0) {
        // ---- TMA producer of this CTA: its rows of A and its half of B, bytes counted by the leader
        int it = 0, issued = 0;
        bool ok = true;
        for (int item = pair; item < total_items && ok; item += n_pairs) {
            int tile, slice, sl;
            t2_item(item, head, tail_log2, tile, slice, sl);
            const int m0 = (tile % m_tiles) * (2 * T2_BM) + (int)rank * T2_BM;
            const int n0 = (tile / m_tiles) * BN_OUT + slice * (BN_OUT >> sl);      // first output column of the item
            const int b_row = (EPI == T2_EPI_SWIGLU) ? (rank == 0 ? n0 : up_row_offset + n0) : n0 + (int)rank * (128 >> sl);
            const uint32_t stage_tx = 2 * T2_KH * (T2_HALF_BYTES + (T2_HALF_BYTES >> sl));     // both CTAs' bytes
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag)) {
                    if (!abort_flag) { atomicExch(err, T2_ERR_EMPTY); abort_flag = 1; }
                    ok = false;
                    break;
                }
                unsigned char* a_s = smem + (size_t)s * T2_STAGE_BYTES;
                const uint32_t full = cluster_addr(&full_bar[s], 0);
                if (rank == 0) mbar_expect_tx(&full_bar[s], stage_tx);
#pragma unroll
                for (int h = 0; h < T2_KH; ++h) {
                    tma_load_2d_pair(a_s + h * T2_HALF_BYTES, &maps.a, (kb * T2_KH + h) * T2_BK, m0, full);
                    tma_load_2d_pair(a_s + (T2_KH + h) * T2_HALF_BYTES, &maps.b[sl], (kb * T2_KH + h) * T2_BK, b_row, full);
                }
                issued = it + 1;
            }
        }
        if (abort_flag && rank == 0) {
            // copies already issued must land before the shared memory goes away (the peer's land in its
            // own shared memory; both CTAs stay until the cluster barrier at the end)
            volatile int no_abort = 0;
            for (int i = max(0, issued - STAGES); i < issued; ++i)
                mbar_wait(&full_bar[i % STAGES], (i / STAGES) & 1, &no_abort);
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer of the pair
        int it = 0, local = 0;
        bool ok = true;
        for (int item = pair; item < total_items && ok; item += n_pairs, ++local) {
            const int buf = local & 1;
            const uint32_t idesc = idesc_bf16(2 * T2_BM, T2_BN >> (item < head ? 0 : tail_log2));
            if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, &abort_flag)) {
                if (!abort_flag) { atomicExch(err, T2_ERR_ACC); abort_flag = 1; }
                break;
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * T2_BN;
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph, &abort_flag)) {
                    if (!abort_flag) { atomicExch(err, T2_ERR_FULL); abort_flag = 1; }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = s_addr(smem + (size_t)s * T2_STAGE_BYTES);
#pragma unroll
                for (int h = 0; h < T2_KH; ++h) {
                    const uint64_t a_desc = smem_desc_sw128(a_addr + h * T2_HALF_BYTES);
                    const uint64_t b_desc = smem_desc_sw128(a_addr + (T2_KH + h) * T2_HALF_BYTES);
#pragma unroll
                    for (int kk = 0; kk < T2_BK / 16; ++kk)
                        umma_bf16_pair(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb | h | kk) != 0);
                }
                umma_commit_pair(&empty_bar[s]);
            }
            if (ok) umma_commit_pair(&acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---- epilogue of this CTA's 128 rows: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        int local = 0;
        bool first = true;
        for (int item = pair; item < total_items; item += n_pairs, ++local) {
            const int buf = local & 1;
            int tile, slice, sl;
            t2_item(item, head, tail_log2, tile, slice, sl);
            const int cols_out = BN_OUT >> sl;                     // output columns of the item (at least 32)
            const int m0 = (tile % m_tiles) * (2 * T2_BM) + (int)rank * T2_BM;
            const int n0 = (tile / m_tiles) * BN_OUT + slice * cols_out;
            const int gm = m0 + row;
            bool ok = mbar_wait(&acc_full[buf], (local >> 1) & 1, &abort_flag);
            if (!ok && !abort_flag) { atomicExch(err, T2_ERR_ACC); abort_flag = 1; }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (first && item + n_pairs >= total_items) { pdl_launch_dependents(); first = false; }
            const uint32_t taddr = tmem_base + buf * T2_BN + ((uint32_t)(quarter * 32) << 16);
            if constexpr (EPI == T2_EPI_QKV) {
                // this thread's token: its place in the cache and its angles
                const bool row_ok = gm < M;
                int slot = row_ok ? qk.slots[gm] : -1;
                if (slot >= qk.n_slots) {
                    atomicExch(err, RLLM_ERR_SLOT);
                    slot = -1;
                }
                const float2* cs = (qk.cs_table && row_ok) ? qk.cs_table + (size_t)gm * (HD / 2) : nullptr;
#pragma unroll 1
                for (int hh = 0; hh < cols_out / HD; ++hh) {
                    const int head = n0 / HD + hh;
                    float v[HD];
#pragma unroll
                    for (int c = 0; c < HD / 32; ++c)
                        tmem_ld32(taddr + hh * HD + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(&v[32 * c]));
                    tmem_ld_wait();
                    if (hh == cols_out / HD - 1) {               // all of this warp's TMEM reads of the item are done
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
                    }
                    if (!row_ok || head >= qk.H + 2 * qk.K) continue;
                    const int kind = head < qk.H ? 0 : (head < qk.H + qk.K ? 1 : 2);
                    bf16* dst = nullptr;
                    if (kind == 0) {
                        dst = qk.q_out + ((size_t)gm * qk.H + head) * HD;
                    } else if (slot >= 0 && qk.write_kv) {
                        const int kvh = kind == 1 ? head - qk.H : head - qk.H - qk.K;
                        dst = (kind == 1 ? qk.k_cache : qk.v_cache) +
                              (((size_t)(slot / qk.bs) * qk.K + kvh) * qk.bs + (slot % qk.bs)) * HD;
                    }
                    if (!dst) continue;
                    const float* nw = kind == 0 ? qk.q_norm_w : (kind == 1 ? qk.k_norm_w : nullptr);
                    float rs = 1.f;
                    if (nw) {
                        float ss = 0.f;
#pragma unroll
                        for (int i = 0; i < HD; ++i) ss += v[i] * v[i];
                        rs = 1.0f / sqrtf(ss / (float)HD + qk.eps);
                    }
#pragma unroll
                    for (int i = 0; i < HD / 2; i += 2) {
                        float4 c4 = make_float4(1.f, 0.f, 1.f, 0.f);
                        if (cs && kind != 2) c4 = *reinterpret_cast<const float4*>(cs + i);      // two (cos, sin) pairs
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            float a = v[i + e], b = v[i + e + HD / 2];
                            if (nw) { a = a * rs * __ldg(nw + i + e); b = b * rs * __ldg(nw + i + e + HD / 2); }
                            if (kind != 2) {
                                const float cx = e ? c4.z : c4.x, cy = e ? c4.w : c4.y;
                                const float a2 = a * cx - b * cy, b2 = a * cy + b * cx;
                                a = a2; b = b2;
                            }
                            v[i + e] = a; v[i + e + HD / 2] = b;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < HD / 8; ++j) {
                        uint4 u;
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                        u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
                        u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
                        reinterpret_cast<uint4*>(dst)[j] = u;
                    }
                }
            } else {
#pragma unroll 1
            for (int c0 = 0; c0 < cols_out; c0 += 32) {
                uint32_t r[32];
                float v[32];
                tmem_ld32(taddr + c0, r);
                if (EPI == T2_EPI_SWIGLU) {
                    uint32_t u[32];
                    tmem_ld32(taddr + cols_out + c0, u);          // the up columns follow the item's gate columns
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
                if (c0 + 32 >= cols_out) {                   // all of this warp's TMEM reads of the item are done
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
                }
                const int gn = n0 + c0;
                if (gm < M && gn < N) {
                    TC* dst = C + (size_t)gm * ldc + gn;
                    const int n_valid = min(32, N - gn);
                    if (EPI == T2_EPI_ACCUM) {
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
                    t2_store_row32<TC>(dst, v, n_valid);
                }
            }
            }
        }
    }
    __syncwarp();          // the lanes that had no role meet the elected one: the barriers below want whole warps
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();    // the leader's MMAs read the peer's shared memory and arrive at its barriers: leave together
    if (warp == 1) tmem_dealloc_pair(tmem_base, 2 * T2_BN);
}

// ---------------------------------------------------------------- host side
static int t2_make_tmap(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows = 128) {
    TmapEncodeFn enc = tmap_encoder();
    if (!enc) return 30001;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {T2_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 30000 + (int)r;
}

template <int EPI, typename TC, int STAGES, int HD = 128>
static int launch_tc2(const T2Maps& maps, void* C, int ldc, int M, int N, int K, int up, int* err, cudaStream_t stream,
                      const T2Qkv& qk = T2Qkv()) {
    constexpr int BN_OUT = (EPI == T2_EPI_SWIGLU) ? T2_BN / 2 : T2_BN;
    constexpr size_t smem = (size_t)STAGES * T2_STAGE_BYTES + 1024;
    auto kern = gemm_tc2_kernel<EPI, TC, STAGES, HD>;
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
    const int tiles = ((M + 2 * T2_BM - 1) / (2 * T2_BM)) * ((N + BN_OUT - 1) / BN_OUT);
    // the tiles of the last, partial wave are cut into 4 or 2 slices when that fits the pairs
    const int all_pairs = n_sm / 2;
    const int rem = tiles % all_pairs;
    int tail_log2 = 0;
    const int max_log2 = EPI == T2_EPI_QKV ? (HD == 64 ? 2 : 1) : 2;       // a slice holds whole heads
    if (rem > 0 && rem * 4 <= all_pairs && max_log2 >= 2) tail_log2 = 2;
    else if (rem > 0 && rem * 2 <= all_pairs) tail_log2 = 1;
    const int tail_tiles = tail_log2 ? rem : 0;
    const int items = tiles - tail_tiles + (tail_tiles << tail_log2);
    const int pairs = items < all_pairs ? items : all_pairs;
    return rllm_launch_clusters(kern, dim3(2 * pairs), dim3(T2_THREADS), smem, stream, dim3(2, 1, 1), maps, (TC*)C, ldc,
                                M, N, K, up, err, tail_tiles, tail_log2, qk);
}

// C[M,N] (+)= A[M,K] . B[N,K]^T with two SMs per 256 x 256 tile.  Arguments, epilogues and return
// values as rllm_gemm_tc (gemm_tc.cu).
RLLM_API int rllm_gemm_tc2(const void* A, const void* B, void* C, int c_dtype, int M, int N, int K, int lda, int ldb,
                           int ldc, int epilogue, int up_row_offset, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || !err)
        return (int)cudaErrorInvalidValue;
    if (epilogue == T2_EPI_ACCUM && c_dtype != RLLM_F32) return (int)cudaErrorInvalidValue;
    T2Maps maps;
    int st = t2_make_tmap(&maps.a, A, M, K, lda);
    if (st) return st;
    const int b_rows = epilogue == T2_EPI_SWIGLU ? up_row_offset + N : N;
    for (int i = 0; i < 3; ++i) {
        st = t2_make_tmap(&maps.b[i], B, b_rows, K, ldb, 128 >> i);
        if (st) return st;
    }
    if (epilogue == T2_EPI_STORE) {
        return c_dtype == RLLM_F32 ? launch_tc2<T2_EPI_STORE, float, 3>(maps, C, ldc, M, N, K, 0, err, stream)
                                   : launch_tc2<T2_EPI_STORE, bf16, 3>(maps, C, ldc, M, N, K, 0, err, stream);
    } else if (epilogue == T2_EPI_ACCUM) {
        return launch_tc2<T2_EPI_ACCUM, float, 3>(maps, C, ldc, M, N, K, 0, err, stream);
    } else if (epilogue == T2_EPI_SWIGLU) {
        return c_dtype == RLLM_F32
                   ? launch_tc2<T2_EPI_SWIGLU, float, 3>(maps, C, ldc, M, N, K, up_row_offset, err, stream)
                   : launch_tc2<T2_EPI_SWIGLU, bf16, 3>(maps, C, ldc, M, N, K, up_row_offset, err, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// The fused q/k/v projection of a prompt step with the q/k norm, the rotary encoding and the cache
// write in its epilogue: A [M, Kdim] rows, W [(H + 2 Kh) * hd, Kdim] the stacked projections (q heads,
// k heads, v heads), head size 64 or 128, bfloat16 queries and cache.  cs_table [M, hd / 2] float2
// (cos, sin) or null; q_norm_w, k_norm_w [hd] float32 or null; slots [M].
RLLM_API int rllm_qkv_tc2(const void* A, const void* W, int M, int Kdim, int lda, int ldw, void* q_out, void* k_cache,
                          void* v_cache, const int* slots, const void* cs_table, const float* q_norm_w,
                          const float* k_norm_w, int H, int Kh, int hd, int bs, float eps, int write_kv,
                          long long n_slots, int* err, cudaStream_t stream) {
    if (M <= 0) return 0;
    const int N = (H + 2 * Kh) * hd;
    if (Kdim <= 0 || (Kdim & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || !err ||
        (hd != 64 && hd != 128) || H <= 0 || Kh <= 0 || bs <= 0 || !slots || !q_out || !k_cache || !v_cache ||
        ((uintptr_t)q_out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)cs_table & 15))
        return (int)cudaErrorInvalidValue;
    T2Maps maps;
    int st = t2_make_tmap(&maps.a, A, M, Kdim, lda);
    if (st) return st;
    for (int i = 0; i < 3; ++i) {
        st = t2_make_tmap(&maps.b[i], W, N, Kdim, ldw, 128 >> i);
        if (st) return st;
    }
    T2Qkv qk;
    qk.q_out = (bf16*)q_out; qk.k_cache = (bf16*)k_cache; qk.v_cache = (bf16*)v_cache; qk.slots = slots;
    qk.cs_table = (const float2*)cs_table; qk.q_norm_w = q_norm_w; qk.k_norm_w = k_norm_w;
    qk.H = H; qk.K = Kh; qk.bs = bs; qk.write_kv = write_kv;
    qk.n_slots = (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots); qk.eps = eps;
    if (hd == 128) return launch_tc2<T2_EPI_QKV, bf16, 3, 128>(maps, nullptr, 0, M, N, Kdim, 0, err, stream, qk);
    return launch_tc2<T2_EPI_QKV, bf16, 3, 64>(maps, nullptr, 0, M, N, Kdim, 0, err, stream, qk);
}

TC_DEFINE_WAIT_CONTROLS(rllm_tc2)

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_gemm_tc2)
RLLM_PACKED(rllm_qkv_tc2)
