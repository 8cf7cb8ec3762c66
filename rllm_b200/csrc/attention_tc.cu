// Causal flash attention over the paged cache for prompt portions on the Blackwell tensor cores:
// S = Q K^T and O += P V are tcgen05.mma with the accumulators S (double-buffered) and O in tensor
// memory; Q, K and V tiles arrive by TMA (128-byte swizzle); P goes from the softmax threads to
// tensor memory (two buffers of its own) and is the A operand of the second product from there.
//
//   tile        128 rows = (128 / g) tokens x g query heads of one key/value head (g = H / K),
//               key tiles of 128 keys (whole pages), head size 128
//   warp 0      TMA producer of Q (once, one 3-D box per half of the head) and of the key tiles: a ring
//               of three stages, one 2-D box per page and half
//   warp 11     TMA producer of the value tiles: a ring of two stages
//   warp 1      issuer of S = Q K^T (one thread): a tile's scores as soon as its keys are there and
//               the softmax threads have read the buffer's scores of two tiles before
//   warp 10     issuer of O += P V (one thread): a tile's product when its P is complete
//   warps 2..9  softmax, two groups of four warps; group 0 takes the key tiles 0, 2, 4, ..., group 1 the
//               others, each with the S and P buffer of its number.  One thread per row (= one TMEM
//               lane) in each group: tcgen05.ld of the 128 scores, mask, maximum (four chains) and
//               sum without any shuffle, exp2 with the scale folded in, P as bfloat16 into its buffer.
//               The reference maximum of a row goes from the thread that treats tile j to the thread
//               of the other group that treats tile j+1 (shared memory, a named barrier per warp
//               pair); it is only raised when the new maximum exceeds it by more than 8 (factor 256):
//               then the thread rescales the row of O in TMEM (tcgen05.ld / st).
//   end         group 0 adds the two groups' row sums, O / l -> bfloat16 -> out[token, head, :]
// What a key tile costs, from cycle stamps of one CTA (4,096 tokens): 2,400 cycles with one issuing
// thread, one softmax group and P laid over its scores; then in turn
//   - one thread issued both products: 2,000 cycles of issue a tile (70 per tcgen05.mma, 75 per
//     commit, 110 per barrier looked at)                                    -> two issuing threads
//   - P over its own scores made Q K^T of tile j+2 wait for P V of tile j: softmax -> P V -> Q K^T ->
//     softmax of the tile after next, 4,700 cycles for two tiles            -> P buffers of its own
//   - the softmax threads waited for P V of the tile before in the middle of their tile, which they
//     need only when they rescale O                                         -> at the tile's end
//   - 128 dependent maxima, 500 cycles                                      -> four chains
//   - one softmax group: 2,100 cycles a tile of which the special-function unit works 1,024
//                                                                           -> two groups, 1,800
//   - one TMA warp: a key tile waited behind the value tile before it, which waits for a product
//     two tiles back; keys came 900 cycles late                             -> a warp for each
// What is left is latency inside each group's stream (barrier looks of 130 cycles, the hand-over of
// the maximum, two warps per scheduler) with the special-function unit 57 % busy.
// Every mbarrier wait is bounded (see tcgen05.cuh); a wait that runs out records a code in the
// error word, raises the abort flag, and every role leaves.
//
// Limits: bfloat16, head size 128, page size a power of two from 8 to 128, g a divisor of 128.
// Other shapes take the mma.sync kernel (attention_flash.cu).  Counterpart in AxiomOperator/rllm:
// attn_fa (crates/rllm-cuda/kernels/kernels.cu:3022-3309), an mma.sync kernel.
#include "tcgen05.cuh"
#include <math.h>

#define AT_HD 128
#define AT_BM 128
#define AT_BN 128
#define AT_THREADS 384                     // key TMA warp, Q.K^T issuer, two groups of four softmax warps, P.V issuer, value TMA warp
#define AT_HALF_BYTES (128 * 128)          // 128 rows x 64 elements x 2 bytes
#define AT_TILE_BYTES (2 * AT_HALF_BYTES)
#define AT_KS 3                            // key tiles in flight: Q.K^T of tile j+1 is issued a tile ahead, and a tile
                                           // takes 2,000 to 3,000 cycles to come in, about what a tile costs
#define AT_VS 2                            // value tiles in flight
#define AT_TABLE_SMEM 4096                 // block-table entries kept in shared memory (more are read from global)

enum { AT_ERR_Q = 11, AT_ERR_KV = 12, AT_ERR_S = 13, AT_ERR_P = 14, AT_ERR_STAGE = 15 };

struct AttnTcParams {
    bf16* out;                  // [n, H, 128]
    const int* positions;       // [n]
    const int* cu_q;            // [R+1]
    const int* block_table;     // [R, table_stride]
    const int* tile_req;        // [tiles]
    const int* tile_tok0;       // [tiles]
    int table_stride, H, K, bs, window, TT, g, n_tiles;
    int n_pages;                // a table entry outside [0, n_pages) is refused (page 0 is read, RLLM_ERR_PAGE)
    float scale_log2;
    int* err;
};

// K-major, 128-byte swizzle (Q, K, P): see smem_desc_sw128.  MN-major (V: dims contiguous):
// leading byte offset = distance between the two 64-dim halves, stride byte offset = 8 keys.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t lbo_bytes) {
    const uint32_t lo = ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

// tcgen05.mma with the A operand in tensor memory (rows = lanes, two bfloat16 per 32-bit column) and B
// from shared memory: the P.V product reads P where the softmax threads left it.
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 2^x by the special-function unit alone (two units in the last place of float32, far below the
// bfloat16 rounding of P that follows); exp2f() costs several instructions more for denormal results.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                               // 32 KB
    unsigned char* sK = smem + AT_TILE_BYTES;               // AT_KS x 32 KB
    unsigned char* sV = smem + (1 + AT_KS) * AT_TILE_BYTES; // AT_VS x 32 KB
    __shared__ __align__(8) uint64_t q_full, k_full[AT_KS], v_full[AT_VS], k_empty[AT_KS], v_empty[AT_VS], s_full[2],
        s_empty[2], p_full[2], p_empty[2];
    __shared__ float m_sh[AT_BM], mg_sh[AT_BM], l_sh[AT_BM];      // per row: reference maximum; group 1's own, and its sum
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ int s_table[AT_TABLE_SMEM];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = p.n_tiles - 1 - (int)blockIdx.x;       // long tiles first
    const int kvh = blockIdx.y;
    const int req = p.tile_req[tile], tok0 = p.tile_tok0[tile];
    const int nt = min(p.TT, p.cu_q[req + 1] - tok0);
    const int head0 = kvh * p.g;
    const int pos_first = p.positions[tok0], pos_last = p.positions[tok0 + nt - 1];
    int kb = p.window > 0 ? max(0, pos_first + 1 - p.window) : 0;
    kb = kb / AT_BN * AT_BN;
    const int n_kt = (pos_last + 1 - kb + AT_BN - 1) / AT_BN;      // >= 1

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
        mbar_init(&q_full, 1);
        for (int s = 0; s < AT_KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < AT_VS; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 128); }
        // p_full has one barrier per S buffer: a softmax warp may be one tile ahead of the others (the
        // scores of tile j + 1 are ready early) and must not add its arrival to the phase of tile j
        mbar_init(&p_full[0], 128);
        mbar_init(&p_full[1], 128);
        mbar_init(&p_empty[0], 1);
        mbar_init(&p_empty[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, 512);
        tmem_relinquish();
    } else if (warp >= 2) {
        // The request's block table goes to shared memory once (the lookups would otherwise be a
        // chain of dependent global loads in front of every tile).  It was uploaded before the
        // step's first kernel, so it is fetched here, beside the set-up of barriers and tensor
        // memory and before the wait for the kernel before this one.
        const int* table = p.block_table + (size_t)req * p.table_stride;
        const int first_blk = kb / p.bs, n_blk = pos_last / p.bs - first_blk + 1;
        for (int i = tid - 64; i < min(n_blk, AT_TABLE_SMEM); i += AT_THREADS - 64) s_table[i] = table[first_blk + i];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // S buffers at columns 0 and 128, O at 256, P buffers (two keys per column) at 384 and 448.  P has
    // columns of its own: laid over its scores it made Q.K^T of tile j + 2 wait for P.V of tile j, and
    // the chain softmax -> P.V -> Q.K^T -> softmax of the tile after next was what a tile cost.
    const uint32_t tS0 = tmem_base, tO = tmem_base + 256, tP0 = tmem_base + 384;
    pdl_wait();                                             // queries and this step's keys come from earlier kernels

    if (warp == 0 || warp == 11) {
        // ------------------------------------------------------------ TMA producers (a whole warp each):
        // warp 0 brings Q and the key tiles, warp 11 the value tiles.  One warp for both made a key
        // tile wait in line behind the value tile before it, which itself waits for a product two
        // tiles back to release its stage.
        const bool keys = warp == 0;
        // Lane pg issues the two boxes (one per 64-dim half) of page pg of a tile; the pages come
        // from the table in shared memory (above).
        const int* table = p.block_table + (size_t)req * p.table_stride;
        const int pages = AT_BN / p.bs;                      // pages per key tile (<= 16)
        const int last_blk = pos_last / p.bs;                // last block that exists for this request
        const int first_blk = kb / p.bs;
        const int n_blk = last_blk - first_blk + 1;
        if (keys && lane == 0) {
            mbar_expect_tx(&q_full, AT_TILE_BYTES);
            tma_load_3d(sQ, &tmQ, 0, head0, tok0, &q_full);
            tma_load_3d(sQ + AT_HALF_BYTES, &tmQ, 64, head0, tok0, &q_full);
        }
        int k_issued = 0, v_issued = 0;
        bool ok = true;
        auto page_row = [&](int j) {                                // first cache row of this lane's page of tile j
            const int rel = min(j * pages + lane, n_blk - 1);      // pages past the context: the last valid page, masked
            if (lane >= pages) return 0;
            int page = rel < AT_TABLE_SMEM ? s_table[rel] : table[first_blk + rel];
            if ((unsigned)page >= (unsigned)p.n_pages) {           // (a box outside the tensor map would read as zeros anyway)
                atomicExch(p.err, RLLM_ERR_PAGE);
                page = 0;
            }
            return (page * p.K + kvh) * p.bs;
        };
        auto load_k = [&](int j) -> bool {
            const int s = j % AT_KS;
            const uint32_t ph = (j / AT_KS) & 1;
            const int y = page_row(j);
            bool got = mbar_wait(&k_empty[s], ph ^ 1, &abort_flag);
            got = __all_sync(0xffffffffu, got);
            if (!got) return false;
            if (lane == 0) mbar_expect_tx(&k_full[s], AT_TILE_BYTES);
            __syncwarp();
            if (lane < pages) {
                unsigned char* dst = sK + s * AT_TILE_BYTES + lane * p.bs * 128;
                tma_load_2d(dst, &tmK, 0, y, &k_full[s]);
                tma_load_2d(dst + AT_HALF_BYTES, &tmK, 64, y, &k_full[s]);
            }
            k_issued = j + 1;
            return true;
        };
        auto load_v = [&](int j) -> bool {
            const int s = j % AT_VS;
            const uint32_t ph = (j / AT_VS) & 1;
            const int y = page_row(j);
            bool got = mbar_wait(&v_empty[s], ph ^ 1, &abort_flag);
            got = __all_sync(0xffffffffu, got);
            if (!got) return false;
            if (lane == 0) mbar_expect_tx(&v_full[s], AT_TILE_BYTES);
            __syncwarp();
            if (lane < pages) {
                unsigned char* dst = sV + s * AT_TILE_BYTES + lane * p.bs * 128;
                tma_load_2d(dst, &tmV, 0, y, &v_full[s]);
                tma_load_2d(dst + AT_HALF_BYTES, &tmV, 64, y, &v_full[s]);
            }
            v_issued = j + 1;
            return true;
        };
        for (int j = 0; j < n_kt && ok; ++j) ok = keys ? load_k(j) : load_v(j);
        if (!ok && lane == 0 && !abort_flag) { atomicExch(p.err, AT_ERR_STAGE); abort_flag = 1; }
        if (abort_flag && lane == 0) {
            // copies that were issued must land before the CTA's shared memory goes away
            volatile int no_abort = 0;
            if (keys) mbar_wait(&q_full, 0, &no_abort);
            for (int j = max(0, k_issued - AT_KS); j < k_issued; ++j) mbar_wait(&k_full[j % AT_KS], (j / AT_KS) & 1, &no_abort);
            for (int j = max(0, v_issued - AT_VS); j < v_issued; ++j) mbar_wait(&v_full[j % AT_VS], (j / AT_VS) & 1, &no_abort);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ issuer of S = Q.K^T
        // Two threads issue the products, this one the scores, one of warp 6 the P.V products: a single
        // thread spent 2,000 of the 2,400 cycles of a key tile issuing (about 70 cycles per
        // tcgen05.mma, 75 per commit, 110 per barrier it looks at) and was what a tile cost.
        constexpr uint32_t idesc_s = idesc_bf16(AT_BM, AT_BN);                 // Q, K both K-major
        bool ok = mbar_wait(&q_full, 0, &abort_flag);
        if (!ok && !abort_flag) { atomicExch(p.err, AT_ERR_Q); abort_flag = 1; }
        const uint32_t q_addr = s_addr(sQ);
        for (int j = 0; j < n_kt && ok; ++j) {
            const int s = j & 1, ks = j % AT_KS;
            const uint32_t ph = (j >> 1) & 1;
            ok = mbar_wait(&k_full[ks], (j / AT_KS) & 1, &abort_flag) &&
                 mbar_wait(&s_empty[s], ph ^ 1, &abort_flag);                  // softmax of tile j-2 has read S[s]
            if (!ok) break;
            tc_fence_after();
            const uint32_t k_addr = s_addr(sK + ks * AT_TILE_BYTES);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_bf16(tS0 + s * AT_BN, smem_desc_sw128(q_addr + h * AT_HALF_BYTES) + 2 * kk,
                              smem_desc_sw128(k_addr + h * AT_HALF_BYTES) + 2 * kk, idesc_s, (h | kk) != 0);
            umma_commit(&k_empty[ks]);
            umma_commit(&s_full[s]);
        }
        if (!ok && !abort_flag) { atomicExch(p.err, AT_ERR_KV); abort_flag = 1; }
    } else if (warp == 10 && lane == 0) {
        // ------------------------------------------------------------ issuer of O += P.V
        constexpr uint32_t idesc_o = idesc_bf16(AT_BM, AT_HD) | (1u << 16);    // V is MN-major
        bool ok = true;
        for (int j = 0; j < n_kt && ok; ++j) {
            const int s = j & 1, vs = j % AT_VS;
            ok = mbar_wait(&p_full[s], (j >> 1) & 1, &abort_flag) && mbar_wait(&v_full[vs], (j / AT_VS) & 1, &abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t v_addr = s_addr(sV + vs * AT_TILE_BYTES);
#pragma unroll
            for (int k8 = 0; k8 < 8; ++k8)        // 16 keys a step: P advances 8 columns (two keys a column), V 16 rows
                umma_bf16_ts(tO, tP0 + s * (AT_BN / 2) + k8 * 8, smem_desc_sw128_mn(v_addr + k8 * 16 * 128, AT_HALF_BYTES),
                             idesc_o, (j | k8) != 0);
            umma_commit(&v_empty[vs]);
            umma_commit(&p_empty[s]);
        }
        if (!ok && !abort_flag) { atomicExch(p.err, AT_ERR_KV); abort_flag = 1; }
    } else if (warp >= 2 && warp < 10) {
        // ------------------------------------------------------------ softmax and epilogue: one row per thread
        // Two groups of four warps: group 0 takes the key tiles 0, 2, 4, ..., group 1 the tiles 1, 3, 5, ...,
        // each with the S and P buffers of its number, so that the exponentials of one tile (the
        // special-function unit's 1,024 cycles) run beside the loads, maxima and barrier round trips
        // of the next.  Row r belongs to thread r of both groups.  What the two share per row is the
        // reference maximum: it is handed from the thread that treats tile j to the one that treats
        // tile j+1 through shared memory and a named barrier of the two warps, right after the
        // maximum of tile j is known.  Each group keeps its own part of the row sum, relative to the
        // reference it last saw; O is one accumulator, rescaled by whichever thread raises the reference.
        const int wg = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int tl = r / p.g, hl = r % p.g;
        const bool valid = tl < nt;
        const int pos_r = valid ? p.positions[tok0 + tl] : -1;
        const int first_r = p.window > 0 ? max(0, pos_r + 1 - p.window) : 0;
        const int bar_mine = 1 + wg * 4 + quarter;           // arrived at by this warp, waited for by its partner
        const int bar_partner = 1 + (1 - wg) * 4 + quarter;
        const int b = wg;
        float m_mine = -INFINITY, l = 0.f;
        bool ok = true;
        // Every iteration passes the named barriers, whatever happened: they have no time-out.  A wait
        // that fails makes the rest of the thread's work empty (ok == false, uniform over the warp).
        for (int j = wg; j < n_kt; j += 2) {
            const uint32_t ph = (j >> 1) & 1;
            const int kt = kb + j * AT_BN;
            if (ok && !mbar_wait(&s_full[b], ph, &abort_flag)) {
                if (!abort_flag) { atomicExch(p.err, AT_ERR_S); abort_flag = 1; }
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            float sv[AT_BN];
            float mx = -INFINITY;
            if (ok) {
                tc_fence_after();
                // the whole row of scores with one wait: four loads of 32 columns in flight together
                uint32_t rr[AT_BN / 32][32];
#pragma unroll
                for (int c0 = 0; c0 < AT_BN / 32; ++c0) tmem_ld32(tS0 + b * AT_BN + lane_base + c0 * 32, rr[c0]);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < AT_BN; ++c) sv[c] = __uint_as_float(rr[c >> 5][c & 31]);
                tc_fence_before();
                mbar_arrive(&s_empty[b]);
                // The maximum is taken over the raw scores (the scale is positive) and the scale goes
                // into the exponent's multiply-add: one FFMA and one MUFU per score.
                const bool need_mask = (kt + AT_BN > pos_r + 1) || (kt < first_r);
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < AT_BN; ++c)
                        if (kt + c > pos_r || kt + c < first_r) sv[c] = -INFINITY;
                }
                // four chains of 32: one chain of 128 maxima is 128 dependent instructions (500 cycles a tile)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < AT_BN; c += 4) {
                    mx4[0] = fmaxf(mx4[0], sv[c]); mx4[1] = fmaxf(mx4[1], sv[c + 1]);
                    mx4[2] = fmaxf(mx4[2], sv[c + 2]); mx4[3] = fmaxf(mx4[3], sv[c + 3]);
                }
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            }
            // the row's reference after tile j-1, from the partner; then this tile's decision, for the partner
            if (j > 0) asm volatile("bar.sync %0, 64;" ::"r"(bar_partner) : "memory");
            float m_ref = j > 0 ? m_sh[r] : -INFINITY;
            float alpha = 1.f;
            bool rescale = false;
            if (ok) {
                if (m_ref == -INFINITY) m_ref = mx;                          // nothing accumulated yet for this row
                else if (mx > m_ref + 8.f) { alpha = exp2f(m_ref - mx); m_ref = mx; rescale = true; }
            }
            m_sh[r] = m_ref;
            if (j + 1 < n_kt) asm volatile("bar.arrive %0, 64;" ::"r"(bar_mine) : "memory");
            if (m_mine != m_ref) {                                           // this group's sum follows the reference
                l = m_mine == -INFINITY ? 0.f : l * exp2f(m_mine - m_ref);
                m_mine = m_ref;
            }
            // O is shared with the products in flight: it is rescaled only after P.V of the tile
            // before (the partner's) has completed; P[b] is written only after P.V of this group's
            // tile before (j-2) has read it.  p_empty[x] counts the products of the tiles of group x:
            // a thread looks at every phase of both, in order and each once (a parity wait is only
            // right for the phase after the last one seen), and at the partner's before its own
            // arrival lets the next product start, so that no barrier is ever two phases ahead of it.
            // A warp that rescales looks at the partner's here; the others at the end of the tile,
            // when that product has long completed.
            // tcgen05.ld / st are warp-wide: the whole warp goes through when any of its rows rescales
            const bool warp_rescales = __any_sync(0xffffffffu, rescale);
            bool seen_partner = j == 0;
            if (ok && warp_rescales && j > 0) {
                if (!mbar_wait(&p_empty[1 - b], ((j - 1) >> 1) & 1, &abort_flag)) {
                    if (!abort_flag) { atomicExch(p.err, AT_ERR_P); abort_flag = 1; }
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                seen_partner = true;
                if (ok) {
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < AT_HD; c0 += 32) {
                        uint32_t rr2[32];
                        tmem_ld32(tO + lane_base + c0, rr2);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) rr2[i] = __float_as_uint(__uint_as_float(rr2[i]) * alpha);
                        tmem_st32(tO + lane_base + c0, rr2);
                    }
                    tmem_st_wait();
                }
            }
            if (ok && j >= 2 && !mbar_wait(&p_empty[b], ph ^ 1, &abort_flag)) {   // P.V of tile j-2 has read P[b]
                if (!abort_flag) { atomicExch(p.err, AT_ERR_P); abort_flag = 1; }
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                const float mref = m_ref == -INFINITY ? 0.f : m_ref;
                float sum = 0.f;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    uint32_t pk[32];                                       // half the row's P, two keys per word
#pragma unroll
                    for (int c = 0; c < 64; c += 2) {
                        const float e0 = ex2_approx(fmaf(sv[hh * 64 + c], p.scale_log2, -mref));
                        const float e1 = ex2_approx(fmaf(sv[hh * 64 + c + 1], p.scale_log2, -mref));
                        sum += e0 + e1;
                        __nv_bfloat162 pp = __floats2bfloat162_rn(e0, e1);
                        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&pp);
                    }
                    tmem_st32(tP0 + b * (AT_BN / 2) + lane_base + hh * 32, pk);
                }
                l += sum;
                tmem_st_wait();
                if (!seen_partner && !mbar_wait(&p_empty[1 - b], ((j - 1) >> 1) & 1, &abort_flag)) {
                    if (!abort_flag) { atomicExch(p.err, AT_ERR_P); abort_flag = 1; }
                    ok = false;
                }
                if (ok) {
                    tc_fence_before();
                    mbar_arrive(&p_full[b]);
                }
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        // group 1 hands its part of the row sum to group 0, which writes the rows out
        if (wg == 1) {
            l_sh[r] = l;
            mg_sh[r] = m_mine;
            asm volatile("bar.arrive 9, 256;" ::: "memory");
        } else {
            asm volatile("bar.sync 9, 256;" ::: "memory");
            const int jl = n_kt - 1;                                   // the last product: all before it have completed too
            if (ok && !mbar_wait(&p_empty[jl & 1], (jl >> 1) & 1, &abort_flag)) {
                if (!abort_flag) { atomicExch(p.err, AT_ERR_P); abort_flag = 1; }
                ok = false;
            }
            const float m_fin = m_sh[r];
            const float m_other = mg_sh[r];
            if (n_kt > 1 && m_other != -INFINITY) l = (m_mine == -INFINITY ? 0.f : l * exp2f(m_mine - m_fin)) + l_sh[r] * exp2f(m_other - m_fin);
            else if (m_mine != -INFINITY && m_mine != m_fin) l *= exp2f(m_mine - m_fin);
        }
        pdl_launch_dependents();
        if (wg == 0 && __all_sync(0xffffffffu, ok)) {              // warp-uniform: the TMEM loads are warp-wide
            tc_fence_after();
            const bool store = valid && l > 0.f;
            const float inv = store ? 1.0f / l : 0.f;
            bf16* dst = p.out + ((size_t)(tok0 + (valid ? tl : 0)) * p.H + head0 + hl) * AT_HD;
#pragma unroll
            for (int c0 = 0; c0 < AT_HD; c0 += 32) {
                uint32_t rr[32];
                tmem_ld32(tO + lane_base + c0, rr);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 u;
                    __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(rr[8 * q]) * inv, __uint_as_float(rr[8 * q + 1]) * inv);
                    __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(rr[8 * q + 2]) * inv, __uint_as_float(rr[8 * q + 3]) * inv);
                    __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(rr[8 * q + 4]) * inv, __uint_as_float(rr[8 * q + 5]) * inv);
                    __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(rr[8 * q + 6]) * inv, __uint_as_float(rr[8 * q + 7]) * inv);
                    u.x = *reinterpret_cast<uint32_t*>(&a0); u.y = *reinterpret_cast<uint32_t*>(&a1);
                    u.z = *reinterpret_cast<uint32_t*>(&a2); u.w = *reinterpret_cast<uint32_t*>(&a3);
                    if (store) reinterpret_cast<uint4*>(dst + c0)[q] = u;
                }
            }
        }
    }
    __syncwarp();          // the lanes of the MMA warp that had no role meet the elected one: the barrier wants whole warps
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// q, out [n, H, 128] bfloat16; caches [pages, K, bs, 128] bfloat16; tiles of TT = 128 / (H / K) tokens.
// Returns cudaErrorInvalidValue for shapes outside the limits named at the top of this file.
RLLM_API int rllm_attention_tc(const void* q, const void* k_cache, const void* v_cache, void* out, int n_tokens,
                               long long n_pages, const int* positions, const int* cu_q, const int* block_table,
                               int table_stride, const int* tile_req, const int* tile_tok0, int n_tiles, int H, int K,
                               int hd, int bs, float scale, int window, int* err, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (hd != AT_HD || K <= 0 || H % K || bs < 8 || bs > 128 || (bs & (bs - 1)) || !err) return (int)cudaErrorInvalidValue;
    const int g = H / K;
    if (g > 128 || 128 % g) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
        return (int)cudaErrorInvalidValue;
    const int TT = 128 / g;
    CUtensorMap tq, tk, tv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)H, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)H * hd * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)g, (cuuint32_t)TT};
        int st = tmap_encode_bf16(&tq, q, 3, dims, strides, box);
        if (st) return st;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)n_pages * K * bs};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)bs};
        int st = tmap_encode_bf16(&tk, k_cache, 2, dims, strides, box);
        if (st) return st;
        st = tmap_encode_bf16(&tv, v_cache, 2, dims, strides, box);
        if (st) return st;
    }
    AttnTcParams p;
    p.out = (bf16*)out; p.positions = positions; p.cu_q = cu_q; p.block_table = block_table; p.tile_req = tile_req;
    p.tile_tok0 = tile_tok0; p.table_stride = table_stride; p.H = H; p.K = K; p.bs = bs; p.window = window; p.TT = TT;
    p.g = g; p.n_tiles = n_tiles; p.scale_log2 = scale * 1.4426950408889634f; p.err = err;
    p.n_pages = (int)(n_pages > 0x7fffffffLL ? 0x7fffffffLL : n_pages);
    constexpr int smem = (1 + AT_KS + AT_VS) * AT_TILE_BYTES + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    return rllm_launch(attention_tc_kernel, dim3(n_tiles, K), dim3(AT_THREADS), smem, stream, tq, tk, tv, p);
}

TC_DEFINE_WAIT_CONTROLS(rllm_attn_tc)

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_attention_tc)
