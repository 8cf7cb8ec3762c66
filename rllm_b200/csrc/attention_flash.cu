// Paged causal flash attention on the tensor cores (bfloat16 in, float32 softmax and accumulation),
// for prompt portions and for decode, over the same paged cache.
//
// Rows of a tile are (token, query head of one key/value head) pairs: the GQA group shares every
// key/value tile that is staged in shared memory (AxiomOperator/rllm lays its prefill tiles out the
// same way: crates/rllm-cuda/kernels/kernels.cu:3022-3309, attn_fa; its decode kernel is the
// split-context attn_decode, 2786-3011, with attn_decode_combine, 2964-2984).
//
//   S = Q K^T  : mma.sync m16n8k16, A = Q fragments kept in registers, B = K rows via ldmatrix
//   softmax    : online, float32, exp2 with the scale folded in, masks for causality and window
//   O += P V   : P re-used from the S accumulators as A fragments, B = V via ldmatrix.trans
//
// Shapes:
//   prefill: NW = 4 warps x 16 rows, key tiles of 64, whole key range, writes normalized output
//            (head size 128 with a suitable group size takes the tcgen05 kernel in attention_tc.cu)
//   decode : the key range cut into splits of `split_keys` keys (a function of the position only,
//            never of the batch); unnormalized partials (o, m, l) per split that
//            paged_flash_combine merges in split order.  Two kernels write those partials:
//            - paged_decode_attention_kernel, tiles of at most 8 (token, head) rows, the product
//              turned round (keys as the M side of the MMA); one warp per CTA; the default;
//            - the 1-warp, 16-row instance of the template for callers with tiles of 9 to 16 rows.
// K/V tiles come in through cp.async (16-byte chunks, zero-filled beyond the context) into a
// double buffer with an XOR swizzle on the chunk index, so ldmatrix is free of bank conflicts.
// Any page size; head size 64 or 128 (other sizes take the plain kernel).
#include "common.cuh"
#include <math.h>

struct FlashParams {
    const bf16* q;            // [n, H, HD]
    const bf16* k_cache;      // [pages, K, bs, HD]
    const bf16* v_cache;
    bf16* out;                // [n, H, HD]
    float* part_o;            // [tile, kvh*chunks, split, rows, HD]   (decode)
    float* part_ml;           // [tile, kvh*chunks, split, rows, 2]
    const int* positions;     // [n]
    const int* cu_q;          // [R+1]
    const int* block_table;   // [R, table_stride]
    const int* tile_req;      // [tiles] request row of each tile
    const int* tile_tok0;     // [tiles] first flat token of each tile
    int table_stride;
    int n_pages;              // pages of the pool: a table entry outside [0, n_pages) is refused (page 0 is read, *err set)
    int* err;                 // the error word, or null
    int H, K, bs, window;
    int TT, GH, head_chunks;  // tokens per tile, heads per token in a tile, chunks of the GQA group
    int split_keys;           // 0: no split
    int part_rows;            // rows kept per partial (TT * GH)
    float scale_log2;         // softmax scale * log2(e)
};

// A table entry outside the pool is refused: page 0 is read in its place (its keys are masked or
// not, the step's results are not to be used either way) and the error word says so.
__device__ __forceinline__ int checked_page(const FlashParams& p, int page) {
    if ((unsigned)page >= (unsigned)p.n_pages) {
        if (p.err) atomicExch(p.err, RLLM_ERR_PAGE);
        return 0;
    }
    return page;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// The NW warps take 16 rows each and share every key tile (ring of two).
template <int HD, int NW, int BN>
__global__ void __launch_bounds__(NW * 32) paged_flash_attention_kernel(const FlashParams p) {
    constexpr int CH = HD / 8;                    // 16-byte chunks per key row
    constexpr int TILE_BYTES = BN * HD * 2;
    constexpr int NT_S = BN / 8;                  // score n-tiles
    constexpr int NT_O = HD / 8;                  // output n-tiles
    extern __shared__ __align__(128) unsigned char smem[];   // [2 stages][K tile, V tile]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    pdl_wait();          // queries, positions and this step's keys come from the kernels before

    const int tile = blockIdx.x;
    const int req = p.tile_req[tile], tok0 = p.tile_tok0[tile];
    const int nt = min(p.TT, p.cu_q[req + 1] - tok0);
    const int grp = p.H / p.K;
    const int kvh = blockIdx.y / p.head_chunks, hc = blockIdx.y % p.head_chunks;
    const int head0 = kvh * grp + hc * p.GH;
    const int nh = min(p.GH, grp - hc * p.GH);
    const int pos_first = p.positions[tok0], pos_last = p.positions[tok0 + nt - 1];
    int lo = p.window > 0 ? max(0, pos_first + 1 - p.window) : 0;
    lo = lo / BN * BN;
    int kb = lo, ke = pos_last + 1;
    if (p.split_keys > 0) {
        kb = lo + blockIdx.z * p.split_keys;
        ke = min(ke, kb + p.split_keys);
    }
    const size_t part_base = (((size_t)tile * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z) * p.part_rows;

    // this thread's two rows: (token, head) pairs
    const int R0 = warp * 16 + g, R1 = R0 + 8;
    const int tl0 = R0 / p.GH, hl0 = R0 % p.GH, tl1 = R1 / p.GH, hl1 = R1 % p.GH;
    const bool valid0 = tl0 < nt && hl0 < nh, valid1 = tl1 < nt && hl1 < nh;
    const int pos0 = valid0 ? p.positions[tok0 + tl0] : -1, pos1 = valid1 ? p.positions[tok0 + tl1] : -1;
    const int first0 = p.window > 0 ? max(0, pos0 + 1 - p.window) : 0;
    const int first1 = p.window > 0 ? max(0, pos1 + 1 - p.window) : 0;
    const int hi0 = min(pos0 + 1, ke), hi1 = min(pos1 + 1, ke);

    if (kb >= ke) {                                // an empty split: mark it so
        if (p.split_keys > 0 && t == 0) {
            if (R0 < p.part_rows) { p.part_ml[(part_base + R0) * 2] = -INFINITY; p.part_ml[(part_base + R0) * 2 + 1] = 0.f; }
            if (R1 < p.part_rows) { p.part_ml[(part_base + R1) * 2] = -INFINITY; p.part_ml[(part_base + R1) * 2 + 1] = 0.f; }
        }
        return;
    }

    // Q fragments
    uint32_t qf[HD / 16][4];
    {
        const bf16* q0 = p.q + ((size_t)(tok0 + (valid0 ? tl0 : 0)) * p.H + head0 + (valid0 ? hl0 : 0)) * HD;
        const bf16* q1 = p.q + ((size_t)(tok0 + (valid1 ? tl1 : 0)) * p.H + head0 + (valid1 ? hl1 : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            qf[ks][0] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
            qf[ks][2] = valid0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
            qf[ks][3] = valid1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    const int* table = p.block_table + (size_t)req * p.table_stride;
    // Each thread copies the same 16-byte chunk column of several rows: the chunk index is fixed,
    // the page of a row is looked up once per row (a shift when the page size is a power of two).
    static_assert((NW * 32) % CH == 0, "threads must cover whole rows of chunks");
    constexpr int ROWS_PER_PASS = NW * 32 / CH;
    const int my_chunk = tid % CH, my_row0 = tid / CH;
    const int last_blk = (ke - 1) / p.bs;
    auto load_tile = [&](int stage, int kt) {
        unsigned char* sk = smem + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* sv = sk + TILE_BYTES;
        // page by page: one table look-up and one base address per page, then a stride per row
        int row0 = 0;                                    // first tile row of the current page
        while (row0 < BN) {
            const int key0 = kt + row0;
            const int blk = key0 / p.bs, off0 = key0 - blk * p.bs;
            const int rows_here = min(p.bs - off0, BN - row0);
            const int page = checked_page(p, table[min(blk, last_blk)]);  // beyond the range: any valid address, zero fill
            const size_t base = (((size_t)page * p.K + kvh) * p.bs + off0) * HD + my_chunk * 8;
            const bf16* ksrc = p.k_cache + base;
            const bf16* vsrc = p.v_cache + base;
            // this thread's rows are those congruent to my_row0 modulo ROWS_PER_PASS
            int r = (my_row0 - row0 % ROWS_PER_PASS + ROWS_PER_PASS) % ROWS_PER_PASS;
#pragma unroll 4
            for (; r < rows_here; r += ROWS_PER_PASS) {
                const int row = row0 + r;
                const bool ok = blk <= last_blk && kt + row < ke;
                const uint32_t dst = row * (HD * 2) + ((my_chunk ^ (row & 7)) << 4);
                cp_async16(smem_u32(sk + dst), ksrc + (ok ? r * HD : 0), ok ? 16 : 0);
                cp_async16(smem_u32(sv + dst), vsrc + (ok ? r * HD : 0), ok ? 16 : 0);
            }
            row0 += rows_here;
        }
    };

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int n_tiles = (ke - kb + BN - 1) / BN;
    load_tile(0, kb);
    cp_async_commit();
    const int mi = lane >> 3, ri = lane & 7;
    for (int it = 0; it < n_tiles; ++it) {
        const int kt = kb + it * BN;
        if (it + 1 < n_tiles) load_tile((it + 1) & 1, kt + BN);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* sk = smem + (size_t)(it & 1) * 2 * TILE_BYTES;
        const unsigned char* sv = sk + TILE_BYTES;

        // ---- S = Q K^T
        float s[NT_S][4];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                const int row = np * 16 + (mi >> 1) * 8 + ri;
                const int chunk = ks * 2 + (mi & 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4(smem_u32(sk + row * (HD * 2) + ((chunk ^ ri) << 4)), b0, b1, b2, b3);
                mma_bf16(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                mma_bf16(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
            }
        }
        // ---- scale, mask, online softmax
        const bool need_mask = (kt + BN > min(hi0, hi1)) || (kt < max(first0, first1));
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * p.scale_log2;
                if (need_mask) {
                    const int key = kt + 8 * j + 2 * t + (e & 1);
                    const bool vis = (e < 2) ? (key >= first0 && key < hi0) : (key >= first1 && key < hi1);
                    if (!vis) v = -INFINITY;
                }
                s[j][e] = v;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = exp2f(m0 - ms0), al1 = exp2f(m1 - ms1);      // exp2(-inf) = 0
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            s[j][0] = exp2f(s[j][0] - ms0); s[j][1] = exp2f(s[j][1] - ms0);
            s[j][2] = exp2f(s[j][2] - ms1); s[j][3] = exp2f(s[j][3] - ms1);
            rs0 += s[j][0] + s[j][1];
            rs1 += s[j][2] + s[j][3];
        }
        l0 = l0 * al0 + rs0;
        l1 = l1 * al1 + rs1;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                const int row = kk * 16 + (mi & 1) * 8 + ri;
                const int chunk = dp * 2 + (mi >> 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(smem_u32(sv + row * (HD * 2) + ((chunk ^ ri) << 4)), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();                           // the stage may be overwritten from here on
    }
    pdl_launch_dependents();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    if (p.split_keys > 0) {
        if (R0 < p.part_rows) {
            float* po = p.part_o + (part_base + R0) * HD;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) *reinterpret_cast<float2*>(po + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
            if (t == 0) { p.part_ml[(part_base + R0) * 2] = m0; p.part_ml[(part_base + R0) * 2 + 1] = valid0 ? l0 : 0.f; }
        }
        if (R1 < p.part_rows) {
            float* po = p.part_o + (part_base + R1) * HD;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) *reinterpret_cast<float2*>(po + 8 * j + 2 * t) = make_float2(o[j][2], o[j][3]);
            if (t == 0) { p.part_ml[(part_base + R1) * 2] = m1; p.part_ml[(part_base + R1) * 2 + 1] = valid1 ? l1 : 0.f; }
        }
    } else {
        if (valid0) {
            const float inv = l0 > 0.f ? 1.0f / l0 : 0.f;
            bf16* po = p.out + ((size_t)(tok0 + tl0) * p.H + head0 + hl0) * HD;
#pragma unroll
            for (int j = 0; j < NT_O; ++j)
                *reinterpret_cast<uint32_t*>(po + 8 * j + 2 * t) = pack_bf16(o[j][0] * inv, o[j][1] * inv);
        }
        if (valid1) {
            const float inv = l1 > 0.f ? 1.0f / l1 : 0.f;
            bf16* po = p.out + ((size_t)(tok0 + tl1) * p.H + head0 + hl1) * HD;
#pragma unroll
            for (int j = 0; j < NT_O; ++j)
                *reinterpret_cast<uint32_t*>(po + 8 * j + 2 * t) = pack_bf16(o[j][2] * inv, o[j][3] * inv);
        }
    }
}

// Merges the partials of the decode shape in split order (fixed order: the result is reproducible)
// and writes the normalized output.  grid (tiles, K * head_chunks, rows), one thread per output dim.

// ---------------------------------------------------------------------------------------------------
// Decode with at most 8 query rows per tile: the product is turned round.  In the kernel above the
// query rows are the M side of the MMA (16 rows, of which a decode step with a GQA group of 4 uses 4).
// Here the KEYS are the M side (16 keys per MMA, all of them real) and the query rows the N side
// (8 columns):
//
//   S^T[key, row] = K . Q^T  : A = K rows via ldmatrix, B = Q fragments kept in registers
//   softmax over the keys    : across the 8 lanes that share a column pair, float32
//   O^T[d, row] += V^T . P^T : A = V via ldmatrix.trans, B = P^T from the S^T accumulators through
//                              movmatrix (an 8x8 transpose inside the warp)
//
// Half the MMAs, ldmatrix and exponentials of the 16-row form for the same keys, and half the
// accumulators; the kernel is bound by the latency of its own instruction stream (one warp per
// CTA, few warps per SM), so that is what counts.  Same splits, partials and combine kernel.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

template <int HD, int BN, int NS>
__global__ void __launch_bounds__(32) paged_decode_attention_kernel(const FlashParams p) {
    constexpr int CH = HD / 8;
    constexpr int TILE_BYTES = BN * HD * 2;
    constexpr int KB = BN / 16;                   // blocks of 16 keys per tile
    constexpr int DT = HD / 16;                   // blocks of 16 head dims
    extern __shared__ __align__(128) unsigned char smem[];   // [NS stages][K tile, V tile]
    const int lane = threadIdx.x, g = lane >> 2, t = lane & 3;
    // No griddepcontrol.wait yet: the tiles, positions and block tables were uploaded before the
    // step's first kernel, and the keys of earlier steps are in the cache; only the queries and
    // this step's own keys come from the kernels before (see below).
    const int tile = blockIdx.x;
    const int req = p.tile_req[tile], tok0 = p.tile_tok0[tile];
    const int nt = min(p.TT, p.cu_q[req + 1] - tok0);
    const int grp = p.H / p.K;
    const int kvh = blockIdx.y / p.head_chunks, hc = blockIdx.y % p.head_chunks;
    const int head0 = kvh * grp + hc * p.GH;
    const int nh = min(p.GH, grp - hc * p.GH);
    const int pos_first = p.positions[tok0], pos_last = p.positions[tok0 + nt - 1];
    int lo = p.window > 0 ? max(0, pos_first + 1 - p.window) : 0;
    lo = lo / BN * BN;
    int kb = lo, ke = pos_last + 1;
    if (p.split_keys > 0) {
        kb = lo + blockIdx.z * p.split_keys;
        ke = min(ke, kb + p.split_keys);
    }
    const size_t part_base = (((size_t)tile * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z) * p.part_rows;

    // the two columns (query rows) of this lane's accumulators: 2t and 2t + 1
    int rowc[2], tlc[2], hlc[2], firstc[2], hic[2];
    bool validc[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        rowc[x] = 2 * t + x;
        tlc[x] = rowc[x] / p.GH;
        hlc[x] = rowc[x] % p.GH;
        validc[x] = tlc[x] < nt && hlc[x] < nh;
        const int pos = validc[x] ? p.positions[tok0 + tlc[x]] : -1;
        firstc[x] = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
        hic[x] = min(pos + 1, ke);
    }
    if (kb >= ke) {                                // an empty split: mark it so
        pdl_wait();                                // the partials of the layer before may still be read
        if (p.split_keys > 0 && g == 0) {
#pragma unroll
            for (int x = 0; x < 2; ++x)
                if (rowc[x] < p.part_rows) {
                    p.part_ml[(part_base + rowc[x]) * 2] = -INFINITY;
                    p.part_ml[(part_base + rowc[x]) * 2 + 1] = 0.f;
                }
        }
        return;
    }

    const int* table = p.block_table + (size_t)req * p.table_stride;
    constexpr int ROWS_PER_PASS = 32 / CH;
    static_assert(32 % CH == 0, "a warp must cover whole rows of chunks");
    const int my_chunk = lane % CH, my_row0 = lane / CH;
    const int last_blk = (ke - 1) / p.bs;
    // Fast path (page size a power of two and at least a tile): a tile lies in one page, so one
    // table look-up and one base address per tile; this lane's rows are my_row0 + i * ROWS_PER_PASS,
    // their swizzled positions are fixed and kept in registers.
    constexpr int MY_ROWS = BN / ROWS_PER_PASS;
    const bool one_page = (p.bs & (p.bs - 1)) == 0 && p.bs >= BN;
    const int bs_shift = __ffs(p.bs) - 1;
    uint32_t dst_off[MY_ROWS];
#pragma unroll
    for (int i = 0; i < MY_ROWS; ++i) {
        const int row = my_row0 + i * ROWS_PER_PASS;
        dst_off[i] = row * (HD * 2) + ((my_chunk ^ (row & 7)) << 4);
    }
    const uint32_t smem_base = smem_u32(smem);
    auto load_tile = [&](int stage, int kt) {
        if (one_page) {
            const int blk = kt >> bs_shift, off0 = kt & (p.bs - 1);
            const int page = checked_page(p, table[min(blk, last_blk)]);
            const size_t base = (((size_t)page * p.K + kvh) * p.bs + off0 + my_row0) * HD + my_chunk * 8;
            const bf16* ksrc = p.k_cache + base;
            const bf16* vsrc = p.v_cache + base;
            const uint32_t sk = smem_base + stage * 2 * TILE_BYTES, sv = sk + TILE_BYTES;
            const int left = ke - kt - my_row0;             // rows i with i * ROWS_PER_PASS < left exist
#pragma unroll
            for (int i = 0; i < MY_ROWS; ++i) {
                const bool ok = i * ROWS_PER_PASS < left;   // beyond the range: zero fill, any valid address
                const int src = ok ? i * ROWS_PER_PASS * HD : 0;
                cp_async16(sk + dst_off[i], ksrc + src, ok ? 16 : 0);
                cp_async16(sv + dst_off[i], vsrc + src, ok ? 16 : 0);
            }
            return;
        }
        unsigned char* sk = smem + (size_t)stage * 2 * TILE_BYTES;
        unsigned char* sv = sk + TILE_BYTES;
        int row0 = 0;
        while (row0 < BN) {
            const int key0 = kt + row0;
            const int blk = key0 / p.bs, off0 = key0 - blk * p.bs;
            const int rows_here = min(p.bs - off0, BN - row0);
            const int page = checked_page(p, table[min(blk, last_blk)]);
            const size_t base = (((size_t)page * p.K + kvh) * p.bs + off0) * HD + my_chunk * 8;
            const bf16* ksrc = p.k_cache + base;
            const bf16* vsrc = p.v_cache + base;
            int r = (my_row0 - row0 % ROWS_PER_PASS + ROWS_PER_PASS) % ROWS_PER_PASS;
#pragma unroll 4
            for (; r < rows_here; r += ROWS_PER_PASS) {
                const int row = row0 + r;
                const bool ok = blk <= last_blk && kt + row < ke;
                const uint32_t dst = row * (HD * 2) + ((my_chunk ^ (row & 7)) << 4);
                cp_async16(smem_u32(sk + dst), ksrc + (ok ? r * HD : 0), ok ? 16 : 0);
                cp_async16(smem_u32(sv + dst), vsrc + (ok ? r * HD : 0), ok ? 16 : 0);
            }
            row0 += rows_here;
        }
    };

    float o[DT][4];                                // O^T: (d = 16 dp + g, + 8) x (rows 2t, 2t + 1)
#pragma unroll
    for (int j = 0; j < DT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float mx[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.f, 0.f};

    const int n_tiles = (ke - kb + BN - 1) / BN;
    // The first NS - 1 tiles are requested before the wait when they hold keys of earlier steps
    // only (all splits of a request but its last one or two): the kernel starts while the one
    // before it still runs, and its first memory round trip is over when that one ends.
    const int written_from = p.positions[p.cu_q[req]];          // first position this step writes for the request
    const bool ahead = kb + min(n_tiles, NS - 1) * BN <= written_from;
    if (ahead) {
#pragma unroll
        for (int i = 0; i < NS - 1; ++i) {         // NS - 1 tiles ahead; empty groups keep the count uniform
            if (i < n_tiles) load_tile(i, kb + i * BN);
            cp_async_commit();
        }
    }
    pdl_wait();
    if (!ahead) {
#pragma unroll
        for (int i = 0; i < NS - 1; ++i) {
            if (i < n_tiles) load_tile(i, kb + i * BN);
            cp_async_commit();
        }
    }
    // Q as the B operand: column g is query row g
    uint32_t qf[DT][2];
    {
        const int tlq = g / p.GH, hlq = g % p.GH;
        const bool validq = tlq < nt && hlq < nh;
        const bf16* qr = p.q + ((size_t)(tok0 + (validq ? tlq : 0)) * p.H + head0 + (validq ? hlq : 0)) * HD;
#pragma unroll
        for (int ks = 0; ks < DT; ++ks) {
            qf[ks][0] = validq ? *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = validq ? *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    // ldmatrix lane roles.  K (A of S^T, no transpose): matrices (keys 0-7 | 8-15) x (d 0-7 | 8-15).
    // V (A of O^T, transposed): matrices (d 0-7 | 8-15) x (keys 0-7 | 8-15).
    const int mat = lane >> 3, ri = lane & 7;
    const int k_row = (mat & 1) * 8 + ri, k_ch = mat >> 1;
    const int v_row = (mat >> 1) * 8 + ri, v_ch = mat & 1;
    for (int it = 0; it < n_tiles; ++it) {
        const int kt = kb + it * BN;
        if (it + NS - 1 < n_tiles) load_tile((it + NS - 1) % NS, kt + (NS - 1) * BN);
        cp_async_commit();
        cp_async_wait<NS - 1>();
        __syncwarp();
        const unsigned char* sk = smem + (size_t)(it % NS) * 2 * TILE_BYTES;
        const unsigned char* sv = sk + TILE_BYTES;

        // ---- S^T = K Q^T
        float s[KB][4];
#pragma unroll
        for (int j = 0; j < KB; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < DT; ++ks) {
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                const int row = j * 16 + k_row;
                uint32_t a0, a1, a2, a3;
                ldsm_x4(smem_u32(sk + row * (HD * 2) + (((ks * 2 + k_ch) ^ (row & 7)) << 4)), a0, a1, a2, a3);
                mma_bf16(s[j], a0, a1, a2, a3, qf[ks][0], qf[ks][1]);
            }
        }
        // ---- scale, mask, online softmax over the keys (lanes of equal t hold one column pair)
        const bool need_mask = (kt + BN > min(hic[0], hic[1])) || (kt < max(firstc[0], firstc[1]));
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < KB; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * p.scale_log2;
                if (need_mask) {
                    const int key = kt + 16 * j + g + (e >> 1) * 8;
                    const int x = e & 1;
                    if (!(key >= firstc[x] && key < hic[x])) v = -INFINITY;
                }
                s[j][e] = v;
            }
            tmax[0] = fmaxf(tmax[0], fmaxf(s[j][0], s[j][2]));
            tmax[1] = fmaxf(tmax[1], fmaxf(s[j][1], s[j][3]));
        }
        float al[2], ms[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 4));
            tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 8));
            tmax[x] = fmaxf(tmax[x], __shfl_xor_sync(0xffffffffu, tmax[x], 16));
            const float mn = fmaxf(mx[x], tmax[x]);
            ms[x] = mn == -INFINITY ? 0.f : mn;
            al[x] = exp2f(mx[x] - ms[x]);                          // exp2(-inf) = 0
            mx[x] = mn;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < KB; ++j) {
            s[j][0] = exp2f(s[j][0] - ms[0]); s[j][1] = exp2f(s[j][1] - ms[1]);
            s[j][2] = exp2f(s[j][2] - ms[0]); s[j][3] = exp2f(s[j][3] - ms[1]);
            rs[0] += s[j][0] + s[j][2];
            rs[1] += s[j][1] + s[j][3];
        }
        lsum[0] = lsum[0] * al[0] + rs[0];          // this lane's share of the keys; summed over lanes at the end
        lsum[1] = lsum[1] * al[1] + rs[1];
        if (__any_sync(0xffffffffu, al[0] != 1.f || al[1] != 1.f)) {       // the maxima seldom move after the first tiles
#pragma unroll
            for (int j = 0; j < DT; ++j) { o[j][0] *= al[0]; o[j][1] *= al[1]; o[j][2] *= al[0]; o[j][3] *= al[1]; }
        }
        // ---- O^T += V^T P^T
#pragma unroll
        for (int j = 0; j < KB; ++j) {
            const uint32_t b0 = movmatrix_trans(pack_bf16(s[j][0], s[j][1]));     // keys 0-7 of the block
            const uint32_t b1 = movmatrix_trans(pack_bf16(s[j][2], s[j][3]));     // keys 8-15
#pragma unroll
            for (int dp = 0; dp < DT; ++dp) {
                const int row = j * 16 + v_row;
                uint32_t a0, a1, a2, a3;
                ldsm_x4_t(smem_u32(sv + row * (HD * 2) + (((dp * 2 + v_ch) ^ (row & 7)) << 4)), a0, a1, a2, a3);
                mma_bf16(o[dp], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncwarp();                              // the stage may be overwritten from here on
    }
    pdl_launch_dependents();
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        lsum[x] += __shfl_xor_sync(0xffffffffu, lsum[x], 4);
        lsum[x] += __shfl_xor_sync(0xffffffffu, lsum[x], 8);
        lsum[x] += __shfl_xor_sync(0xffffffffu, lsum[x], 16);
    }
    if (p.split_keys > 0) {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            if (rowc[x] >= p.part_rows) continue;
            float* po = p.part_o + (part_base + rowc[x]) * HD;
#pragma unroll
            for (int dp = 0; dp < DT; ++dp) { po[16 * dp + g] = o[dp][x]; po[16 * dp + 8 + g] = o[dp][2 + x]; }
            if (g == 0) {
                p.part_ml[(part_base + rowc[x]) * 2] = mx[x];
                p.part_ml[(part_base + rowc[x]) * 2 + 1] = validc[x] ? lsum[x] : 0.f;
            }
        }
    } else {
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            if (!validc[x]) continue;
            const float inv = lsum[x] > 0.f ? 1.0f / lsum[x] : 0.f;
            bf16* po = p.out + ((size_t)(tok0 + tlc[x]) * p.H + head0 + hlc[x]) * HD;
#pragma unroll
            for (int dp = 0; dp < DT; ++dp) {
                po[16 * dp + g] = from_f<bf16>(o[dp][x] * inv);
                po[16 * dp + 8 + g] = from_f<bf16>(o[dp][2 + x] * inv);
            }
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(HD) paged_flash_combine_kernel(const FlashParams p, int n_splits) {
    extern __shared__ float wgt[];               // [n_splits] m, then the weight, of each split; [n_splits] l
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, R = blockIdx.z;
    const int req = p.tile_req[tile], tok0 = p.tile_tok0[tile];
    const int nt = min(p.TT, p.cu_q[req + 1] - tok0);
    const int grp = p.H / p.K;
    const int kvh = blockIdx.y / p.head_chunks, hc = blockIdx.y % p.head_chunks;
    const int head0 = kvh * grp + hc * p.GH;
    const int nh = min(p.GH, grp - hc * p.GH);
    const int tl = R / p.GH, hl = R % p.GH;
    if (tl >= nt || hl >= nh) return;
    const int d = threadIdx.x;
    const size_t base = ((size_t)tile * gridDim.y + blockIdx.y) * n_splits;
    // The splits' (m, l) are read side by side, one per thread, not one after the other: the kernel is
    // a chain of memory round trips, so their number is what it costs.  Then the weights
    // exp2(m_z - M) * [l_z > 0] and their sum go to shared memory, and every thread adds its column
    // of the partial outputs in split order with all loads in flight at once.
    __shared__ float red[HD / 32];
    float m_loc = -INFINITY;
    for (int z = d; z < n_splits; z += HD) {
        const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + ((base + z) * p.part_rows + R) * 2);
        wgt[z] = ml.x;
        wgt[n_splits + z] = ml.y;
        if (ml.y > 0.f) m_loc = fmaxf(m_loc, ml.x);
    }
    m_loc = warp_max(m_loc);
    if ((d & 31) == 0) red[d >> 5] = m_loc;
    __syncthreads();
    float M = red[0];
#pragma unroll
    for (int w = 1; w < HD / 32; ++w) M = fmaxf(M, red[w]);
    for (int z = d; z < n_splits; z += HD) {
        const float l = wgt[n_splits + z];
        wgt[z] = l > 0.f ? exp2f(wgt[z] - M) : 0.f;
    }
    __syncthreads();
    float num = 0.f, den = 0.f;
    const float* po = p.part_o + (base * p.part_rows + R) * HD + d;
    const size_t zstride = (size_t)p.part_rows * HD;
    int z = 0;
    for (; z + 4 <= n_splits; z += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = po[(z + u) * zstride];      // a split without keys wrote nothing: the value is dropped below
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float w = wgt[z + u];
            if (w > 0.f) { num += v[u] * w; den += wgt[n_splits + z + u] * w; }
        }
    }
    for (; z < n_splits; ++z) {
        const float w = wgt[z];
        if (w > 0.f) { num += po[z * zstride] * w; den += wgt[n_splits + z] * w; }
    }
    p.out[((size_t)(tok0 + tl) * p.H + head0 + hl) * HD + d] = from_f<bf16>(den > 0.f ? num / den : 0.f);
}

template <int HD>
static int launch_flash(const FlashParams& p, int mode, int n_tiles, int n_splits, cudaStream_t stream) {
    dim3 grid(n_tiles, p.K * p.head_chunks, mode == 0 ? 1 : n_splits);
    if (mode == 0) {
        constexpr int NW = 4, BN = 64;
        const int smem = 2 * 2 * BN * HD * 2;
        auto kern = paged_flash_attention_kernel<HD, NW, BN>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        return rllm_launch(kern, grid, dim3(NW * 32), smem, stream, p);
    }
    // decode shape: one warp per CTA, the keys-as-M kernel for tiles of at most 8 rows, else the 16-row
    // instance of the template with a ring of two 32-key tiles.  (A 4-warp variant that split a CTA's
    // keys and requested them all at once was faster at batch 1 until the 8-row kernel asked for its
    // first tiles before the dependency wait: 11.3 against 10.6 us; it is gone.)
    int st;
    if (p.part_rows <= 8) {
        // tiles of at most 8 query rows: the keys as the M side of the MMA.  Tiles of 16 keys in a ring
        // of three (24 KB): nine CTAs share an SM, which counts for more here than a deeper ring
        // (measured at batch 8 and 64, context 2,048: 32-key tiles x 2 stages 24.8 / 109 us,
        // 16 x 3: 21.0 / 104, 16 x 4: 25.6 / 112, 32 x 4: 30.8 / 166).
        constexpr int BN = 16, NS = 3;
        st = rllm_launch(paged_decode_attention_kernel<HD, BN, NS>, grid, dim3(32), NS * 2 * BN * HD * 2, stream, p);
    } else {
        constexpr int BN = 32;
        st = rllm_launch(paged_flash_attention_kernel<HD, 1, BN>, grid, dim3(32), 2 * 2 * BN * HD * 2, stream, p);
    }
    if (st) return st;
    return rllm_launch(paged_flash_combine_kernel<HD>, dim3(n_tiles, p.K * p.head_chunks, p.part_rows), dim3(HD),
                       2 * n_splits * sizeof(float), stream, p, n_splits);
}

// mode 0: prefill shape (64-row tiles, no split; part_* unused).  mode 1: decode shape (16-row tiles,
// n_splits splits of split_keys keys; part_o needs tiles*K*head_chunks*n_splits*part_rows*hd floats,
// part_ml the same with 2 in place of hd).  TT * GH must not exceed the tile's rows; split_keys must be
// a multiple of 32.  Returns cudaErrorInvalidValue for a
// head size other than 64 or 128.
RLLM_API int rllm_paged_flash_attention(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        float* part_o, float* part_ml, const int* positions, const int* cu_q,
                                        const int* block_table, int table_stride, const int* tile_req,
                                        const int* tile_tok0, int n_tiles, int H, int K, int hd, int bs,
                                        float scale, int window, int mode, int TT, int GH, int head_chunks,
                                        int split_keys, int n_splits, long long n_pages, int* err,
                                        cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    const int rows = mode == 0 ? 64 : 16;
    if (K <= 0 || H % K || TT <= 0 || GH <= 0 || TT * GH > rows || head_chunks * GH < H / K || bs <= 0)
        return (int)cudaErrorInvalidValue;
    if (mode == 1 && (split_keys <= 0 || split_keys % 32 || n_splits <= 0 || !part_o || !part_ml))
        return (int)cudaErrorInvalidValue;
    FlashParams p;
    p.q = (const bf16*)q; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache; p.out = (bf16*)out;
    p.part_o = part_o; p.part_ml = part_ml; p.positions = positions; p.cu_q = cu_q; p.block_table = block_table;
    p.tile_req = tile_req; p.tile_tok0 = tile_tok0; p.table_stride = table_stride;
    p.n_pages = (int)(n_pages > 0x7fffffffLL ? 0x7fffffffLL : n_pages); p.err = err;
    p.H = H; p.K = K; p.bs = bs; p.window = window; p.TT = TT; p.GH = GH; p.head_chunks = head_chunks;
    p.split_keys = mode == 0 ? 0 : split_keys; p.part_rows = TT * GH;
    p.scale_log2 = scale * 1.4426950408889634f;
    if (hd == 128) return launch_flash<128>(p, mode, n_tiles, n_splits, stream);
    if (hd == 64) return launch_flash<64>(p, mode, n_tiles, n_splits, stream);
    return (int)cudaErrorInvalidValue;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free entry point for callers that cannot allocate device memory (see
// attention_flash_static.h for who they are and for the rules of use).  The partials of the decode
// shape live in the file-scope array below instead of caller-provided scratch.
#include "attention_flash_static.h"
#include <stdio.h>

// [rows][128 + 2] floats: per row the unnormalized output (head size <= 128) and (max, sum).
static __device__ __align__(256) float g_static_scratch[(size_t)RLLM_FLASH_STATIC_SCRATCH_ROWS * (128 + 2)];

#define RLLM_STATIC_MAX_DEVICES 64
// Device address of g_static_scratch per device.  In host code the array's name is only a handle
// for the runtime, never a pointer a kernel could use: the address comes from cudaGetSymbolAddress.
static float* g_static_scratch_addr[RLLM_STATIC_MAX_DEVICES];
static thread_local char g_static_error[256] = "";

RLLM_API const char* rllm_paged_flash_decode_static_error(void) { return g_static_error; }

RLLM_API int rllm_paged_flash_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                            const int* positions, const int* cu_q, const int* block_table,
                                            int table_stride, const int* tile_req, const int* tile_tok0,
                                            int n_tiles, int H, int K, int hd, int bs, float scale, int window,
                                            int TT, int GH, int head_chunks, int split_keys, int n_splits,
                                            cudaStream_t stream) {
    g_static_error[0] = 0;
    if (n_tiles <= 0) return 0;
    if (K <= 0 || head_chunks <= 0 || n_splits <= 0 || TT <= 0 || GH <= 0) return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tiles * K * head_chunks * n_splits * TT * GH;
    if (rows > RLLM_FLASH_STATIC_SCRATCH_ROWS || hd > 128) {
        snprintf(g_static_error, sizeof g_static_error,
                 "rllm_paged_flash_decode_static: %lld partial rows of head size %d requested "
                 "(tiles %d x kv heads %d x head chunks %d x splits %d x rows %d); the static scratch holds "
                 "%d rows of head size <= 128",
                 rows, hd, n_tiles, K, head_chunks, n_splits, TT * GH, RLLM_FLASH_STATIC_SCRATCH_ROWS);
        return RLLM_FLASH_STATIC_TOO_LARGE;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= RLLM_STATIC_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (!g_static_scratch_addr[dev]) {
        // set-up, once per device, with that device current
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_addr[dev] = ptr;
    }
    float* part_o = g_static_scratch_addr[dev];
    float* part_ml = part_o + (size_t)RLLM_FLASH_STATIC_SCRATCH_ROWS * 128;
    return rllm_paged_flash_attention(q, k_cache, v_cache, out, part_o, part_ml, positions, cu_q, block_table,
                                      table_stride, tile_req, tile_tok0, n_tiles, H, K, hd, bs, scale, window,
                                      /*mode=*/1, TT, GH, head_chunks, split_keys, n_splits,
                                      /*n_pages: the caller vouches for its table*/ 0x7fffffffLL, /*err=*/nullptr, stream);
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_paged_flash_attention)
