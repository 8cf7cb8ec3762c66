// Embedding gather, residual-add + RMSNorm (with optional row gather), SwiGLU
// activation, and the fused per-head q/k RMSNorm + NeoX rotary + paged K/V write.
// All arithmetic is float32 whatever the storage type; no fast-math intrinsics.
//
// Counterparts in AxiomOperator/rllm: crates/rllm-cuda/kernels/kernels.cu
// embed_* (670-692), rms_norm / add_rms_norm (771-820), silu_mul (1212-1219),
// qkv_norm_rope_store (1108-1186).  The formulas follow its CPU backend
// (crates/rllm-cpu/src/lib.rs:190-298).
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = table[tokens[t], :] as float32.  A token id outside [0, vocab) writes code 4 to
// *err (the error word that the entry points read) and reads row 0; the host checks ids before
// launch, this is the backstop.
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d, int vocab, int* err) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0 && err) atomicExch(err, 4);
        tok = 0;
    }
    const TW* src = table + (size_t)tok * d;
    float* dst = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f<TW>(src[i]);
}

RLLM_API int rllm_embed(const void* table, int table_dtype, const int* tokens, float* out, int n,
                        int d, int vocab, int* err, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == RLLM_F32)
        return rllm_launch(embed_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)table, tokens, out, d, vocab, err);
    return rllm_launch(embed_kernel<bf16>, dim3(n), dim3(threads), 0, stream, (const bf16*)table, tokens, out, d, vocab, err);
}

// ------------------------------------------------------------------ add + RMSNorm
// For output row r: src = rows ? rows[r] : r; v = x[src] (+ delta[src]);
// if write_x the sum is stored back to x[src] (the residual stream);
// out[r] = v * (1/sqrt(mean(v^2) + eps)) * w.   x is the float32 residual stream.
template <typename TD, typename TO>
__global__ void add_rms_norm_kernel(float* x, const TD* delta,
                                    const int* __restrict__ rows, const float* __restrict__ w,
                                    TO* __restrict__ out, int d, float eps, int write_x) {
    __shared__ float red[33];
    pdl_launch_dependents();          // the product that follows fetches its first weights beside this kernel
    pdl_wait();

    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v += to_f<TD>(dr[i]);
            if (write_x) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i];
        if (dr && !write_x) v += to_f<TD>(dr[i]);
        o[i] = from_f<TO>(v * rs * w[i]);
    }
}

template <typename T> __device__ __forceinline__ float2 load2(const T* p);
template <> __device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load2<bf16>(const bf16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void store2(T* p, float a, float b);
template <> __device__ __forceinline__ void store2<float>(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <> __device__ __forceinline__ void store2<bf16>(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// Same operation for d a multiple of 4 and at most 256 * 4 * NV: one pass over global memory, the row
// lives in registers between the sum of squares and the scaling (float4 loads, 256 threads a row).
template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(256)
add_rms_norm_vec_kernel(float* x, const TD* delta, const int* __restrict__ rows,
                        const float* __restrict__ w, TO* __restrict__ out, int d, float eps, int write_x) {
    __shared__ float red[33];
    pdl_launch_dependents();          // as above
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int i = (it * 256 + threadIdx.x) * 4;
        v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < d) {
            v[it] = *reinterpret_cast<const float4*>(xr + i);
            if (dr) {
                v[it].x += to_f<TD>(dr[i]); v[it].y += to_f<TD>(dr[i + 1]);
                v[it].z += to_f<TD>(dr[i + 2]); v[it].w += to_f<TD>(dr[i + 3]);
                if (write_x) *reinterpret_cast<float4*>(xr + i) = v[it];
            }
            ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
        }
    }
    ss = block_sum(ss, red);
    const float rs = 1.0f / sqrtf(ss / (float)d + eps);
    TO* o = out + (size_t)r * d;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
        const int i = (it * 256 + threadIdx.x) * 4;
        if (i < d) {
            const float4 ww = *reinterpret_cast<const float4*>(w + i);
            store2<TO>(o + i, v[it].x * rs * ww.x, v[it].y * rs * ww.y);
            store2<TO>(o + i + 2, v[it].z * rs * ww.z, v[it].w * rs * ww.w);
        }
    }
}

template <typename TD, typename TO>
static int launch_norm(float* x, const void* delta, const int* rows, const float* w, void* out, int n_rows, int d,
                       float eps, int write_x, cudaStream_t stream) {
    const bool vec = d % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
#define VEC(NV)                                                                                        \
    return rllm_launch(add_rms_norm_vec_kernel<TD, TO, NV>, dim3(n_rows), dim3(256), 0, stream, x,     \
                       (const TD*)delta, rows, w, (TO*)out, d, eps, write_x)
    if (vec && d <= 1024) VEC(1);
    if (vec && d <= 2048) VEC(2);
    if (vec && d <= 4096) VEC(4);
    if (vec && d <= 8192) VEC(8);
#undef VEC
    int threads = 32;
    while (threads < d / 4 && threads < 1024) threads <<= 1;
    return rllm_launch(add_rms_norm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream, x, (const TD*)delta,
                       rows, w, (TO*)out, d, eps, write_x);
}

RLLM_API int rllm_add_rms_norm(float* x, const void* delta, int delta_dtype, const int* rows,
                               const float* w, void* out, int out_dtype, int n_rows, int d,
                               float eps, int write_x, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (delta_dtype == RLLM_F32 && out_dtype == RLLM_F32)
        return launch_norm<float, float>(x, delta, rows, w, out, n_rows, d, eps, write_x, stream);
    if (delta_dtype == RLLM_F32 && out_dtype == RLLM_BF16)
        return launch_norm<float, bf16>(x, delta, rows, w, out, n_rows, d, eps, write_x, stream);
    if (delta_dtype == RLLM_BF16 && out_dtype == RLLM_F32)
        return launch_norm<bf16, float>(x, delta, rows, w, out, n_rows, d, eps, write_x, stream);
    return launch_norm<bf16, bf16>(x, delta, rows, w, out, n_rows, d, eps, write_x, stream);
}

// Plain residual add x += delta (used after the last layer when no norm follows).
template <typename TD>
__global__ void add_inplace_kernel(float* x, const TD* delta, size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_f<TD>(delta[i]);
}
RLLM_API int rllm_add_inplace(float* x, const void* delta, int delta_dtype, long long n,
                              cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (delta_dtype == RLLM_F32)
        return rllm_launch(add_inplace_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x, (const float*)delta, (size_t)n);
    return rllm_launch(add_inplace_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, x, (const bf16*)delta, (size_t)n);
}

// ------------------------------------------------------------------ SwiGLU
// in [n, 2F] holds gate in columns [0,F) and up in [F,2F); out[t,j] = gate/(1+exp(-gate)) * up.
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* in, TO* out, int F, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / F;
    const int j = (int)(i - t * F);
    const float g = to_f<TI>(in[t * 2 * F + j]);
    const float u = to_f<TI>(in[t * 2 * F + F + j]);
    out[i] = from_f<TO>(g / (1.0f + expf(-g)) * u);
}
template <typename TI, typename TO>
__global__ void silu_mul_vec2_kernel(const TI* in, TO* out, int F, size_t total2) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i2 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // pairs of outputs
    if (i2 >= total2) return;
    const size_t i = i2 * 2;
    const size_t t = i / F;
    const int j = (int)(i - t * F);
    const TI* g = in + t * 2 * F + j;
    const TI* u = g + F;
    const float g0 = to_f<TI>(g[0]), g1 = to_f<TI>(g[1]);
    store2<TO>(out + i, g0 / (1.0f + expf(-g0)) * to_f<TI>(u[0]), g1 / (1.0f + expf(-g1)) * to_f<TI>(u[1]));
}

RLLM_API int rllm_silu_mul(const void* in, int in_dtype, void* out, int out_dtype, int n, int F,
                           cudaStream_t stream) {
    const size_t total = (size_t)n * F;
    if (total == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    const bool vec = F % 2 == 0 && ((uintptr_t)out & 7) == 0;
    const unsigned blocks2 = (unsigned)((total / 2 + threads - 1) / threads);
#define LAUNCH(TI, TO)                                                                                       \
    if (vec)                                                                                                 \
        return rllm_launch(silu_mul_vec2_kernel<TI, TO>, dim3(blocks2), dim3(threads), 0, stream, (const TI*)in, \
                           (TO*)out, F, total / 2);                                                          \
    return rllm_launch(silu_mul_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)in, (TO*)out, F, total)
    if (in_dtype == RLLM_F32 && out_dtype == RLLM_F32) { LAUNCH(float, float); }
    if (in_dtype == RLLM_F32 && out_dtype == RLLM_BF16) { LAUNCH(float, bf16); }
    if (in_dtype == RLLM_BF16 && out_dtype == RLLM_F32) { LAUNCH(bf16, float); }
    LAUNCH(bf16, bf16);
#undef LAUNCH
}

// ------------------------------------------------------------------ q/k norm + rotary + paged KV write
// Over the fused projection row qkv[t] = [q (H*hd) | k (K*hd) | v (K*hd)]:
//   q, k heads: optional RMSNorm over the head (weight of hd entries shared by all heads),
//               then rotate-half rotary on pairs (i, i+hd/2) with the (cos, sin) of the token's angles
//               from cs_table [n, hd/2] (rope_table below: angle = position * inv_freq[i], worked out
//               once per step for all layers; a null table means no rotation);
//   q -> q_out[t, h, :];  k, v -> the paged cache at slot = slots[t]
//   (page = slot / bs, offset = slot % bs, layout [page][kv_head][bs][hd]); slot < 0 writes nothing;
//   a slot beyond the pool (>= n_slots) writes nothing and sets the error word (RLLM_ERR_SLOT).
// write_kv == 0 skips the cache (a layer that reads another layer's cache).
//
// One block per token and group of 8 * HPW heads (head size a multiple of 4, at most 256): each warp
// takes HPW heads (8 apart), a lane holding two neighbouring pairs (j, j + hd/2), (j + 1, j + 1 + hd/2)
// of each so that loads and stores are 8 and 4 bytes wide (U = 1: head sizes up to 128, one unit a
// lane; U = 2: up to 256).  No shared memory, no barrier: the loads of
// all of a warp's heads are in flight at once, and the token's angles are fetched once per lane.  A
// head's arithmetic does not depend on HPW: a decode step (HPW = 1: most blocks, shortest chain) and
// a prompt step (two heads a warp) give the same bits.
template <typename TI, typename TO, typename TC, int HPW, int U>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_token_kernel(const TI* qkv, const float* __restrict__ q_norm_w,
                                const float* __restrict__ k_norm_w, const float2* cs_table,
                                const int* __restrict__ positions, const int* __restrict__ slots,
                                TO* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache, int H,
                                int K, int hd, int bs, float eps, int write_kv, int n_slots, int* err) {
    // The attention kernel that follows may start at once: before its own wait (which ends when this
    // grid has completed, and so the product before it) it reads only the step's index arrays and
    // keys of earlier steps, and that part of it then runs beside this kernel and the end of the one before.
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_heads = write_kv ? H + 2 * K : H;
    const size_t width = (size_t)(H + 2 * K) * hd;
    const int units = half >> 1;                  // float2 units per half head
    // this warp's heads are asked for first: their values arrive while the rest is worked out
    float a[HPW][U][2], b[HPW][U][2];
    float2 cs[U][2];                              // (cos, sin) of this lane's pairs
#pragma unroll
    for (int u = 0; u < U; ++u) {
        cs[u][0] = cs[u][1] = make_float2(1.f, 0.f);
        if (cs_table != nullptr && lane + 32 * u < units) {
            const float4 c4 = *reinterpret_cast<const float4*>(cs_table + (size_t)t * half + (lane + 32 * u) * 2);
            cs[u][0] = make_float2(c4.x, c4.y);
            cs[u][1] = make_float2(c4.z, c4.w);
        }
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int hx = (blockIdx.y * HPW + i) * 8 + warp;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            a[i][u][0] = a[i][u][1] = b[i][u][0] = b[i][u][1] = 0.f;
            if (hx < n_heads && lane + 32 * u < units) {
                const TI* src = qkv + (size_t)t * width + (size_t)hx * hd + (lane + 32 * u) * 2;
                const float2 lo = load2<TI>(src), hi = load2<TI>(src + half);
                a[i][u][0] = lo.x; a[i][u][1] = lo.y;
                b[i][u][0] = hi.x; b[i][u][1] = hi.y;
            }
        }
    }
    int slot = slots[t];
    if (slot >= n_slots) {
        if (tid == 0 && blockIdx.y == 0 && err) atomicExch(err, RLLM_ERR_SLOT);
        slot = -1;
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int hx = (blockIdx.y * HPW + i) * 8 + warp;
        if (hx >= n_heads) continue;              // warp-uniform
        const int kind = hx < H ? 0 : (hx < H + K ? 1 : 2);
        TO* qdst = nullptr;
        TC* cdst = nullptr;
        if (kind == 0) {
            qdst = q_out + ((size_t)t * H + hx) * hd;
        } else if (slot >= 0) {
            const int kvh = kind == 1 ? hx - H : hx - H - K;
            cdst = (kind == 1 ? k_cache : v_cache) + (((size_t)(slot / bs) * K + kvh) * bs + (slot % bs)) * hd;
        }
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u)
            ss += a[i][u][0] * a[i][u][0] + a[i][u][1] * a[i][u][1] + b[i][u][0] * b[i][u][0] + b[i][u][1] * b[i][u][1];
        const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
        float rs = 1.f;
        if (nw) rs = 1.0f / sqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = (lane + 32 * u) * 2;
            if (lane + 32 * u < units) {
                float o[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float av = a[i][u][e], bv = b[i][u][e];
                    if (nw) { av = av * rs * nw[j + e]; bv = bv * rs * nw[j + e + half]; }
                    if (kind != 2) {
                        const float2 c = cs[u][e];
                        const float a2 = av * c.x - bv * c.y, b2 = av * c.y + bv * c.x;
                        av = a2; bv = b2;
                    }
                    o[e] = av; o[2 + e] = bv;
                }
                if (qdst) { store2<TO>(qdst + j, o[0], o[1]); store2<TO>(qdst + j + half, o[2], o[3]); }
                if (cdst) { store2<TC>(cdst + j, o[0], o[1]); store2<TC>(cdst + j + half, o[2], o[3]); }
            }
        }
    }
}

// cs_table[t, i] = (cos, sin) of position[t] * inv_freq[i], float32, accurate sincosf: the angles of
// a step's tokens, worked out once for all layers that share a rotary table.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ out, int half, int total) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float sn, c;
    sincosf((float)positions[i / half] * inv_freq[i % half], &sn, &c);
    out[i] = make_float2(c, sn);
}

RLLM_API int rllm_rope_table(const int* positions, const float* inv_freq, void* out, int n, int half,
                             cudaStream_t stream) {
    if (n <= 0 || half <= 0) return 0;
    const int total = n * half;
    return rllm_launch(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, positions, inv_freq,
                       (float2*)out, half, total);
}

RLLM_API int rllm_qk_norm_rope_store(const void* qkv, int in_dtype, const float* q_norm_w,
                                     const float* k_norm_w, const void* cs_table,
                                     const int* positions, const int* slots, void* q_out, int q_dtype,
                                     void* k_cache, void* v_cache, int cache_dtype, int n, int H, int K,
                                     int hd, int bs, float eps, int write_kv, long long n_slots, int* err,
                                     cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hd % 4 != 0 || hd > 256 || ((uintptr_t)qkv & 7) || ((uintptr_t)q_out & 7) || ((uintptr_t)k_cache & 7) ||
        ((uintptr_t)v_cache & 7) || ((uintptr_t)cs_table & 15))
        return (int)cudaErrorInvalidValue;
    // heads per warp: one for the few tokens of a decode step (most blocks, shortest chain), two for a
    // prompt step (2,048 tokens of 48 heads, back to back over inputs larger than L2: 22.7 us with one,
    // 20.1 with two, 22.8 with four, 22.6 with six; 11.5 at the copy peak)
    const int n_heads = write_kv ? H + 2 * K : H;
    const int hpw = n > 64 ? 2 : 1;
    const dim3 grid(n, (n_heads + 8 * hpw - 1) / (8 * hpw));
#define LAUNCH_H(TI, TO, TC, HPW)                                                                     \
    do {                                                                                              \
        if (hd <= 128)                                                                                \
            return rllm_launch(qk_norm_rope_store_token_kernel<TI, TO, TC, HPW, 1>, grid, dim3(256), 0, stream,      \
                               (const TI*)qkv, q_norm_w, k_norm_w, (const float2*)cs_table, positions, slots,        \
                               (TO*)q_out, (TC*)k_cache, (TC*)v_cache, H, K, hd, bs, eps, write_kv,   \
                               (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots), err);          \
        return rllm_launch(qk_norm_rope_store_token_kernel<TI, TO, TC, HPW, 2>, grid, dim3(256), 0, stream,          \
                           (const TI*)qkv, q_norm_w, k_norm_w, (const float2*)cs_table, positions, slots,            \
                           (TO*)q_out, (TC*)k_cache, (TC*)v_cache, H, K, hd, bs, eps, write_kv,       \
                           (int)(n_slots > 0x7fffffffLL ? 0x7fffffffLL : n_slots), err);              \
    } while (0)
#define LAUNCH(TI, TO, TC)                                                                            \
    do {                                                                                              \
        if (hpw == 1) { LAUNCH_H(TI, TO, TC, 1); }                                                    \
        LAUNCH_H(TI, TO, TC, 2);                                                                      \
    } while (0)
    if (q_dtype != cache_dtype) return (int)cudaErrorInvalidValue;
    if (in_dtype == RLLM_F32 && q_dtype == RLLM_F32) { LAUNCH(float, float, float); }
    if (in_dtype == RLLM_F32 && q_dtype == RLLM_BF16) { LAUNCH(float, bf16, bf16); }
    if (in_dtype == RLLM_BF16 && q_dtype == RLLM_BF16) { LAUNCH(bf16, bf16, bf16); }
    LAUNCH(bf16, float, float);
#undef LAUNCH
#undef LAUNCH_H
}

// the packed-argument forms (common.cuh) for the host runtime's replay of recorded launches
RLLM_PACKED(rllm_embed)
RLLM_PACKED(rllm_add_rms_norm)
RLLM_PACKED(rllm_add_inplace)
RLLM_PACKED(rllm_silu_mul)
RLLM_PACKED(rllm_rope_table)
RLLM_PACKED(rllm_qk_norm_rope_store)
