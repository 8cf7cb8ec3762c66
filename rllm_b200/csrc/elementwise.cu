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
// out[t, :] = table[tokens[t], :] as float32.  A token id outside [0, vocab) sets
// *err and reads row 0 (the host checks ids before launch; this is the backstop).
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d, int vocab, int* err) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0 && err) atomicExch(err, 1);
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
__global__ void add_rms_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                    const int* __restrict__ rows, const float* __restrict__ w,
                                    TO* __restrict__ out, int d, float eps, int write_x) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();

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

RLLM_API int rllm_add_rms_norm(float* x, const void* delta, int delta_dtype, const int* rows,
                               const float* w, void* out, int out_dtype, int n_rows, int d,
                               float eps, int write_x, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    int threads = 32;
    while (threads < d / 4 && threads < 1024) threads <<= 1;
#define LAUNCH(TD, TO)                                                                           \
    return rllm_launch(add_rms_norm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream, x,    \
                       (const TD*)delta, rows, w, (TO*)out, d, eps, write_x)
    if (delta_dtype == RLLM_F32 && out_dtype == RLLM_F32) LAUNCH(float, float);
    else if (delta_dtype == RLLM_F32 && out_dtype == RLLM_BF16) LAUNCH(float, bf16);
    else if (delta_dtype == RLLM_BF16 && out_dtype == RLLM_F32) LAUNCH(bf16, float);
    else LAUNCH(bf16, bf16);
#undef LAUNCH
}

// Plain residual add x += delta (used after the last layer when no norm follows).
template <typename TD>
__global__ void add_inplace_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
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
__global__ void silu_mul_kernel(const TI* __restrict__ in, TO* __restrict__ out, int F, size_t total) {
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
RLLM_API int rllm_silu_mul(const void* in, int in_dtype, void* out, int out_dtype, int n, int F,
                           cudaStream_t stream) {
    const size_t total = (size_t)n * F;
    if (total == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define LAUNCH(TI, TO) \
    return rllm_launch(silu_mul_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)in, (TO*)out, F, total)
    if (in_dtype == RLLM_F32 && out_dtype == RLLM_F32) LAUNCH(float, float);
    else if (in_dtype == RLLM_F32 && out_dtype == RLLM_BF16) LAUNCH(float, bf16);
    else if (in_dtype == RLLM_BF16 && out_dtype == RLLM_F32) LAUNCH(bf16, float);
    else LAUNCH(bf16, bf16);
#undef LAUNCH
}

// ------------------------------------------------------------------ q/k norm + rotary + paged KV write
// One block per (token, head) over the fused projection row qkv[t] = [q (H*hd) | k (K*hd) | v (K*hd)].
//   q, k heads: optional RMSNorm over the head (weight of hd entries shared by all heads),
//               then rotate-half rotary with angle = position * inv_freq[i] on pairs (i, i+hd/2)
//               (inv_freq has hd/2 entries; a null inv_freq means no rotation);
//   q -> q_out[t, h, :];  k, v -> the paged cache at slot = slots[t]
//   (page = slot / bs, offset = slot % bs, layout [page][kv_head][bs][hd]); slot < 0 writes nothing.
// write_kv == 0 skips the cache (a layer that reads another layer's cache).
template <typename TI, typename TO, typename TC>
__global__ void qk_norm_rope_store_kernel(const TI* __restrict__ qkv, const float* __restrict__ q_norm_w,
                                          const float* __restrict__ k_norm_w,
                                          const float* __restrict__ inv_freq,
                                          const int* __restrict__ positions, const int* __restrict__ slots,
                                          TO* __restrict__ q_out, TC* __restrict__ k_cache,
                                          TC* __restrict__ v_cache, int H, int K, int hd, int bs,
                                          float eps, int write_kv) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();

    const int t = blockIdx.x, hx = blockIdx.y;
    const int half = hd >> 1;
    const int i = threadIdx.x;
    const bool active = i < half;
    const int width = (H + 2 * K) * hd;
    const int kind = hx < H ? 0 : (hx < H + K ? 1 : 2);     // 0 q, 1 k, 2 v
    if (kind != 0 && !write_kv) return;
    const TI* src = qkv + (size_t)t * width + (size_t)hx * hd;
    float a = 0.f, b = 0.f;
    if (active) { a = to_f<TI>(src[i]); b = to_f<TI>(src[i + half]); }
    if (kind != 2) {
        const float* nw = kind == 0 ? q_norm_w : k_norm_w;
        if (nw) {
            const float ss = block_sum(a * a + b * b, red);
            const float rs = 1.0f / sqrtf(ss / (float)hd + eps);
            if (active) { a = a * rs * nw[i]; b = b * rs * nw[i + half]; }
        }
        // rotary over the whole head: pairs (i, i + hd/2)
        if (inv_freq && active) {
            float s, c;
            sincosf((float)positions[t] * inv_freq[i], &s, &c);
            const float a2 = a * c - b * s, b2 = a * s + b * c;
            a = a2; b = b2;
        }
    }
    if (!active) return;
    if (kind == 0) {
        TO* dst = q_out + ((size_t)t * H + hx) * hd;
        dst[i] = from_f<TO>(a);
        dst[i + half] = from_f<TO>(b);
    } else {
        const int slot = slots[t];
        if (slot < 0) return;
        const int kvh = kind == 1 ? hx - H : hx - H - K;
        TC* base = kind == 1 ? k_cache : v_cache;
        TC* dst = base + (((size_t)(slot / bs) * K + kvh) * bs + (slot % bs)) * hd;
        dst[i] = from_f<TC>(a);
        dst[i + half] = from_f<TC>(b);
    }
}

RLLM_API int rllm_qk_norm_rope_store(const void* qkv, int in_dtype, const float* q_norm_w,
                                     const float* k_norm_w, const float* inv_freq,
                                     const int* positions, const int* slots, void* q_out, int q_dtype,
                                     void* k_cache, void* v_cache, int cache_dtype, int n, int H, int K,
                                     int hd, int bs, float eps, int write_kv, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hd % 2 != 0 || hd > 2048) return (int)cudaErrorInvalidValue;
    const int threads = ((hd / 2 + 31) / 32) * 32;
    dim3 grid(n, H + 2 * K);
#define LAUNCH(TI, TO, TC)                                                                        \
    return rllm_launch(qk_norm_rope_store_kernel<TI, TO, TC>, grid, dim3(threads), 0, stream,     \
                       (const TI*)qkv, q_norm_w, k_norm_w, inv_freq, positions, slots, (TO*)q_out, \
                       (TC*)k_cache, (TC*)v_cache, H, K, hd, bs, eps, write_kv)
    if (q_dtype != cache_dtype) return (int)cudaErrorInvalidValue;
    if (in_dtype == RLLM_F32 && q_dtype == RLLM_F32) LAUNCH(float, float, float);
    else if (in_dtype == RLLM_F32 && q_dtype == RLLM_BF16) LAUNCH(float, bf16, bf16);
    else if (in_dtype == RLLM_BF16 && q_dtype == RLLM_BF16) LAUNCH(bf16, bf16, bf16);
    else LAUNCH(bf16, float, float);
#undef LAUNCH
}
