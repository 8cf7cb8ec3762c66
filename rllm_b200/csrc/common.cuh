// Shared device helpers for the sm_100a kernels: element conversion, fixed-order
// reductions and the launch-status convention (every extern "C" launcher returns
// the cudaError_t of its launch as an int; 0 is success).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define RLLM_API extern "C" __attribute__((visibility("default")))

// Codes that kernels write to the error word when a range check refuses an index (the access is then
// skipped or redirected to page 0 and the step's results are not to be used; nothing traps).
enum : int { RLLM_ERR_TOKEN = 4, RLLM_ERR_SLOT = 5, RLLM_ERR_PAGE = 6 };

// Element type codes shared with the Python wrappers.
enum : int { RLLM_F32 = 0, RLLM_BF16 = 1 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum in a fixed order (butterfly inside a warp, then warps in index
// order), so the result does not depend on scheduling.  `red` holds >= 33 floats.
// All threads of the block must call it; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < nw; ++i) t += red[i];
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int i = 1; i < nw; ++i) t = fmaxf(t, red[i]);
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Programmatic dependent launch (griddepcontrol): `pdl_wait` blocks until the kernels this one
// depends on have completed and their writes are visible (a no-op for an ordinary launch);
// `pdl_launch_dependents` lets the next kernel of the stream begin to launch early.  A kernel
// launched with the attribute may only touch memory that earlier kernels write after its wait.
// Pointers to such memory carry no __restrict__ and are never read with __ldg: a read-only load
// (ld.global.nc) is "invariant" to the compiler, which may move it above the wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" :::); }

// Host side: every kernel of this package is launched through rllm_launch.  With the switch on
// (RLLM_B200_PDL=0 in the environment turns it off) kernels carry the programmatic stream
// serialization attribute, so a kernel's launch and its loads of data that no kernel writes
// (weights) overlap the tail of the kernel before it.  Every kernel therefore calls pdl_wait()
// before it reads or writes anything an earlier kernel may have written, and before it exits.
#include <stdlib.h>
static inline int rllm_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("RLLM_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on;
}
template <typename... KArgs, typename... Args>
static inline int rllm_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = rllm_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The same with the CTAs grouped into thread-block clusters of `cluster` CTAs along each dimension.
template <typename... KArgs, typename... Args>
static inline int rllm_launch_clusters(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (rllm_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Clusters of `cluster_y` CTAs along grid dimension y.
template <typename... KArgs, typename... Args>
static inline int rllm_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      int cluster_y, Args... args) {
    return rllm_launch_clusters(kern, grid, block, smem, stream, dim3(1, cluster_y > 1 ? cluster_y : 1, 1), args...);
}

#define RLLM_LAUNCH_STATUS() ((int)cudaGetLastError())

// Every launcher also has a form that takes its arguments packed into 64-bit words, one per argument
// in order (pointers and integers as they are, a float as its 32 bits): `name_packed(words)`.  The
// host runtime replays recorded launches through these without knowing a launcher's signature.
#include <cstring>
#include <utility>
template <typename T> struct RllmWord {
    static T get(unsigned long long w) { return (T)(long long)w; }
};
template <typename T> struct RllmWord<T*> {
    static T* get(unsigned long long w) { return reinterpret_cast<T*>((uintptr_t)w); }
};
template <> struct RllmWord<float> {
    static float get(unsigned long long w) {
        const uint32_t bits = (uint32_t)w;
        float f;
        memcpy(&f, &bits, sizeof f);
        return f;
    }
};
template <typename R, typename... A, size_t... I>
static inline R rllm_call_packed_impl(R (*fn)(A...), const unsigned long long* w, std::index_sequence<I...>) {
    return fn(RllmWord<A>::get(w[I])...);
}
template <typename R, typename... A>
static inline R rllm_call_packed(R (*fn)(A...), const unsigned long long* w) {
    return rllm_call_packed_impl(fn, w, std::index_sequence_for<A...>{});
}
#define RLLM_PACKED(name) \
    RLLM_API int name##_packed(const unsigned long long* w) { return rllm_call_packed(&name, w); }
