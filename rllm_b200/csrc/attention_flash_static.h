// Declaration of the allocation-free decode attention entry point (defined at the end of
// attention_flash.cu).  This entry point has no counterpart in AxiomOperator/rllm: its device
// code always gets scratch from its backend's allocator.
//
// Who needs it: a caller that may not allocate device memory at the moment it wants attention.
// Examples are a serving loop that has handed every byte of the GPU to its own pools and treats
// cudaMalloc as a bug (cudaMalloc also synchronizes the whole device, stalling every stream), a
// plain C or C++ host that links this library without torch and therefore has no caching
// allocator to ask, and code running between other libraries' captured or timed regions where
// an allocation would disturb them.  Such a caller passes inputs and outputs only.
//
// The split-key decode kernel needs scratch for its partial results (unnormalized output,
// running maximum and sum per row and split).  Here that scratch is a file-scope
// `static __device__` array inside the library: RLLM_FLASH_STATIC_SCRATCH_ROWS rows of
// (128 + 2) floats = 16.25 MiB, held on every GPU that loads the library until the process ends.
//
// Rules of use:
//  * The very first call on a device looks up the array's device address (cudaGetSymbolAddress,
//    with that device current).  Make that first call outside any stream capture.
//  * A call whose partials do not fit (tiles * kv_heads * head_chunks * n_splits * TT * GH rows
//    above the maximum) is refused: it returns RLLM_FLASH_STATIC_TOO_LARGE, launches nothing,
//    and rllm_paged_flash_decode_static_error() describes the sizes.
//  * All calls share the one array, and it keeps whatever the previous call left.  Nothing in it
//    has to start at zero: every row a call reads was written by that call first.  Two calls that
//    overlap on the GPU (different streams, or graphs replayed concurrently) race on it; order them.
//  * It allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define RLLM_FLASH_STATIC_SCRATCH_ROWS 32768
#define RLLM_FLASH_STATIC_TOO_LARGE 20001

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as rllm_paged_flash_attention in its decode shape (mode 1), without
// the two scratch pointers.  Returns 0, a cudaError_t, or RLLM_FLASH_STATIC_TOO_LARGE.
int rllm_paged_flash_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int* positions, const int* cu_q, const int* block_table,
                                   int table_stride, const int* tile_req, const int* tile_tok0, int n_tiles,
                                   int H, int K, int hd, int bs, float scale, int window, int TT, int GH,
                                   int head_chunks, int split_keys, int n_splits, cudaStream_t stream);

// Text of the last refusal on the calling thread ("" if none).
const char* rllm_paged_flash_decode_static_error(void);

#ifdef __cplusplus
}
#endif
