// ll_attn_mma_static: the tensor-core paged attention with its scratch memory built in.
//
// This entry point has no counterpart in ppppppppig/lite_lang.  It exists for callers
// that must not allocate device memory while they run: a host program that gave all
// free device memory to its own pools at start-up (so a later cudaMalloc would fail or
// stall every stream), or a plug-in inside another runtime whose allocator it cannot
// reach.  The split-key attention kernel needs scratch memory for the partial results of
// its splits and a few counters; ll_attn_mma takes both from the caller, this variant
// keeps them in a fixed array that is part of the loaded library.
//
//   * The array is LL_ATTN_STATIC_SCRATCH_BYTES (8 MiB) of floats plus
//     LL_ATTN_STATIC_COUNTERS counters.  Every GPU on which the library is loaded holds
//     that much memory until the process exits, whether or not the entry point is used.
//   * A launch that would need more (row_blocks * nkv * nsplit * 16 * (hd + 2) floats, or
//     row_blocks * nkv counters) is refused with LL_ATTN_STATIC_TOO_LARGE and nothing is
//     launched; ll_attn_mma_static_error() then says how much was asked for.
//   * The first call on a device looks up the array's device address (once per device,
//     with that device current).  Make that first call outside any stream capture.
//   * All calls share the one array, and it keeps what the last call left in it.  The
//     counters are cleared on the stream before every launch; the partial results are
//     always written before they are read.  Two calls that run at the same time on the
//     GPU (different streams) would race on the array: issue them on one stream, or
//     otherwise keep them from overlapping.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
//
// Arguments are those of ll_attn_mma without `scratch` and `counters`; inputs and outputs
// are still the caller's.  Returns 0, a cudaError_t, or LL_ATTN_STATIC_TOO_LARGE.
#pragma once

#include <cuda_runtime.h>

#define LL_ATTN_STATIC_SCRATCH_BYTES (8l << 20)
#define LL_ATTN_STATIC_COUNTERS 4096
#define LL_ATTN_STATIC_TOO_LARGE 100001

#ifdef __cplusplus
extern "C" {
#endif

int ll_attn_mma_static(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                       const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                       const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh, int nkv,
                       int hd, int page_size, int num_pages, int window, float scale, int nsplit, int* status,
                       cudaStream_t stream);

// Text of the last refusal or set-up failure of ll_attn_mma_static on the calling thread.
const char* ll_attn_mma_static_error(void);

#ifdef __cplusplus
}
#endif
