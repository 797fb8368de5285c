// See attention_mma_static.h.  The kernel is the one of attention_mma.cu, unchanged; only
// where its scratch memory comes from differs.
#include "attention_mma.cu"
#include "attention_mma_static.h"

#include <stdio.h>

#define LLS_MAX_DEVICES 64
#define LLS_SCRATCH_FLOATS (LL_ATTN_STATIC_SCRATCH_BYTES / (long)sizeof(float))

// Device memory that comes with the library.  In host code these names are only handles
// for cudaGetSymbolAddress; the kernel gets the addresses looked up below.
static __device__ __align__(256) float lls_scratch[LLS_SCRATCH_FLOATS];
static __device__ __align__(256) int lls_counters[LL_ATTN_STATIC_COUNTERS];

static float* lls_scratch_addr[LLS_MAX_DEVICES];
static int* lls_counters_addr[LLS_MAX_DEVICES];
static thread_local char lls_error[256];

extern "C" const char* ll_attn_mma_static_error(void) { return lls_error; }

// Once per device, with that device current: the device addresses of the two arrays.
static int lls_setup(int device) {
  if (lls_scratch_addr[device] != nullptr && lls_counters_addr[device] != nullptr) return 0;
  float* s = nullptr;
  int* c = nullptr;
  cudaError_t err = cudaGetSymbolAddress((void**)&s, lls_scratch);
  if (err == cudaSuccess) err = cudaGetSymbolAddress((void**)&c, lls_counters);
  if (err != cudaSuccess) {
    snprintf(lls_error, sizeof(lls_error), "ll_attn_mma_static: cudaGetSymbolAddress failed on device %d: %s", device,
             cudaGetErrorString(err));
    return (int)err;
  }
  lls_scratch_addr[device] = s;
  lls_counters_addr[device] = c;
  return 0;
}

extern "C" int ll_attn_mma_static(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                                  const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                                  const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh,
                                  int nkv, int hd, int page_size, int num_pages, int window, float scale, int nsplit,
                                  int* status, cudaStream_t stream) {
  lls_error[0] = 0;
  if (row_blocks <= 0 || n_entries <= 0) return 0;
  if (nkv <= 0 || nsplit < 1 || hd <= 0) {
    snprintf(lls_error, sizeof(lls_error), "ll_attn_mma_static: nkv, nsplit and hd must be positive");
    return (int)cudaErrorInvalidValue;
  }
  const long need_floats = ll_attn_mma_scratch_floats(row_blocks, nkv, nsplit, hd);
  const long need_counters = (long)row_blocks * nkv;
  if (need_floats > LLS_SCRATCH_FLOATS || need_counters > LL_ATTN_STATIC_COUNTERS) {
    snprintf(lls_error, sizeof(lls_error),
             "ll_attn_mma_static: this launch needs %ld scratch floats and %ld counters; the built-in array holds "
             "%ld and %d (use ll_attn_mma with scratch of your own, or fewer splits)",
             need_floats, need_counters, (long)LLS_SCRATCH_FLOATS, LL_ATTN_STATIC_COUNTERS);
    return LL_ATTN_STATIC_TOO_LARGE;
  }
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= LLS_MAX_DEVICES) {
    snprintf(lls_error, sizeof(lls_error), "ll_attn_mma_static: no usable current device (%d)", device);
    return err != cudaSuccess ? (int)err : (int)cudaErrorInvalidDevice;
  }
  const int rc = lls_setup(device);
  if (rc != 0) return rc;
  // the counters must be zero when the kernel starts; whatever an earlier call left is cleared here
  err = cudaMemsetAsync(lls_counters_addr[device], 0, sizeof(int) * (size_t)need_counters, stream);
  if (err != cudaSuccess) {
    snprintf(lls_error, sizeof(lls_error), "ll_attn_mma_static: clearing the counters failed: %s",
             cudaGetErrorString(err));
    return (int)err;
  }
  return ll_attn_mma(out, out_stride, q, q_stride, k_cache, v_cache, block_table, bt_stride, cu_q, ctx_len, req_slot,
                     n_entries, row_blocks, nh, nkv, hd, page_size, num_pages, window, scale, nsplit,
                     lls_scratch_addr[device], lls_counters_addr[device], status, stream);
}
