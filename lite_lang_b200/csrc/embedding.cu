// Token embedding: out[t, :] = table[ids[t], :].
//
// One block per token; rows are copied in 16-byte pieces when the row size
// allows it.  An id outside [0, vocab) writes a row of zeros and raises
// LL_ERR_TOKEN_RANGE in the status word instead of reading out of bounds.
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(T* __restrict__ out, const T* __restrict__ table,
                                    const int* __restrict__ ids, int hidden, int vocab, int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = (id >= 0 && id < vocab);
  if (!ok && threadIdx.x == 0) set_status(status, LL_ERR_TOKEN_RANGE);
  T* dst = out + (size_t)t * hidden;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  const int row_bytes = hidden * (int)sizeof(T);
  if ((row_bytes & 15) == 0) {
    const int n16 = row_bytes >> 4;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) d4[i] = ok ? s4[i] : make_uint4(0, 0, 0, 0);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : from_f32<T>(0.f);
  }
}

extern "C" int ll_embed_gather(int dtype, void* out, const void* table, const int* ids, int num_tokens,
                               int hidden, int vocab, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(embed_gather_kernel<T>, dim3(num_tokens), dim3(128), 0, stream, (T*)out,
                                     (const T*)table, ids, hidden, vocab, status));
  return LL_LAUNCH_RESULT();
}

// Token ids that are still on the device: ids[i] = results[feed[i]] where feed[i] >= 0.  A decode step that
// is launched before the host has seen the tokens sampled by the step before takes them from that step's
// result buffer this way.  A feed index outside [0, max_results) leaves ids[i] as the host wrote it.
__global__ void feed_tokens_kernel(int* __restrict__ ids, const int* __restrict__ feed, const int* __restrict__ results,
                                   int n, int max_results) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int f = feed[i];
    if (f >= 0 && f < max_results) ids[i] = results[f];
  }
}

extern "C" int ll_feed_tokens(int* ids, const int* feed, const int* results, int n, int max_results,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  ll_launch(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, feed, results, n, max_results);
  return LL_LAUNCH_RESULT();
}
