// RMSNorm, alone and fused with the residual sum.
//
//   y = x / sqrt(mean(x^2) + eps) * w          (w is float32 whatever T is)
//
// The fused form first computes r = residual + delta in float32, rounds r to
// the storage type (that rounded value is both what is written back as the new
// residual and what the norm sees, so fused and unfused runs agree bit for
// bit), then normalises.  With `rows` given only those rows are read and
// nothing is written back (the last norm before the logits).
//
// One block per row; the row is kept in shared memory between the two passes.
#include "common.cuh"

template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ w,
                               float eps, int hidden, long x_stride, long out_stride) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int r = blockIdx.x;
  const T* xr = x + (size_t)r * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_f32<T>(xr[i]);
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * out_stride;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(row[i] * inv * w[i]);
}

template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ out, T* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ partial, int parts, long part_stride,
                                   const float* __restrict__ w, float eps, int hidden,
                                   const int* __restrict__ rows, int write_residual) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int i_out = blockIdx.x;
  const int r = rows ? rows[i_out] : i_out;
  T* res = residual + (size_t)r * hidden;
  const T* del = delta ? delta + (size_t)r * hidden : nullptr;
  const float* par = partial ? partial + (size_t)r * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32<T>(res[i]);
    if (del) {
      v = round_to<T>(v + to_f32<T>(del[i]));
      if (write_residual) res[i] = from_f32<T>(v);
    } else if (par) {
      // delta arrives as float32 partial sums of a product split over k: add the parts, round the
      // sum to the storage type as the unsplit product would have been, then add it
      float d = 0.f;
      for (int q = 0; q < parts; ++q) d += par[(size_t)q * part_stride + i];
      v = round_to<T>(v + round_to<T>(d));
      if (write_residual) res[i] = from_f32<T>(v);
    }
    row[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)i_out * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(row[i] * inv * w[i]);
}

static int norm_threads(int hidden) {
  int t = 32;
  while (t < 512 && t * 4 < hidden) t <<= 1;
  return t;
}

extern "C" int ll_rmsnorm(int dtype, void* out, const void* x, const float* w, float eps, int rows, int hidden,
                          long x_stride, long out_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(rmsnorm_kernel<T>, dim3(rows), dim3(norm_threads(hidden)), smem, stream, (T*)out, (const T*)x, w, eps,
              hidden, x_stride, out_stride);
  });
  return LL_LAUNCH_RESULT();
}

// out[i] = norm(residual[r] + delta[r]) with r = rows ? rows[i] : i.
// delta may be null (plain norm of residual rows), or given instead as `partial`: float32
// [parts][tokens, hidden] partial sums (part_stride elements apart) that are added up first.
// write_residual stores the rounded sum back into residual (only sensible without `rows`).
extern "C" int ll_add_rmsnorm(int dtype, void* out, void* residual, const void* delta, const float* partial,
                              int parts, long part_stride, const float* w, float eps, int n_out, int hidden,
                              const int* rows, int write_residual, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(add_rmsnorm_kernel<T>, dim3(n_out), dim3(norm_threads(hidden)), smem, stream, (T*)out, (T*)residual,
              (const T*)delta, partial, parts, part_stride, w, eps, hidden, rows, write_residual);
  });
  return LL_LAUNCH_RESULT();
}
