// Shared device helpers of the lite_lang_b200 kernels (sm_100a).
//
// Every kernel family is one .cu file that exports plain C launchers
// ("extern C", raw pointers, explicit stream).  The element type of
// activations, weights and cache is chosen at run time by `dtype`:
// 0 = float32 (true 32-bit path), 1 = bfloat16.  All arithmetic inside the
// kernels is float32 whatever the storage type is.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LL_DTYPE_F32 0
#define LL_DTYPE_BF16 1

// error codes written to the status word (first error wins)
#define LL_ERR_TOKEN_RANGE 1
#define LL_ERR_SLOT_RANGE 2
#define LL_ERR_PAGE_RANGE 3
#define LL_ERR_POSITION_RANGE 4

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// value after a round trip through the storage type
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

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

// Sum over the block; every thread gets the result.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

#define LL_DISPATCH_DTYPE(dtype, ...)              \
  do {                                             \
    if ((dtype) == LL_DTYPE_F32) {                 \
      using T = float;                             \
      __VA_ARGS__;                                 \
    } else if ((dtype) == LL_DTYPE_BF16) {         \
      using T = bf16;                              \
      __VA_ARGS__;                                 \
    } else {                                       \
      return (int)cudaErrorInvalidValue;           \
    }                                              \
  } while (0)

#define LL_LAUNCH_RESULT() ((int)cudaGetLastError())
