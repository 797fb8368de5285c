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

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this package starts with LL_PDL_WAIT():
// it may be scheduled while the kernel before it on the stream is still running, and
// blocks there until that kernel has finished and its writes are visible.  What a kernel
// does before the wait must not depend on earlier kernels (the weight-streaming product
// starts its TMA copies of the weights there).  LL_PDL_TRIGGER() lets the next kernel be
// scheduled.  Every CTA executes the wait before it exits, so "the kernel before has
// finished" carries over along the whole chain.  Launched without the attribute (grids of
// many waves, or LITE_LANG_B200_PDL=0) both instructions do nothing.
// ---------------------------------------------------------------------------------------
#define LL_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#define LL_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")

// ---------------------------------------------------------------------------------------
// Timeline build (LITE_LANG_B200_TIMELINE=1 when the libraries are built and loaded; off otherwise, and then
// nothing of it is compiled).  Thread 0 of every CTA of the decode step's products and of the decode attention
// writes %globaltimer at three places (the CTA has started, the wait for the kernel before is over, the CTA is
// done) into the words behind the status word: 64-bit slot ((kernel * 512 + CTA) * 4 + event), plain stores that
// nobody waits for.  Later launches of a kernel overwrite earlier ones, so what is read back afterwards is the
// last layer of the last step.  Kernels: 0 q|k|v, 1 decode attention, 2 narrow product to bfloat16 (o), 3 gated,
// 4 narrow product to float32 partial sums (down), 5 wide (logits).
// ---------------------------------------------------------------------------------------
#define LL_TIMELINE_KERNELS 6
#define LL_TIMELINE_CTAS 512
#ifdef LL_TIMELINE
__device__ __forceinline__ void ll_timeline_stamp(int* status, int kernel, int event) {
  if (threadIdx.x == 0 && status != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    if (cta < LL_TIMELINE_CTAS)
      reinterpret_cast<unsigned long long*>(status + 4)[((size_t)kernel * LL_TIMELINE_CTAS + cta) * 4 + event] = t;
  }
}
#define LL_TIMELINE_STAMP(status, kernel, event) ll_timeline_stamp(status, kernel, event)
#else
#define LL_TIMELINE_STAMP(status, kernel, event)
#endif

#include <stdlib.h>
#include <utility>
static inline bool ll_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LITE_LANG_B200_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Launch with the programmatic-serialization attribute when the grid is small enough to be
// resident at once (a dependent kernel that waits on an SM must not keep CTAs of a grid of
// many waves from running).
// cluster_z > 1 makes every cluster_z consecutive CTAs along z one thread-block cluster.
template <typename... KArgs, typename... Args>
static inline void ll_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  const unsigned long long ctas = (unsigned long long)grid.x * grid.y * grid.z;
  attr[0].val.programmaticStreamSerializationAllowed = (ll_pdl_enabled() && ctas <= 1024) ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster_z > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = (unsigned)cluster_z;
    cfg.numAttrs = 2;
  }
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

template <typename... KArgs, typename... Args>
static inline void ll_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  ll_launch_cluster(kernel, grid, block, smem, stream, 1, std::forward<Args>(args)...);
}
