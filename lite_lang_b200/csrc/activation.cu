// SiLU-gated product of the feed-forward: out[t, i] = silu(gu[t, i]) * gu[t, I + i].
//
// gate is the first I columns of the fused projection, up the last I.  The
// whole expression is evaluated in float32 and rounded once.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, long total, int inter) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long idx0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = idx0; idx < total; idx += step) {
    const long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32<T>(gu[t * 2 * inter + i]);
    const float u = to_f32<T>(gu[t * 2 * inter + inter + i]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// 8 bf16 values a thread; needs inter % 8 == 0.
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, long total8, int inter8) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long idx0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = idx0; idx < total8; idx += step) {
    const long t = idx / inter8;
    const int i = (int)(idx - t * inter8);
    const uint4 gv = reinterpret_cast<const uint4*>(gu)[t * 2 * inter8 + i];
    const uint4 uv = reinterpret_cast<const uint4*>(gu)[t * 2 * inter8 + inter8 + i];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]);
      const float2 u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    reinterpret_cast<uint4*>(out)[idx] = ov;
  }
}

// SMs of the current device (asked once per device): the grid-stride kernels launch 16 blocks an SM at most
static int silu_device_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int ll_silu_mul(int dtype, void* out, const void* gate_up, int num_tokens, int inter, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long total = (long)num_tokens * inter;
  const long most = (long)silu_device_sms() * 16;
  if (dtype == LL_DTYPE_BF16 && (inter % 8) == 0) {
    const long total8 = total / 8;
    const int blocks = (int)min((total8 + 255) / 256, most);
    ll_launch(silu_mul_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (bf16*)out, (const bf16*)gate_up, total8,
              inter / 8);
    return LL_LAUNCH_RESULT();
  }
  const int blocks = (int)min((total + 255) / 256, most);
  LL_DISPATCH_DTYPE(dtype, ll_launch(silu_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out,
                                     (const T*)gate_up, total, inter));
  return LL_LAUNCH_RESULT();
}
