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
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
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
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
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

// bfloat16 rows whose length is a multiple of 8 and at most 8 * 1024: every thread keeps 8 values in
// registers (one 16-byte load per operand), so the row is read once and nothing goes through shared
// memory.  Same arithmetic and the same roundings as the generic kernel.
__global__ void __launch_bounds__(1024)
add_rmsnorm_bf16x8_kernel(bf16* __restrict__ out, bf16* __restrict__ residual, const bf16* __restrict__ delta,
                          const float* __restrict__ partial, int parts, long part_stride,
                          const float* __restrict__ w, float eps, int hidden, const int* __restrict__ rows,
                          int write_residual) {
  __shared__ float scratch[32];
  const int i0 = threadIdx.x * 8;
  const bool active = i0 < hidden;
  // the norm weights do not depend on the kernel before: they are on their way before the wait for it
  float4 wa = make_float4(0.f, 0.f, 0.f, 0.f), wb = wa;
  if (active) {
    wa = *reinterpret_cast<const float4*>(w + i0);
    wb = *reinterpret_cast<const float4*>(w + i0 + 4);
  }
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int i_out = blockIdx.x;
  const int r = rows ? rows[i_out] : i_out;
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = 0.f;
  if (active) {
    bf16* res = residual + (size_t)r * hidden + i0;
    // every load of the row's piece is asked for before the first one is used: the residual values, the delta or
    // the first four parts of a split product (a chain of a trip to L2 a part otherwise, in the middle of the step's
    // chain of kernels)
    const uint4 rv = *reinterpret_cast<const uint4*>(res);
    uint4 dv = make_uint4(0u, 0u, 0u, 0u);
    float4 pa[4], pb[4];
    const float* par = partial ? partial + (size_t)r * hidden + i0 : nullptr;
    if (delta) {
      dv = *reinterpret_cast<const uint4*>(delta + (size_t)r * hidden + i0);
    } else if (partial) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (q < parts) {
          pa[q] = *reinterpret_cast<const float4*>(par + (size_t)q * part_stride);
          pb[q] = *reinterpret_cast<const float4*>(par + (size_t)q * part_stride + 4);
        }
      }
    }
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(r2[k]);
      v[2 * k] = f.x;
      v[2 * k + 1] = f.y;
    }
    bool changed = false;
    if (delta) {
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(d2[k]);
        v[2 * k] = round_to<bf16>(v[2 * k] + f.x);
        v[2 * k + 1] = round_to<bf16>(v[2 * k + 1] + f.y);
      }
      changed = true;
    } else if (partial) {
      float d[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) d[k] = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {     // (the same order of additions as a plain loop over the parts)
        if (q < parts) {
          d[0] += pa[q].x; d[1] += pa[q].y; d[2] += pa[q].z; d[3] += pa[q].w;
          d[4] += pb[q].x; d[5] += pb[q].y; d[6] += pb[q].z; d[7] += pb[q].w;
        }
      }
      for (int q = 4; q < parts; ++q) {
        const float4 a = *reinterpret_cast<const float4*>(par + (size_t)q * part_stride);
        const float4 b = *reinterpret_cast<const float4*>(par + (size_t)q * part_stride + 4);
        d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w;
        d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = round_to<bf16>(v[k] + round_to<bf16>(d[k]));
      changed = true;
    }
    if (changed && write_residual) {
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
      *reinterpret_cast<uint4*>(res) = ov;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  if (active) {
    const float ww[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      o2[k] = __floats2bfloat162_rn(v[2 * k] * inv * ww[2 * k], v[2 * k + 1] * inv * ww[2 * k + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)i_out * hidden + i0) = ov;
  }
}

// Many bfloat16 rows (portions of prompts): a warp a row, eight rows a block.  A lane holds every 32nd
// 16-byte piece of the row in registers (all of them asked for at once, so that a row is a few loads in
// flight per lane instead of one), the sum of squares goes through the warp's shuffles, nothing through
// shared memory and there is no block barrier.  Same arithmetic and the same roundings as the kernels
// above; only the order of the float32 sum of squares differs.  MAXC: pieces a lane holds (rows of up to
// 256 MAXC values; wider rows, and steps of fewer than 1,024 rows, stay with the block-a-row kernel).
template <int MAXC>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(bf16* __restrict__ out, bf16* __restrict__ residual, const bf16* __restrict__ delta,
                        const float* __restrict__ w, float eps, int hidden, const int* __restrict__ rows, int n_out,
                        int write_residual) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int lane = threadIdx.x & 31;
  const int i_out = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (i_out >= n_out) return;
  const int r = rows ? rows[i_out] : i_out;
  bf16* res = residual + (size_t)r * hidden;
  uint4 rv[MAXC], dv[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i0 = (c * 32 + lane) * 8;
    rv[c] = make_uint4(0u, 0u, 0u, 0u);
    dv[c] = make_uint4(0u, 0u, 0u, 0u);
    if (i0 < hidden) {
      rv[c] = *reinterpret_cast<const uint4*>(res + i0);
      if (delta) dv[c] = *reinterpret_cast<const uint4*>(delta + (size_t)r * hidden + i0);
    }
  }
  float v[MAXC][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i0 = (c * 32 + lane) * 8;
    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv[c]);
    const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[c]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(r2[k]);
      v[c][2 * k] = f.x;
      v[c][2 * k + 1] = f.y;
      if (delta) {
        const float2 g = __bfloat1622float2(d2[k]);
        v[c][2 * k] = round_to<bf16>(f.x + g.x);
        v[c][2 * k + 1] = round_to<bf16>(f.y + g.y);
      }
    }
    if (delta && write_residual && i0 < hidden) {
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(v[c][2 * k], v[c][2 * k + 1]);
      *reinterpret_cast<uint4*>(res + i0) = ov;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[c][k] * v[c][k];
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  bf16* o = out + (size_t)i_out * hidden;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i0 = (c * 32 + lane) * 8;
    if (i0 < hidden) {
      const float4 wa = __ldg(reinterpret_cast<const float4*>(w + i0)), wb = __ldg(reinterpret_cast<const float4*>(w + i0 + 4));
      const float ww[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o2[k] = __floats2bfloat162_rn(v[c][2 * k] * inv * ww[2 * k], v[c][2 * k + 1] * inv * ww[2 * k + 1]);
      *reinterpret_cast<uint4*>(o + i0) = ov;
    }
  }
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
  // (measured warm on a B200, rows of 1,536 / 2,048 / 3,584 values: 2,048 rows 5.2 / 5.9 / 18.8 us against the
  // block-a-row kernel's 6.2 / 7.7 / 13.5; 256 rows 4.4 / 4.8 / 7.8 against 2.5 / 2.6 / 2.9: too few warps then)
  if (dtype == LL_DTYPE_BF16 && (hidden % 8) == 0 && hidden <= 2048 && partial == nullptr && n_out >= 1024) {
    // many rows: a warp a row
    const dim3 grid((n_out + 7) / 8);
#define LL_ROWS_LAUNCH(C)                                                                                          \
  ll_launch(add_rmsnorm_rows_kernel<C>, grid, dim3(256), 0, stream, (bf16*)out, (bf16*)residual, (const bf16*)delta, \
            w, eps, hidden, rows, n_out, write_residual)
    if (hidden <= 512) LL_ROWS_LAUNCH(2);
    else if (hidden <= 1024) LL_ROWS_LAUNCH(4);
    else LL_ROWS_LAUNCH(8);
#undef LL_ROWS_LAUNCH
    return LL_LAUNCH_RESULT();
  }
  if (dtype == LL_DTYPE_BF16 && (hidden % 8) == 0 && hidden <= 8 * 1024 && (part_stride % 4) == 0) {
    const int threads = ((hidden / 8 + 31) / 32) * 32;
    ll_launch(add_rmsnorm_bf16x8_kernel, dim3(n_out), dim3(threads), 0, stream, (bf16*)out, (bf16*)residual,
              (const bf16*)delta, partial, parts, part_stride, w, eps, hidden, rows, write_residual);
    return LL_LAUNCH_RESULT();
  }
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
