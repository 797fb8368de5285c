// Bias, rotary position encoding and the write into the paged cache, in one pass
// over the fused q|k|v projection of the step's tokens.
//
// Row t of `qkv` holds nh query heads, then nkv key heads, then nkv value
// heads, each of head_dim values.  For every token:
//   * bias (float32, optional) is added to q, k and v in float32;
//   * the first `rot_dim` values of each q and k head are rotated by the angle
//     of the token's position, pairs being (i, i + rot_dim/2): "half-split".
//     cos and sin come from a float32 table [max_pos, rot_dim] whose row p holds
//     cos(p * f_i) for i < rot_dim/2 and then sin(p * f_i); the table is made on
//     the host so that the angles are the same float32 numbers everywhere;
//   * q is written back in place (rounded once to the storage type);
//   * k and v are written into the cache at the token's slot
//     (slot = page * page_size + offset; -1 skips the write).
// Each of the three steps can be switched off, which gives the unfused forms
// (bias only, rotation only, store only) that other position encodings use.
//
// Cache plane layout: K and V are each [num_pages, nkv, page_size, head_dim].
#include "common.cuh"

template <typename T>
__global__ void bias_rope_store_kernel(T* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                                       const int* __restrict__ positions, const float* __restrict__ cos_sin,
                                       int max_pos, int rot_dim, int do_rope, int nh, int nkv, int hd,
                                       const int* __restrict__ slot_map, T* __restrict__ k_cache,
                                       T* __restrict__ v_cache, int page_size, long num_slots, int write_q,
                                       int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  T* row = qkv + (size_t)t * qkv_stride;
  int pos = positions ? positions[t] : 0;
  if (do_rope && (pos < 0 || pos >= max_pos)) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_POSITION_RANGE);
    pos = 0;
  }
  long slot = slot_map ? (long)slot_map[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const int half = rot_dim >> 1;
  const float* cs = cos_sin + (size_t)pos * rot_dim;

  // q and k heads: rotation pairs and the untouched tail
  const int n_rot_heads = nh + nkv;
  const int per_head = hd - half;  // work items of a head: `half` pairs + (hd - rot_dim) singles
  for (int w = threadIdx.x; w < n_rot_heads * per_head; w += blockDim.x) {
    const int h = w / per_head;
    const int i = w - h * per_head;
    T* head = row + (size_t)h * hd;
    const float* b = bias ? bias + (size_t)h * hd : nullptr;
    const bool is_k = h >= nh;
    T* dst = nullptr;
    if (is_k && slot >= 0) dst = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + off) * hd;
    if (i < half) {
      float x0 = to_f32<T>(head[i]);
      float x1 = to_f32<T>(head[i + half]);
      if (b) {
        x0 += b[i];
        x1 += b[i + half];
      }
      float o0 = x0, o1 = x1;
      if (do_rope) {
        const float c = cs[i], s = cs[half + i];
        o0 = x0 * c - x1 * s;
        o1 = x0 * s + x1 * c;
      }
      if (!is_k) {
        if (write_q) {
          head[i] = from_f32<T>(o0);
          head[i + half] = from_f32<T>(o1);
        }
      } else {
        if (write_q) {  // keep the row itself consistent for callers that read k from it
          head[i] = from_f32<T>(o0);
          head[i + half] = from_f32<T>(o1);
        }
        if (dst) {
          dst[i] = from_f32<T>(o0);
          dst[i + half] = from_f32<T>(o1);
        }
      }
    } else {
      const int j = rot_dim + (i - half);
      float x = to_f32<T>(head[j]);
      if (b) x += b[j];
      if (write_q) head[j] = from_f32<T>(x);
      if (dst) dst[j] = from_f32<T>(x);
    }
  }
  // v heads: bias and store
  for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
    const int h = w / hd;
    const int j = w - h * hd;
    T* head = row + (size_t)(nh + nkv + h) * hd;
    float x = to_f32<T>(head[j]);
    if (bias) x += bias[(size_t)(nh + nkv + h) * hd + j];
    if (write_q && bias) head[j] = from_f32<T>(x);
    if (slot >= 0) v_cache[(((size_t)page * nkv + h) * page_size + off) * hd + j] = from_f32<T>(x);
  }
}

// bfloat16, whole-head rotation (rot_dim == hd), hd a multiple of 16: a thread takes 8 consecutive
// values of the first half of a head and their 8 partners from the second half (16-byte accesses), or
// 8 values of a v head.  Same arithmetic and roundings as the generic kernel.
__global__ void __launch_bounds__(256)
bias_rope_store_bf16x8_kernel(bf16* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                              const int* __restrict__ positions, const float* __restrict__ cos_sin, int max_pos, int nh,
                              int nkv, int hd, const int* __restrict__ slot_map, bf16* __restrict__ k_cache,
                              bf16* __restrict__ v_cache, int page_size, long num_slots, int* status) {
  LL_PDL_TRIGGER();
  LL_TIMELINE_STAMP(status, 0, 0);   // (where the projection is a library product, this kernel stands for q|k|v)
  LL_PDL_WAIT();
  LL_TIMELINE_STAMP(status, 0, 1);
  const int t = blockIdx.x;
  bf16* row = qkv + (size_t)t * qkv_stride;
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_POSITION_RANGE);
    pos = 0;
  }
  long slot = slot_map ? (long)slot_map[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const int half = hd >> 1;
  const int cph = half / 8;                   // 8-value pieces in half a head
  const float* cs = cos_sin + (size_t)pos * hd;
  const int n_rot = (nh + nkv) * cph, n_v = nkv * (hd / 8);
  for (int w = threadIdx.x; w < n_rot + n_v; w += blockDim.x) {
    if (w < n_rot) {
      const int h = w / cph, i0 = (w - h * cph) * 8;
      bf16* head = row + (size_t)h * hd;
      const uint4 a = *reinterpret_cast<const uint4*>(head + i0);
      const uint4 b = *reinterpret_cast<const uint4*>(head + i0 + half);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
      float x0[8], x1[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = __bfloat1622float2(a2[k]), fb = __bfloat1622float2(b2[k]);
        x0[2 * k] = fa.x; x0[2 * k + 1] = fa.y;
        x1[2 * k] = fb.x; x1[2 * k + 1] = fb.y;
      }
      if (bias) {
        const float* bb = bias + (size_t)h * hd + i0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          x0[k] += bb[k];
          x1[k] += bb[k + half];
        }
      }
      uint4 o0, o1;
      __nv_bfloat162* p0 = reinterpret_cast<__nv_bfloat162*>(&o0);
      __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(&o1);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float c0 = cs[i0 + 2 * k], c1 = cs[i0 + 2 * k + 1];
        const float s0 = cs[half + i0 + 2 * k], s1 = cs[half + i0 + 2 * k + 1];
        p0[k] = __floats2bfloat162_rn(x0[2 * k] * c0 - x1[2 * k] * s0, x0[2 * k + 1] * c1 - x1[2 * k + 1] * s1);
        p1[k] = __floats2bfloat162_rn(x0[2 * k] * s0 + x1[2 * k] * c0, x0[2 * k + 1] * s1 + x1[2 * k + 1] * c1);
      }
      *reinterpret_cast<uint4*>(head + i0) = o0;
      *reinterpret_cast<uint4*>(head + i0 + half) = o1;
      if (h >= nh && slot >= 0) {
        bf16* dst = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + off) * hd;
        *reinterpret_cast<uint4*>(dst + i0) = o0;
        *reinterpret_cast<uint4*>(dst + i0 + half) = o1;
      }
    } else {
      const int wv = w - n_rot;
      const int h = wv / (hd / 8), j0 = (wv - h * (hd / 8)) * 8;
      bf16* head = row + (size_t)(nh + nkv + h) * hd;
      uint4 a = *reinterpret_cast<const uint4*>(head + j0);
      if (bias) {
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
        const float* bb = bias + (size_t)(nh + nkv + h) * hd + j0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(a2[k]);
          a2[k] = __floats2bfloat162_rn(f.x + bb[2 * k], f.y + bb[2 * k + 1]);
        }
        *reinterpret_cast<uint4*>(head + j0) = a;
      }
      if (slot >= 0)
        *reinterpret_cast<uint4*>(v_cache + (((size_t)page * nkv + h) * page_size + off) * hd + j0) = a;
    }
  }
  LL_TIMELINE_STAMP(status, 0, 2);
}

// qkv: [num_tokens, (nh + 2 nkv) * hd] with row stride qkv_stride (elements).
// bias: float32 [(nh + 2 nkv) * hd] or null.  positions: int32 [num_tokens].
// cos_sin: float32 [max_pos, rot_dim] or null (no rotation).
// slot_map: int32 [num_tokens] or null (no store).  num_slots = num_pages * page_size.
extern "C" int ll_bias_rope_store(int dtype, void* qkv, long qkv_stride, const float* bias, const int* positions,
                                  const float* cos_sin, int max_pos, int rot_dim, int nh, int nkv, int hd,
                                  const int* slot_map, void* k_cache, void* v_cache, int page_size, long num_slots,
                                  int num_tokens, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int do_rope = cos_sin != nullptr;
  if (do_rope && (rot_dim <= 0 || (rot_dim & 1) || rot_dim > hd)) return (int)cudaErrorInvalidValue;
  if (dtype == LL_DTYPE_BF16 && do_rope && rot_dim == hd && (hd % 16) == 0 && (qkv_stride % 8) == 0 &&
      positions != nullptr) {
    const int work = (nh + nkv) * (hd / 16) + nkv * (hd / 8);
    const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
    ll_launch(bias_rope_store_bf16x8_kernel, dim3(num_tokens), dim3(threads), 0, stream, (bf16*)qkv, qkv_stride, bias,
              positions, cos_sin, max_pos, nh, nkv, hd, slot_map, (bf16*)k_cache, (bf16*)v_cache, page_size,
              num_slots, status);
    return LL_LAUNCH_RESULT();
  }
  if (!do_rope) rot_dim = 0;
  const int write_q = (bias != nullptr) || do_rope;
  LL_DISPATCH_DTYPE(dtype, ll_launch(bias_rope_store_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)qkv,
                                     qkv_stride, bias, positions, cos_sin, max_pos, rot_dim, do_rope, nh, nkv, hd,
                                     slot_map, (T*)k_cache, (T*)v_cache, page_size, num_slots, write_q, status));
  return LL_LAUNCH_RESULT();
}
