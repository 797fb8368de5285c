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
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
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
  if (!do_rope) rot_dim = 0;
  const int write_q = (bias != nullptr) || do_rope;
  LL_DISPATCH_DTYPE(dtype, ll_launch(bias_rope_store_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)qkv,
                                     qkv_stride, bias, positions, cos_sin, max_pos, rot_dim, do_rope, nh, nkv, hd,
                                     slot_map, (T*)k_cache, (T*)v_cache, page_size, num_slots, write_q, status));
  return LL_LAUNCH_RESULT();
}
