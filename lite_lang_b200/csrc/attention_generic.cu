// Generic paged attention: any number of new tokens per request, any head size
// up to 256, any page size, any group size, float32 or bfloat16 storage.
//
// It is the kernel of the true 32-bit path and the fallback of the bfloat16
// path for shapes the tensor-core kernels do not take.  Every new token t of
// the step is a query at position p = positions[t] of the request in entry
// token_req[t]; it looks at the cached keys lo..p of that request, where
// lo = max(0, p - window + 1) with a window and 0 without.  The new tokens'
// own keys and values are already in the cache when this runs.
//
// One block works on one (token, kv head) pair and on up to GH query heads of
// that kv head's group at once, so keys and values are read once per group.
// Keys are walked in tiles of 32 positions that start at multiples of 32, so
// the order of every sum depends on the position only: the result for a
// position is the same bits however the tokens were cut into steps or batched.
//
// Online softmax (running maximum m, sum l, accumulator) in float32 with expf.
#include "common.cuh"

#define AG_TK 32       // keys per tile
#define AG_THREADS 128
#define AG_WARPS 4
#define AG_GH 8        // query heads per block
#define AG_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(AG_THREADS)
paged_attention_generic_kernel(T* __restrict__ out, long out_stride, const T* __restrict__ q, long q_stride,
                               const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                               const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
                               const int* __restrict__ req_slot, const int* __restrict__ positions, int nh, int nkv,
                               int hd, int page_size, int num_pages, int window, float scale, int* status) {
  extern __shared__ float smem[];
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int t = blockIdx.x;
  const int kvh = blockIdx.y;
  const int group = nh / nkv;
  const int g0 = blockIdx.z * AG_GH;
  const int gcount = min(AG_GH, group - g0);
  const int head0 = kvh * group + g0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  float* qs = smem;                          // [AG_GH][hd]
  float* ks = qs + AG_GH * hd;               // [AG_TK][hd + 1]
  float* vs = ks + AG_TK * (hd + 1);         // [AG_TK][hd]
  float* ps = vs + AG_TK * hd;               // [AG_GH][AG_TK]
  float* alpha_s = ps + AG_GH * AG_TK;       // [AG_GH]
  float* l_s = alpha_s + AG_GH;              // [AG_GH]

  const int entry = token_req[t];
  const int slot = entry >= 0 ? req_slot[entry] : -1;
  const int p = positions[t];
  T* o_row = out + (size_t)t * out_stride + (size_t)head0 * hd;
  if (slot < 0 || p < 0) {  // padding entry of a captured batch: defined output, no reads
    for (int i = tid; i < gcount * hd; i += AG_THREADS) o_row[i] = from_f32<T>(0.f);
    return;
  }
  const int* bt = block_table + (size_t)slot * bt_stride;
  const int lo = (window > 0) ? max(0, p - window + 1) : 0;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head0 * hd;
  for (int i = tid; i < gcount * hd; i += AG_THREADS) qs[i] = to_f32<T>(q_row[i]);

  float m_run[AG_GH / AG_WARPS], l_run[AG_GH / AG_WARPS];
#pragma unroll
  for (int i = 0; i < AG_GH / AG_WARPS; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  float acc[AG_GH][AG_MAX_HD / AG_THREADS];
#pragma unroll
  for (int g = 0; g < AG_GH; ++g)
#pragma unroll
    for (int c = 0; c < AG_MAX_HD / AG_THREADS; ++c) acc[g][c] = 0.f;

  for (int tile0 = (lo / AG_TK) * AG_TK; tile0 <= p; tile0 += AG_TK) {
    __syncthreads();  // previous tile fully consumed (also orders the q load before the first use)
    // ---- load the K and V rows of this tile ----
    for (int j = warp; j < AG_TK; j += AG_WARPS) {
      const int pos = tile0 + j;
      const bool valid = (pos >= lo && pos <= p);
      long base = -1;
      if (valid) {
        const int page = bt[pos / page_size];
        if (page < 0 || page >= num_pages) {
          if (lane == 0) set_status(status, LL_ERR_PAGE_RANGE);
        } else {
          base = (((long)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
        }
      }
      for (int d = lane; d < hd; d += 32) {
        ks[j * (hd + 1) + d] = base >= 0 ? to_f32<T>(k_cache[base + d]) : 0.f;
        vs[j * hd + d] = base >= 0 ? to_f32<T>(v_cache[base + d]) : 0.f;
      }
    }
    __syncthreads();
    // ---- scores and online softmax: warp w owns heads w, w + 4, ... ; lane = key ----
    {
      const int pos = tile0 + lane;
      const bool valid = (pos >= lo && pos <= p);
#pragma unroll
      for (int i = 0; i < AG_GH / AG_WARPS; ++i) {
        const int g = warp + i * AG_WARPS;
        if (g < gcount) {
          float s = 0.f;
          const float* qg = qs + g * hd;
          const float* kj = ks + lane * (hd + 1);
          for (int d = 0; d < hd; ++d) s = fmaf(qg[d], kj[d], s);
          s = valid ? s * scale : -INFINITY;
          const float m_new = fmaxf(m_run[i], warp_max(s));
          const float pj = valid ? expf(s - m_new) : 0.f;
          const float alpha = expf(m_run[i] - m_new);
          l_run[i] = l_run[i] * alpha + warp_sum(pj);
          m_run[i] = m_new;
          ps[g * AG_TK + lane] = pj;
          if (lane == 0) alpha_s[g] = alpha;
        }
      }
    }
    __syncthreads();
    // ---- accumulate P V: thread owns output columns tid, tid + 128 ----
#pragma unroll
    for (int c = 0; c < AG_MAX_HD / AG_THREADS; ++c) {
      const int d = tid + c * AG_THREADS;
      if (d < hd) {
#pragma unroll
        for (int g = 0; g < AG_GH; ++g) {
          if (g < gcount) {
            float a = acc[g][c] * alpha_s[g];
            const float* pg = ps + g * AG_TK;
#pragma unroll 8
            for (int j = 0; j < AG_TK; ++j) a = fmaf(pg[j], vs[j * hd + d], a);
            acc[g][c] = a;
          }
        }
      }
    }
  }
  // ---- normalise and write ----
#pragma unroll
  for (int i = 0; i < AG_GH / AG_WARPS; ++i) {
    const int g = warp + i * AG_WARPS;
    if (g < gcount && lane == 0) l_s[g] = l_run[i];
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < AG_MAX_HD / AG_THREADS; ++c) {
    const int d = tid + c * AG_THREADS;
    if (d < hd) {
#pragma unroll
      for (int g = 0; g < AG_GH; ++g)
        if (g < gcount) o_row[(size_t)g * hd + d] = from_f32<T>(acc[g][c] / l_s[g]);
    }
  }
}

// q: rows of the step's tokens, head h of token t at q + t*q_stride + h*hd.
// out: [num_tokens, nh*hd] with row stride out_stride.
// k_cache / v_cache: one cache plane, each [num_pages, nkv, page_size, hd].
// block_table: int32 [request slots, bt_stride], logical page -> physical page.
// token_req: int32 [num_tokens] entry of each token; req_slot: int32 [entries]
// request slot of each entry (-1: padding); positions: int32 [num_tokens].
// window <= 0 means all earlier positions.
extern "C" int ll_paged_attention_generic(int dtype, void* out, long out_stride, const void* q, long q_stride,
                                          const void* k_cache, const void* v_cache, const int* block_table,
                                          int bt_stride, const int* token_req, const int* req_slot,
                                          const int* positions, int num_tokens, int nh, int nkv, int hd,
                                          int page_size, int num_pages, int window, float scale, int* status,
                                          cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hd <= 0 || hd > AG_MAX_HD || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return (int)cudaErrorInvalidValue;
  const int group = nh / nkv;
  const size_t smem =
      sizeof(float) * ((size_t)AG_GH * hd + (size_t)AG_TK * (hd + 1) + (size_t)AG_TK * hd + AG_GH * AG_TK + 2 * AG_GH);
  dim3 grid(num_tokens, nkv, (group + AG_GH - 1) / AG_GH);
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(paged_attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(paged_attention_generic_kernel<T>, grid, dim3(AG_THREADS), smem, stream, (T*)out, out_stride,
              (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, bt_stride, token_req, req_slot,
              positions, nh, nkv, hd, page_size, num_pages, window, scale, status);
  });
  return LL_LAUNCH_RESULT();
}
