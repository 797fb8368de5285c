// Token choice from float32 logits [rows, vocab].
//
// Greedy: argmax, ties go to the lowest index (what the reference's
// logits.argmax does).  Temperature: p = softmax(logits / T) in float32 and an
// inverse-CDF draw with a uniform number u in [0, 1) that the caller supplies
// (it comes from a counter-based generator keyed by seed, request and token
// index, so batching cannot change a sample).  The chosen token is the first
// index whose cumulative probability, summed in index order, reaches u times
// the total.  A row whose temperature is <= 0 is greedy.
//
// One block of 1024 threads per row.
#include "common.cuh"

#define SM_THREADS 1024

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

__device__ int block_argmax(const float* __restrict__ row, int vocab, float* s_val, int* s_idx, float* max_out) {
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    argmax_combine(best, best_i, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nwarps = (blockDim.x + 31) >> 5;
    best = lane < nwarps ? s_val[lane] : -INFINITY;
    best_i = lane < nwarps ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      argmax_combine(best, best_i, ov, oi);
    }
    if (lane == 0) {
      s_val[0] = best;
      s_idx[0] = best_i;
    }
  }
  __syncthreads();
  if (max_out) *max_out = s_val[0];
  const int r = s_idx[0];
  __syncthreads();
  return r == 0x7fffffff ? 0 : r;  // a row of NaN or -inf everywhere falls back to token 0
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long row_stride, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out, int vocab) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_part[SM_THREADS];
  __shared__ int s_choice;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float mx;
  const int greedy = block_argmax(row, vocab, s_val, s_idx, &mx);
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }
  // contiguous chunk of the vocabulary per thread, so that the CDF runs in index order
  const int chunk = (vocab + SM_THREADS - 1) / SM_THREADS;
  const int c0 = min(vocab, (int)threadIdx.x * chunk), c1 = min(vocab, c0 + chunk);
  const float inv_t = 1.0f / temp;
  float part = 0.f;
  for (int i = c0; i < c1; ++i) part += expf((row[i] - mx) * inv_t);
  s_part[threadIdx.x] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < SM_THREADS; ++i) total += s_part[i];
    const float target = uniform[r] * total;
    float run = 0.f;
    int owner = -1;
    for (int i = 0; i < SM_THREADS; ++i) {
      if (run + s_part[i] >= target && s_part[i] > 0.f) {
        owner = i;
        break;
      }
      run += s_part[i];
    }
    int choice = greedy;
    if (owner >= 0) {
      const int o0 = owner * chunk, o1 = min(vocab, o0 + chunk);
      choice = -1;
      for (int i = o0; i < o1; ++i) {
        const float e = expf((row[i] - mx) * inv_t);
        run += e;
        if (run >= target && e > 0.f) {
          choice = i;
          break;
        }
      }
      if (choice < 0) {  // rounding left the target just above the chunk's sum: last non-zero entry
        for (int i = o1 - 1; i >= o0; --i)
          if (expf((row[i] - mx) * inv_t) > 0.f) {
            choice = i;
            break;
          }
        if (choice < 0) choice = greedy;
      }
    }
    s_choice = choice;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = s_choice;
}

// logits: float32 [rows, vocab] with row stride row_stride; temperature and
// uniform: float32 [rows] or null (all greedy); out: int32 [rows].
extern "C" int ll_sample(const float* logits, long row_stride, const float* temperature, const float* uniform,
                         int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return (int)cudaErrorInvalidValue;
  if (temperature != nullptr && uniform == nullptr) return (int)cudaErrorInvalidValue;
  sample_kernel<<<rows, SM_THREADS, 0, stream>>>(logits, row_stride, temperature, uniform, out, vocab);
  return LL_LAUNCH_RESULT();
}
