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
#include "common.cuh"

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

// ---------------------------------------------------------------------------------------
// Two stages, so that a few rows of a large vocabulary still fill the GPU.
//
// Stage 1: one block per (chunk of SM_CHUNK columns, row): the chunk's maximum m_c and
// its first argmax, and for sampled rows s_c = sum exp((x - m_c) / T) over the chunk.
// Stage 2: one block per row: M = max m_c (ties to the lowest chunk, hence the lowest
// index), total = sum s_c exp((m_c - M) / T); the chunk whose cumulative share reaches
// u * total is found, and the walk inside that chunk is done by the block (partial sums
// per thread, then the owner thread walks its few elements), all in index order.
// ---------------------------------------------------------------------------------------
#define SM_CHUNK 2048
#define SM_T1 256

__global__ void __launch_bounds__(SM_T1)
sample_stage1_kernel(const float* __restrict__ logits, long row_stride, const float* __restrict__ temperature,
                     float* __restrict__ part, int vocab, int nchunks) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_sum[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int chunk = blockIdx.x, r = blockIdx.y;
  const int c0 = chunk * SM_CHUNK, n = min(SM_CHUNK, vocab - c0);
  const float* row = logits + (size_t)r * row_stride + c0;
  float mx;
  const int arg = block_argmax(row, n, s_val, s_idx, &mx);
  const float temp = temperature ? temperature[r] : 0.f;
  float sum = 0.f;
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp;
    float part_sum = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) part_sum += expf((row[i] - mx) * inv_t);
    sum = block_sum(part_sum, s_sum);
  }
  if (threadIdx.x == 0) {
    float* o = part + ((size_t)r * nchunks + chunk) * 3;
    o[0] = mx;
    o[1] = __int_as_float(c0 + arg);
    o[2] = sum;
  }
}

__global__ void __launch_bounds__(SM_T1)
sample_stage2_kernel(const float* __restrict__ logits, long row_stride, const float* __restrict__ temperature,
                     const float* __restrict__ uniform, const float* __restrict__ part, int* __restrict__ out,
                     int vocab, int nchunks) {
  __shared__ float s_part[SM_T1];
  __shared__ float s_M;
  __shared__ int s_arg, s_chunk;
  __shared__ float s_before, s_target;
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int r = blockIdx.x;
  const float* pr = part + (size_t)r * nchunks * 3;
  const float temp = temperature ? temperature[r] : 0.f;
  // the chunks' partial results: thread c reads chunk c's (all in flight at once; one thread going through
  // them one after the other was a chain of memory latencies), then the block reduces
  __shared__ float s_val[SM_T1 / 32];
  __shared__ int s_idx[SM_T1 / 32];
  float best = -INFINITY, my_max = -INFINITY, my_sum = 0.f;
  int best_i = 0x7fffffff;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x) {   // (nchunks <= blockDim.x for every vocabulary up to 500 k)
    my_max = pr[c * 3];
    my_sum = pr[c * 3 + 2];
    argmax_combine(best, best_i, my_max, __float_as_int(pr[c * 3 + 1]));
  }
  const bool one_each = nchunks <= (int)blockDim.x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    argmax_combine(best, best_i, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    s_val[threadIdx.x >> 5] = best;
    s_idx[threadIdx.x >> 5] = best_i;
  }
  if (one_each) s_part[threadIdx.x] = 0.f;
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = s_val[0];
    int arg = s_idx[0];
    for (int w = 1; w < SM_T1 / 32; ++w) argmax_combine(M, arg, s_val[w], s_idx[w]);
    s_M = M;
    s_arg = arg;
    s_chunk = -1;
  }
  __syncthreads();
  if (temp > 0.f) {
    const float inv_t = 1.0f / temp, M = s_M;
    if (one_each) {   // every chunk's share of the total, in chunk order, by its own thread
      if ((int)threadIdx.x < nchunks) s_part[threadIdx.x] = my_sum * expf((my_max - M) * inv_t);
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int c = 0; c < nchunks; ++c)
        total += one_each ? s_part[c] : pr[c * 3 + 2] * expf((pr[c * 3] - M) * inv_t);
      const float target = uniform[r] * total;
      float run = 0.f;
      for (int c = 0; c < nchunks; ++c) {
        const float share = one_each ? s_part[c] : pr[c * 3 + 2] * expf((pr[c * 3] - M) * inv_t);
        if (share > 0.f && run + share >= target) {
          s_chunk = c;
          break;
        }
        run += share;
      }
      s_before = run;
      s_target = target;
    }
  }
  __syncthreads();
  if (!(temp > 0.f) || s_chunk < 0) {  // greedy, or rounding pushed the target past the last chunk
    if (threadIdx.x == 0) out[r] = s_arg;
    return;
  }
  const int chunk = s_chunk;
  const int c0 = chunk * SM_CHUNK, n = min(SM_CHUNK, vocab - c0);
  const float* row = logits + (size_t)r * row_stride + c0;
  const float inv_t = 1.0f / temp, M = s_M;
  constexpr int PER = SM_CHUNK / SM_T1;
  const int i0 = threadIdx.x * PER;
  float mine = 0.f;
  for (int i = i0; i < min(n, i0 + PER); ++i) mine += expf((row[i] - M) * inv_t);
  s_part[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = s_before;
    int owner = -1;
    for (int t = 0; t < SM_T1; ++t) {
      if (s_part[t] > 0.f && run + s_part[t] >= s_target) {
        owner = t;
        break;
      }
      run += s_part[t];
    }
    int choice = -1;
    if (owner >= 0) {
      for (int i = owner * PER; i < min(n, owner * PER + PER); ++i) {
        const float e = expf((row[i] - M) * inv_t);
        run += e;
        if (e > 0.f && run >= s_target) {
          choice = c0 + i;
          break;
        }
      }
      if (choice < 0)  // rounding: the last non-zero element of the owner's piece
        for (int i = min(n, owner * PER + PER) - 1; i >= owner * PER; --i)
          if (expf((row[i] - M) * inv_t) > 0.f) {
            choice = c0 + i;
            break;
          }
    }
    if (choice < 0) {  // rounding: the last non-zero element of the chunk
      for (int i = n - 1; i >= 0; --i)
        if (expf((row[i] - M) * inv_t) > 0.f) {
          choice = c0 + i;
          break;
        }
    }
    out[r] = choice >= 0 ? choice : s_arg;
  }
}

extern "C" long ll_sample_scratch_floats(int rows, int vocab) {
  return (long)rows * ((vocab + SM_CHUNK - 1) / SM_CHUNK) * 3;
}

// logits: float32 [rows, vocab] with row stride row_stride; temperature and
// uniform: float32 [rows] or null (all greedy); out: int32 [rows]; scratch: float32,
// ll_sample_scratch_floats(rows, vocab) elements.
extern "C" int ll_sample(const float* logits, long row_stride, const float* temperature, const float* uniform,
                         int* out, int rows, int vocab, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || scratch == nullptr || rows > 65535) return (int)cudaErrorInvalidValue;
  if (temperature != nullptr && uniform == nullptr) return (int)cudaErrorInvalidValue;
  const int nchunks = (vocab + SM_CHUNK - 1) / SM_CHUNK;
  ll_launch(sample_stage1_kernel, dim3(nchunks, rows), dim3(SM_T1), 0, stream, logits, row_stride, temperature,
            scratch, vocab, nchunks);
  ll_launch(sample_stage2_kernel, dim3(rows), dim3(SM_T1), 0, stream, logits, row_stride, temperature, uniform,
            (const float*)scratch, out, vocab, nchunks);
  return LL_LAUNCH_RESULT();
}
