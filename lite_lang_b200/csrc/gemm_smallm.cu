// Matrix product for a few tokens (decode): y[M, N] = x[M, K] * W[N, K]^T, bfloat16 in,
// float32 accumulation, M <= 64.
//
// With so few tokens the product is a stream of the weights through the SMs; what counts
// is bytes in flight, not FLOPs.  The weights take the M side of mma.sync.m16n8k16
// (16 output features a tile), the tokens the N side (8 tokens a tile).  A CTA of 8
// warps owns one feature tile; its warps split K, so each streams its own slice of the 16
// weight rows with 16-byte loads issued a chunk ahead of the arithmetic, and the eight
// partial tiles are added through shared memory.  The token rows are small and are
// re-read from L1/L2.  As in the attention kernel the contraction index of an MMA step is
// mapped to 8 contiguous elements per thread (k-order does not matter for a sum), so both
// operands come straight from global memory in the layout the tensor core wants.
//
// Epilogues: plain (bfloat16 or float32 out), or the SiLU gate of the feed-forward, where
// W holds the gate rows followed by the up rows and the CTA computes both tiles and
// writes silu(gate) * up, so the [M, 2I] intermediate never exists
// (litelang/models/qwen2/layer/transformer_layer.py:79-82 does the product, the
// activation and the second product as three calls).
//
// Needs K % 32 == 0 and 16-byte aligned rows.  N may be any size (the last tile is
// clipped).  Other shapes go to the library product.
#include "common.cuh"

#define GS_WARPS 8
#define GS_THREADS (GS_WARPS * 32)
#define GS_CH 4  // 32-wide k super-steps per chunk

__device__ __forceinline__ void gs_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 gs_ldg_stream(const bf16* p) {  // weights: read once, keep out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 gs_ldg(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }

template <typename OutT> __device__ __forceinline__ OutT gs_out(float v);
template <> __device__ __forceinline__ float gs_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 gs_out<bf16>(float v) { return __float2bfloat16_rn(v); }

template <int MT, bool GATED, typename OutT>
__global__ void __launch_bounds__(GS_THREADS)
gemm_smallm_kernel(OutT* __restrict__ out, long out_stride, const bf16* __restrict__ x, long x_stride,
                   const bf16* __restrict__ w, int M, int N, int K) {
  // N is the number of output features (for GATED: the intermediate size I; W has 2 I rows)
  extern __shared__ float red[];  // [GS_WARPS][GATED ? 2 : 1][16][8 * MT]
  constexpr int TOK = 8 * MT;
  constexpr int NACC = GATED ? 2 : 1;
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int f0 = blockIdx.x * 16;
  const int ra = min(f0 + g, N - 1), rb = min(f0 + g + 8, N - 1);
  const bf16* wp[NACC][2];
  wp[0][0] = w + (size_t)ra * K + 8 * c;
  wp[0][1] = w + (size_t)rb * K + 8 * c;
  if (GATED) {
    wp[NACC - 1][0] = w + (size_t)(N + ra) * K + 8 * c;
    wp[NACC - 1][1] = w + (size_t)(N + rb) * K + 8 * c;
  }
  const bf16* xp[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) xp[j] = x + (size_t)min(8 * j + g, M - 1) * x_stride + 8 * c;

  const int nss = K / 32;
  const int per = (nss + GS_WARPS - 1) / GS_WARPS;
  const int ss0 = warp * per, ss1 = min(nss, ss0 + per);

  float acc[NACC][MT][4];
#pragma unroll
  for (int a = 0; a < NACC; ++a)
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[a][j][0] = acc[a][j][1] = acc[a][j][2] = acc[a][j][3] = 0.f;

  uint4 wbuf[2][NACC][2][GS_CH];
  auto load_chunk = [&](int buf, int ss) {
#pragma unroll
    for (int i = 0; i < GS_CH; ++i) {
      const int s = min(ss + i, ss1 - 1);  // clamped: a repeated load, never out of range
#pragma unroll
      for (int a = 0; a < NACC; ++a) {
        wbuf[buf][a][0][i] = gs_ldg_stream(wp[a][0] + 32 * s);
        wbuf[buf][a][1][i] = gs_ldg_stream(wp[a][1] + 32 * s);
      }
    }
  };
  auto compute_chunk = [&](int buf, int ss) {
#pragma unroll
    for (int i = 0; i < GS_CH; ++i) {
      if (ss + i < ss1) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 xv = gs_ldg(xp[j] + 32 * (ss + i));
#pragma unroll
          for (int a = 0; a < NACC; ++a) {
            const uint4 wa = wbuf[buf][a][0][i], wb = wbuf[buf][a][1][i];
            gs_mma(acc[a][j], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
            gs_mma(acc[a][j], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
          }
        }
      }
    }
  };
  if (ss0 < ss1) {
    load_chunk(0, ss0);
    for (int ss = ss0; ss < ss1; ss += 2 * GS_CH) {
      if (ss + GS_CH < ss1) load_chunk(1, ss + GS_CH);
      compute_chunk(0, ss);
      if (ss + 2 * GS_CH < ss1) load_chunk(0, ss + 2 * GS_CH);
      if (ss + GS_CH < ss1) compute_chunk(1, ss + GS_CH);
    }
  }
  // ---- add the warps' partial tiles ----
#pragma unroll
  for (int a = 0; a < NACC; ++a) {
    float* r = red + ((size_t)(warp * NACC + a) * 16) * TOK;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      r[g * TOK + 8 * j + 2 * c] = acc[a][j][0];
      r[g * TOK + 8 * j + 2 * c + 1] = acc[a][j][1];
      r[(g + 8) * TOK + 8 * j + 2 * c] = acc[a][j][2];
      r[(g + 8) * TOK + 8 * j + 2 * c + 1] = acc[a][j][3];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < 16 * TOK; idx += GS_THREADS) {
    const int tok = idx >> 4, f = idx & 15;
    if (tok >= M || f0 + f >= N) continue;
    float v[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < GS_WARPS; ++wi) s += red[((size_t)(wi * NACC + a) * 16 + f) * TOK + tok];
      v[a] = s;
    }
    float y = v[0];
    if (GATED) {
      // rounded to the storage type first, as the unfused path does between the product and the activation
      const float gt = __bfloat162float(__float2bfloat16_rn(v[0]));
      const float up = __bfloat162float(__float2bfloat16_rn(v[NACC - 1]));
      y = gt / (1.0f + expf(-gt)) * up;
    }
    out[(size_t)tok * out_stride + f0 + f] = gs_out<OutT>(y);
  }
}

template <int MT, bool GATED, typename OutT>
static int gs_launch(void* out, long out_stride, const void* x, long x_stride, const void* w, int M, int N, int K,
                     cudaStream_t stream) {
  const size_t smem = sizeof(float) * GS_WARPS * (GATED ? 2 : 1) * 16 * 8 * MT;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(gemm_smallm_kernel<MT, GATED, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ll_launch(gemm_smallm_kernel<MT, GATED, OutT>, dim3((N + 15) / 16), dim3(GS_THREADS), smem, stream, (OutT*)out,
            out_stride, (const bf16*)x, x_stride, (const bf16*)w, M, N, K);
  return LL_LAUNCH_RESULT();
}

template <bool GATED, typename OutT>
static int gs_dispatch_m(void* out, long out_stride, const void* x, long x_stride, const void* w, int M, int N, int K,
                         cudaStream_t stream) {
  if (M <= 8) return gs_launch<1, GATED, OutT>(out, out_stride, x, x_stride, w, M, N, K, stream);
  if (M <= 16) return gs_launch<2, GATED, OutT>(out, out_stride, x, x_stride, w, M, N, K, stream);
  if (M <= 32) return gs_launch<4, GATED, OutT>(out, out_stride, x, x_stride, w, M, N, K, stream);
  if (M <= 64) return gs_launch<8, GATED, OutT>(out, out_stride, x, x_stride, w, M, N, K, stream);
  return (int)cudaErrorInvalidValue;
}

// x: bfloat16 [M, K] (row stride x_stride), w: bfloat16 [N, K] contiguous (gated: [2 N, K],
// gate rows first), out: [M, N] bfloat16 (out_f32 = 0) or float32 (out_f32 = 1).
extern "C" int ll_gemm_smallm(void* out, long out_stride, int out_f32, const void* x, long x_stride, const void* w,
                              int M, int N, int K, int gated, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K % 32) != 0 || (x_stride % 8) != 0) return (int)cudaErrorInvalidValue;
  if (gated) {
    if (out_f32) return (int)cudaErrorInvalidValue;
    return gs_dispatch_m<true, bf16>(out, out_stride, x, x_stride, w, M, N, K, stream);
  }
  if (out_f32) return gs_dispatch_m<false, float>(out, out_stride, x, x_stride, w, M, N, K, stream);
  return gs_dispatch_m<false, bf16>(out, out_stride, x, x_stride, w, M, N, K, stream);
}
