// Weight-streaming matrix product on the fifth-generation tensor cores (tcgen05), for steps of
// 33..128 tokens (large decode batches): y[M, N] = x[M, K] * W[N, K]^T, bfloat16, float32 accumulation.
//
// The weights are the M side of the MMA (128 output features a tile), the tokens the N side (64 or
// 128 columns).  One persistent CTA per SM with three roles:
//   warp 0    producer: one thread keeps a ring of shared-memory stages filled by TMA
//             (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast): a box of 128 features x 64 k of
//             W (for the gated feed-forward two boxes of 64 rows, the gate rows and the up rows of the same
//             64 features, stacked into one 128-row tile) and a box of the tokens' rows;
//   warp 1    MMA: one thread issues tcgen05.mma.cta_group::1.kind::f16 (128 x NT x 16) straight from
//             the stages through shared-memory descriptors, accumulating in tensor memory; a
//             tcgen05.commit hands each stage back to the producer when the MMAs that read it are done;
//   warps 2-5 epilogue: when a unit's last MMA has completed they read the accumulator from tensor
//             memory (tcgen05.ld, one feature row per thread, so a token's 32 features go out as one
//             64-byte piece), apply the epilogue (plain; float32 partial sums of a product split over k;
//             SiLU gate, where the up half of the tile crosses to the gate half's threads through shared
//             memory) and hand tensor memory back.
// The weights do not depend on the kernel before, so the producer starts streaming them before
// griddepcontrol.wait; the tokens' boxes follow after it.
//
// Every mbarrier wait is bounded (about two seconds of clock): a wait that runs out records
// LL_ERR_WAIT_TIMEOUT and the kernel carries on to its end, frees its tensor memory and returns.
//
// Needs K % 64 == 0 and 16-byte aligned rows.  Rows of W beyond N and tokens beyond M are zero-filled by TMA.
#include <cuda.h>

#include "common.cuh"

#define LL_ERR_WAIT_TIMEOUT 5
#define TC_THREADS 192
#define TC_MODE_PLAIN 0
#define TC_MODE_GATED 1

__device__ __forceinline__ unsigned tc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// `dead` is the calling thread's memory of a wait that ran out: after the first one it waits no more.
__device__ __forceinline__ void tc_mbar_wait(unsigned bar, unsigned parity, int* status, bool& dead) {
  if (dead || tc_mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!tc_mbar_try(bar, parity)) {
    if (clock64() - t0 > 4000000000ll) {
      set_status(status, LL_ERR_WAIT_TIMEOUT);
      dead = true;
      return;
    }
  }
}
__device__ __forceinline__ void tc_tma_load(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte
// swizzle (what TMA writes): groups of 8 rows are 1024 bytes apart; 16 elements of k are 32 bytes.
__device__ __forceinline__ unsigned long long tc_desc(unsigned smem_addr) {
  return (unsigned long long)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                       unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld8(unsigned taddr, float (&v)[8]) {
  unsigned r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n tcgen05.wait::ld.sync.aligned;"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

struct TcParams {
  void* out;
  long out_stride;
  int M, N, K;   // tokens, output features (gated: the intermediate size; W has 2 N rows), inner size
  int units;     // feature units (128 features each) times ksplit
  int ksplit;    // > 1: out is float32 [ksplit, M, N] partial sums
  int cpp;       // 64-wide k boxes per part
  int vec_ok;    // the output takes 16-byte pieces (aligned base and stride, N a multiple of the piece)
  // SCALED (gated, at most 64 tokens): the tokens' rows are only multiplied by the weight of the norm before this
  // product yet; the rows' sums of squares come in parts [sumsq_units][64] (see gemm_stream.cu: the product before
  // the norm leaves them), and each row of the result is scaled by 1 / sqrt(sum / K + eps) before the activation
  const float* sumsq_in;
  int sumsq_units;
  float norm_eps;
  int* status;
};

// Shared-memory plan.  A stage holds 128 weight rows x 64 k (plain: 128 output features; gated: 64 gate
// rows above 64 up rows of the same 64 features, so that one MMA makes both) and NT token rows x 64 k.
template <int MODE, int NT>
struct TcShape {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int STAGE_BYTES = A_BYTES + NT * 128;
  static constexpr int FEATS = (MODE == TC_MODE_GATED) ? 64 : 128;
  static constexpr int XCH_BYTES = 128 * (NT + 1) * 4;   // the accumulator tile on its way out
  static constexpr int STAGES_FIT = (220 * 1024 - XCH_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + XCH_BYTES;
};

// OUT: 0 bfloat16, 1 float32 (also the partial sums); SCALED: see TcParams
template <int MODE, int NT, int OUT, bool SCALED>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
  using S = TcShape<MODE, NT>;
  constexpr int A_BYTES = S::A_BYTES, STAGE_BYTES = S::STAGE_BYTES, STAGES = S::STAGES;
  constexpr int TMEM_COLS = NT;                            // float32 accumulator columns (power of two >= 32)
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 2);
  float* stg = reinterpret_cast<float*>(bars + 2 * STAGES + 4);   // accumulator rows on their way out, [128][NT + 1]
  const unsigned stage0 = tc_smem(smem);
  const unsigned full0 = tc_smem(bars), empty0 = tc_smem(bars + STAGES);
  const unsigned acc_full = tc_smem(bars + 2 * STAGES), acc_empty = tc_smem(bars + 2 * STAGES + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(full0 + 8 * s, 1);
      tc_mbar_init(empty0 + 8 * s, 1);
    }
    tc_mbar_init(acc_full, 1);
    tc_mbar_init(acc_empty, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for the accumulator(s): allocated and freed by this warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem(tmem_slot)),
                 "r"((unsigned)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_slot;
  LL_PDL_TRIGGER();
  [[maybe_unused]] constexpr int TL_KERNEL = MODE == TC_MODE_GATED ? 3 : 4;   // (the logits, wide and unsplit: 5)
  LL_TIMELINE_STAMP(p.status, (MODE == TC_MODE_PLAIN && p.ksplit == 1) ? 5 : TL_KERNEL, 0);

  bool dead = false;
  const int kboxes = p.K / 64;
  long total = 0;  // stages this CTA goes through
  for (int uu = blockIdx.x; uu < p.units; uu += gridDim.x) {
    const int kp = uu % p.ksplit;
    total += min(kboxes, (kp + 1) * p.cpp) - kp * p.cpp;
  }

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      // weights first (they do not depend on the kernel before), up to a ring's worth; then wait for
      // the kernel before and send the tokens' boxes after them
      int uu = blockIdx.x, kc = 0, kc_end = 0;
      auto open_unit = [&]() {  // the k boxes of unit uu
        if (uu < p.units) {
          const int kp = uu % p.ksplit;
          kc = kp * p.cpp;
          kc_end = min(kboxes, (kp + 1) * p.cpp);
        }
      };
      auto advance = [&]() {
        if (++kc >= kc_end) {
          uu += gridDim.x;
          open_unit();
        }
      };
      auto issue_a = [&](int s) {
        const int u = uu / p.ksplit;
        if (MODE == TC_MODE_GATED) {  // two boxes of 64 rows: gate rows, then the up rows of the same features
          tc_tma_load(stage0 + s * STAGE_BYTES, &wmap, kc * 64, u * 64, full0 + 8 * s);
          tc_tma_load(stage0 + s * STAGE_BYTES + A_BYTES / 2, &wmap, kc * 64, p.N + u * 64, full0 + 8 * s);
        } else {
          tc_tma_load(stage0 + s * STAGE_BYTES, &wmap, kc * 64, u * 128, full0 + 8 * s);
        }
      };
      auto issue_b = [&](int s, int k) {
        tc_tma_load(stage0 + s * STAGE_BYTES + A_BYTES, &xmap, k * 64, 0, full0 + 8 * s);
      };
      const int early = (int)(total < STAGES ? total : STAGES);
      int early_kc[STAGES];
      open_unit();
      for (int s = 0; s < early; ++s) {
        tc_mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        issue_a(s);
        early_kc[s] = kc;
        advance();
      }
      LL_PDL_WAIT();
      for (int s = 0; s < early; ++s) issue_b(s, early_kc[s]);
      for (long it = early; it < total; ++it) {
        const int s = (int)(it % STAGES);
        const unsigned ph = (unsigned)((it / STAGES) & 1);
        tc_mbar_wait(empty0 + 8 * s, ph ^ 1, p.status, dead);
        tc_mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        issue_a(s);
        issue_b(s, kc);
        advance();
      }
    } else {
      LL_PDL_WAIT();
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issue ------------------------------
    LL_PDL_WAIT();
    if (lane == 0) {
      // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = NT, M = 128
      constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NT >> 3) << 17) | ((128u >> 4) << 24);
      long it = 0;
      int unit_no = 0;
      for (int uu = blockIdx.x; uu < p.units; uu += gridDim.x, ++unit_no) {
        const int kp = uu % p.ksplit;
        const int kc0 = kp * p.cpp, kc1 = min(kboxes, (kp + 1) * p.cpp);
        // the epilogue of the unit before must have read the accumulator
        tc_mbar_wait(acc_empty, (unsigned)((unit_no & 1) ^ 1), p.status, dead);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kc = kc0; kc < kc1; ++kc, ++it) {
          const int s = (int)(it % STAGES);
          const unsigned ph = (unsigned)((it / STAGES) & 1);
          tc_mbar_wait(full0 + 8 * s, ph, p.status, dead);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned a_addr = stage0 + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k16 = 0; k16 < 4; ++k16)
            tc_mma(tmem, tc_desc(a_addr + 32 * k16), tc_desc(b_addr + 32 * k16), IDESC, (kc > kc0 || k16 > 0) ? 1u : 0u);
          tc_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
        }
        tc_commit(acc_full);          // the unit's accumulator is complete once all its MMAs are done
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    LL_PDL_WAIT();
#ifdef LL_TIMELINE
    if (tid == 64) {   // (the stamp is thread 0's in the other kernels; here the first epilogue thread's)
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (p.status != nullptr && blockIdx.x < LL_TIMELINE_CTAS)
        reinterpret_cast<unsigned long long*>(p.status + 4)[((size_t)((MODE == TC_MODE_PLAIN && p.ksplit == 1) ? 5 : TL_KERNEL) * LL_TIMELINE_CTAS + blockIdx.x) * 4 + 1] = t;
    }
#endif
    const int ew = warp & 3;               // the 32 tensor-memory lanes this warp may read: 32 ew .. 32 ew + 31
    const int feat_in_unit = 32 * ew + lane;
    // SCALED: the rows' factors, made while the weights stream and the MMAs run: thread (quarter ew, token lane)
    // adds the units ew, ew + 4, ... of its token, the quarters meet in shared memory (a fixed order)
    __shared__ float row_part[SCALED ? 4 : 1][64];
    __shared__ float row_scale[SCALED ? 64 : 1];
    if (SCALED) {
      float part0 = 0.f, part1 = 0.f;     // tokens lane and lane + 32
#pragma unroll 8
      for (int un = ew; un < p.sumsq_units; un += 4) {
        part0 += p.sumsq_in[(size_t)un * 64 + lane];
        part1 += p.sumsq_in[(size_t)un * 64 + 32 + lane];
      }
      row_part[ew][lane] = part0;
      row_part[ew][32 + lane] = part1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ew < 2) {
        const int t = 32 * ew + lane;
        row_scale[t] = 1.0f / sqrtf((row_part[0][t] + row_part[1][t] + row_part[2][t] + row_part[3][t]) / (float)p.K +
                                    p.norm_eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    int unit_no = 0;
    for (int uu = blockIdx.x; uu < p.units; uu += gridDim.x, ++unit_no) {
      const int u = uu / p.ksplit, kp = uu % p.ksplit;
      tc_mbar_wait(acc_full, (unsigned)(unit_no & 1), p.status, dead);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const unsigned taddr = tmem + ((unsigned)(32 * ew) << 16);
      // tensor memory -> shared memory, one accumulator row (feature) per thread; then tensor memory is free
      {
        float* mine = stg + feat_in_unit * (NT + 1);
#pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 8) {
          float v[8];
          tc_ld8(taddr + c0, v);
#pragma unroll
          for (int i = 0; i < 8; ++i) mine[c0 + i] = v[i];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(acc_empty);
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
      // shared memory -> global: a token's features of this unit are contiguous in the output
      constexpr int FE = S::FEATS;
      constexpr int CH = (OUT == 1) ? 4 : 8;  // features in a 16-byte piece
      const int e = tid - 64;
      const int f_base = u * FE;
      auto value = [&](int fl, int t) -> float {
        const float a = stg[fl * (NT + 1) + t];
        if (MODE == TC_MODE_GATED) {
          // gate and up rounded to bfloat16 first, as the unfused path does between product and activation
          const float rs = SCALED ? row_scale[t & 63] : 1.0f;
          const float gt = __bfloat162float(__float2bfloat16_rn(a * rs));
          const float uv = __bfloat162float(__float2bfloat16_rn(stg[(64 + fl) * (NT + 1) + t] * rs));
          // (x * rcp(y), not the IEEE division: that is a chain of dependent instructions with a branch an element)
          return __fdividef(gt, 1.0f + __expf(-gt)) * uv;
        }
        return a;
      };
      if (p.vec_ok) {
        for (int idx = e; idx < p.M * (FE / CH); idx += 128) {
          const int t = idx / (FE / CH), c = idx % (FE / CH);
          const int f0 = f_base + c * CH;
          if (f0 >= p.N) continue;  // N % CH == 0 on this path: a piece is inside or outside as a whole
          float v[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) v[j] = value(c * CH + j, t);
          if (OUT == 1) {
            float* dst = reinterpret_cast<float*>(p.out) + ((size_t)kp * p.M + t) * p.out_stride + f0;
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          } else {
            bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)t * p.out_stride + f0;
            uint4 pk;
            unsigned* w = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              w[j] = *reinterpret_cast<const unsigned*>(&h);
            }
            *reinterpret_cast<uint4*>(dst) = pk;
          }
        }
      } else {
        for (int idx = e; idx < p.M * FE; idx += 128) {
          const int t = idx / FE, fl = idx % FE;
          const int f = f_base + fl;
          if (f >= p.N) continue;
          const float v = value(fl, t);
          if (OUT == 1)
            reinterpret_cast<float*>(p.out)[((size_t)kp * p.M + t) * p.out_stride + f] = v;
          else
            reinterpret_cast<bf16*>(p.out)[(size_t)t * p.out_stride + f] = __float2bfloat16_rn(v);
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the staging tile may be written again
    }
  }
  // ---- everyone is done: free the tensor memory ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  LL_TIMELINE_STAMP(p.status, (MODE == TC_MODE_PLAIN && p.ksplit == 1) ? 5 : TL_KERNEL, 2);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)TMEM_COLS) : "memory");
  }
}

typedef CUresult (*tc_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tc_encode_fn tc_encoder() {
  static tc_encode_fn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (tc_encode_fn)ptr;
  }
  return fn;
}

// Tensor map of a bfloat16 matrix [rows, K] with row stride `stride` elements: boxes of box_rows x 64 k.
static int tc_make_map(CUtensorMap* map, const void* base, long rows, long K, long stride, int box_rows) {
  tc_encode_fn enc = tc_encoder();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int MODE, int NT, int OUT, bool SCALED = false>
static int tc_launch(const TcParams& p, const void* w, const void* x, long x_stride, int sm_count, cudaStream_t stream) {
  constexpr bool GATED = MODE == TC_MODE_GATED;
  CUtensorMap wmap, xmap;
  int rc = tc_make_map(&wmap, w, GATED ? 2l * p.N : (long)p.N, p.K, p.K, GATED ? 64 : 128);
  if (rc == 0) rc = tc_make_map(&xmap, x, p.M, p.K, x_stride, NT);
  if (rc != 0) return rc;
  const size_t smem = TcShape<MODE, NT>::SMEM;
  cudaFuncSetAttribute(gemm_tc_kernel<MODE, NT, OUT, SCALED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int grid = p.units < sm_count ? p.units : sm_count;
  ll_launch(gemm_tc_kernel<MODE, NT, OUT, SCALED>, dim3(grid), dim3(TC_THREADS), smem, stream, p, wmap, xmap);
  return LL_LAUNCH_RESULT();
}

// x: bfloat16 [M, K] (row stride x_stride, a multiple of 8); w: bfloat16 [N, K] contiguous (gated: [2 N, K],
// gate rows first); out: bfloat16 [M, N], or float32 with out_f32 = 1; ksplit > 1: out is float32
// [ksplit, M, N] partial sums (out_stride = N).  33 <= M <= 128 is what it is meant for; any M <= 128 works.
// sumsq (gated, M <= 64; or null): see TcParams.
extern "C" int ll_gemm_tc(void* out, long out_stride, int out_f32, const void* x, long x_stride, const void* w, int M,
                          int N, int K, int gated, int ksplit, int sm_count, const float* sumsq, int sumsq_units,
                          float norm_eps, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (sumsq != nullptr && (!gated || M > 64 || sumsq_units <= 0)) return (int)cudaErrorInvalidValue;
  if (M > 128 || K <= 0 || (K % 64) != 0 || (x_stride % 8) != 0 || sm_count <= 0 || ksplit < 1)
    return (int)cudaErrorInvalidValue;
  if ((ksplit > 1 && (!out_f32 || gated)) || (gated && out_f32)) return (int)cudaErrorInvalidValue;
  TcParams p;
  p.out = out;
  p.out_stride = out_stride;
  p.M = M;
  p.N = N;
  p.K = K;
  p.status = status;
  p.sumsq_in = sumsq;
  p.sumsq_units = sumsq_units;
  p.norm_eps = norm_eps;
  p.cpp = (K / 64 + ksplit - 1) / ksplit;
  p.ksplit = (K / 64 + p.cpp - 1) / p.cpp;
  if (p.ksplit != ksplit) return (int)cudaErrorInvalidValue;
  {
    const int ch = out_f32 ? 4 : 8;
    p.vec_ok = ((uintptr_t)out % 16 == 0 && out_stride % ch == 0 && N % ch == 0) ? 1 : 0;
  }
  p.units = gated ? (N + 63) / 64 : ((N + 127) / 128) * p.ksplit;
  const bool wide = M > 64;
  if (gated && sumsq != nullptr) return tc_launch<TC_MODE_GATED, 64, 0, true>(p, w, x, x_stride, sm_count, stream);
  if (gated) {
    return wide ? tc_launch<TC_MODE_GATED, 128, 0>(p, w, x, x_stride, sm_count, stream)
                : tc_launch<TC_MODE_GATED, 64, 0>(p, w, x, x_stride, sm_count, stream);
  }
  if (out_f32) {
    return wide ? tc_launch<TC_MODE_PLAIN, 128, 1>(p, w, x, x_stride, sm_count, stream)
                : tc_launch<TC_MODE_PLAIN, 64, 1>(p, w, x, x_stride, sm_count, stream);
  }
  return wide ? tc_launch<TC_MODE_PLAIN, 128, 0>(p, w, x, x_stride, sm_count, stream)
              : tc_launch<TC_MODE_PLAIN, 64, 0>(p, w, x, x_stride, sm_count, stream);
}
