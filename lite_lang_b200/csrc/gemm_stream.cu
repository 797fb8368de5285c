// Weight-streaming matrix product for decode: y[M, N] = x[M, K] * W[N, K]^T, bfloat16,
// float32 accumulation, M <= 32 tokens.
//
// A decode step is a stream of every weight through the SMs, so this kernel is built
// around the copy engine, not around the tensor core: persistent CTAs, each with one
// producer warp that keeps a ring of shared-memory stages filled by TMA (tiled
// cp.async.bulk.tensor.2d through a tensor map of W, boxes of 64 k x 16..64 rows with the
// 128-byte swizzle, completion counted by an mbarrier per stage; no multicast), and four
// consumer warps that feed mma.sync.m16n8k16 from the stages and hand them back through a
// second mbarrier.  Bytes in flight are bounded by shared memory (about 100 KB a CTA, two
// CTAs an SM), not by registers or occupancy, and the producer runs ahead over the end of a
// work unit, so the stream does not stop while a unit's results are written.  (One bulk
// copy per weight row was tried first: the SM's copy unit took about 35 cycles a copy
// whatever its size, so 256-byte copies capped the kernel at 2 TB/s.)
//
// The weights take the M side of the MMA (16 rows a tile), the tokens the N side.  As in
// gemm_smallm.cu the contraction index of an MMA step is mapped to 8 contiguous elements
// per thread, so a thread's A fragment is one 16-byte read from a stage row and its B
// fragment one 16-byte read of a token row.  The token rows of a stage's k range travel with
// its weights: a second tensor map (of x, boxes of 8..32 rows x 64 k) puts them behind the
// weight boxes of the stage, after griddepcontrol.wait (the weights start before it).
//
// Four shapes of work unit:
//   WIDE    64 output features x all of K; a stage is 64 rows x 128 k (two boxes); warp w
//           owns rows 16 w .. 16 w + 15.  For wide products (lm_head).
//   GATED   32 features of the SiLU-gated feed-forward; W is [2 I, K], gate rows first.
//           Warp w's tile has 8 gate rows and, as rows 8..15, the up rows of the same 8
//           features, so the thread that holds gate(f, token) also holds up(f, token)
//           and writes silu(gate) * up: the [M, 2 I] intermediate never exists.
//   QKV_ROPE  the fused q|k|v projection of an attention layer with everything that follows it: a unit
//           is 8 features of the first half of a head and their 8 rotation partners from the second half
//           (two TMA boxes of 8 rows), k split over the warps as in NARROW.  After the warps' partial
//           tiles are added, bias and rotary position encoding are applied in float32 and the results
//           go where they belong: q into the output rows, k and v into the pages of the cache.  The
//           [M, (nh + 2 nkv) hd] projection is never written and the rope/store kernel is not launched.
//   NARROW  16 features x all of K; a stage is 16 rows x 256 k (four boxes) and warp w takes
//           one box; the four partial tiles are added through shared memory.  For
//           products with few output features (q|k|v, o, down), where units, not k, are scarce.
//
// Two of them have a variant (template flag SPLIT) that takes over half of an RMS norm that lies between two
// products of a decode step, so that the norm is no kernel, and no link of the step's chain of dependent
// launches, of its own: NARROW adds its result to the residual rows, writes them times the norm's weight
// and leaves each row's sum of squares in parts of 16 columns; GATED multiplies those rows, and a sixth warp
// adds the parts up into the rows' factors 1 / sqrt(mean + eps) meanwhile, which the epilogue applies before the
// activation (see GtParams).
//
// Every wait on an mbarrier is bounded (about two seconds of clock); a wait that runs out
// sets LL_ERR_WAIT_TIMEOUT in the status word and the kernel carries on to its end.
//
// Needs K % 256 == 0 (NARROW) or K % 128 == 0 (WIDE, GATED) and 16-byte aligned rows.
// Rows of W beyond N are filled with zeros by TMA.
#include <cuda.h>

#include "common.cuh"

#define LL_ERR_WAIT_TIMEOUT 5

#define GT_CONSUMERS 4
#define GT_THREADS ((GT_CONSUMERS + 1) * 32)
#define GT_MODE_WIDE 0
#define GT_MODE_GATED 1
#define GT_MODE_NARROW 2
#define GT_MODE_QKV_ROPE 3

template <int MODE> struct GtShape;
// ROWS x KC elements a stage, made of boxes of BOX_ROWS rows x 64 k (128 bytes a row).
template <> struct GtShape<GT_MODE_WIDE> {
  static constexpr int ROWS = 64, KC = 128, BOX_ROWS = 64, STAGES = 6;
};
template <> struct GtShape<GT_MODE_GATED> {
  static constexpr int ROWS = 64, KC = 128, BOX_ROWS = 32, STAGES = 6;
};
template <> struct GtShape<GT_MODE_NARROW> {
  static constexpr int ROWS = 16, KC = 256, BOX_ROWS = 16, STAGES = 12;
};
// two boxes of 8 rows land exactly where the 16-row box of NARROW does, so the consumers are the same
template <> struct GtShape<GT_MODE_QKV_ROPE> {
  static constexpr int ROWS = 16, KC = 256, BOX_ROWS = 8, STAGES = 12;
};

__device__ __forceinline__ unsigned gt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void gt_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gt_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gt_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool gt_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds, records it, and lets the caller go on.
__device__ __forceinline__ void gt_mbar_wait(unsigned bar, unsigned parity, int* status) {
  if (gt_mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!gt_mbar_try(bar, parity)) {
    if (clock64() - t0 > 4000000000ll) {
      set_status(status, LL_ERR_WAIT_TIMEOUT);
      return;
    }
  }
}
// One TMA box: rows [y, y + box rows) x k [x, x + 64) of W into shared memory (x is a multiple of 64
// elements, i.e. of 128 bytes, as TMA's 16-byte rule on the innermost coordinate demands).
__device__ __forceinline__ void gt_tma_load(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 gt_lds16(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void gt_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gt_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GT_CONSUMERS * 32)); }

template <typename OutT> __device__ __forceinline__ OutT gt_out(float v);
template <> __device__ __forceinline__ float gt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 gt_out<bf16>(float v) { return __float2bfloat16_rn(v); }

struct GtParams {
  const bf16* x;
  void* out;
  long x_stride, out_stride;
  int M, N, K;  // N: output features (GATED: the intermediate size; W has 2 N rows)
  int units;    // feature units times ksplit
  int ksplit;   // parts the k range is cut into; > 1: out is float32 [ksplit, M, N] partial sums
  int cpp;      // k chunks (stages) per part
  // QKV_ROPE only: what follows the projection
  const float* bias;       // float32 [(nh + 2 nkv) hd] or null
  const int* positions;    // int32 [M]
  const float* cos_sin;    // float32 [max_pos, hd]: cos half, sin half
  int max_pos;
  int nh, nkv, hd;
  const int* slot_map;     // int32 [M]: cache slot of each token (-1: none)
  bf16* k_cache;
  bf16* v_cache;
  int page_size;
  long num_slots;
  // A norm between two products, split between them.  The product before the norm (NARROW to bfloat16, k not
  // split) adds its result to the residual rows, writes them back, writes them times the norm's weight as its
  // output (what the product after the norm multiplies), and leaves the sum of squares of each row's 16 values
  // of a unit in sumsq_out[unit][64].  The product after the norm (GATED) adds the units' sums of a row in a
  // fixed order and scales the row of its result by 1 / sqrt(sum / hidden + eps): the norm's reduction is off
  // the path between the two, and its kernel, a link of the chain of dependent launches, is gone.
  bf16* res;               // residual rows [M, N], row stride res_stride: read, added to, written
  long res_stride;
  const float* norm_w;     // float32 [N]
  float* sumsq_out;        // float32 [N / 16][64]
  const float* sumsq_in;   // float32 [sumsq_units][64]; null: no row factor
  int sumsq_units;
  float norm_eps, norm_inv_n;
  int* status;
};
#define GT_SUMSQ_ROWS 64   // rows of a sums-of-squares record: the most tokens the kernel takes

// What a stage holds and how many there are.  The token rows of the stage's k range travel with the weights
// (boxes of 8 MT rows x 64 k through a tensor map of x), so the consumers read both operands from shared
// memory.  (They used to read x from global memory chunk by chunk; with a handful of tokens that was a
// chain of L2 latencies inside every product: 12 % of a decode step at batch 8, 10 % at batch 32.)
template <int MODE, int MT> struct GtStage {
  using S = GtShape<MODE>;
  static constexpr int KBOXES = S::KC / 64;                 // boxes along k in a stage
  static constexpr int W_BYTES = S::ROWS * S::KC * 2;
  static constexpr int XBOX_BYTES = 8 * MT * 128;           // 8 MT token rows x 64 k
  static constexpr int STAGE_BYTES = W_BYTES + KBOXES * XBOX_BYTES;
  static constexpr int FIT = (96 * 1024) / STAGE_BYTES;     // the ring stays within 96 KB (two CTAs an SM)
  static constexpr int STAGES = FIT < S::STAGES ? FIT : S::STAGES;
};

// SPLIT: the kernel's part of a norm that is split between the products around it (see GtParams): the NARROW product
// before the norm, or the GATED product after it, which then has a sixth warp that makes the rows' factors.
// BLOCKS: more than 32 tokens (NARROW and QKV_ROPE, up to 64): the tokens in blocks of 32 along grid.y, each block
// a set of CTAs of its own that streams the weights again (they are small products; the second read finds L2).
template <int MODE, int MT, typename OutT, bool SPLIT, bool BLOCKS>
__global__ void __launch_bounds__(GT_THREADS + ((SPLIT && MODE == GT_MODE_GATED) ? 32 : 0))
gemm_stream_kernel(const GtParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
  using S = GtShape<MODE>;
  using G = GtStage<MODE, MT>;
  constexpr int KBOXES = G::KBOXES;
  constexpr int BOX_BYTES = S::BOX_ROWS * 128;       // one box: BOX_ROWS rows of 128 bytes, swizzled
  constexpr int RBOXES = S::ROWS / S::BOX_ROWS;      // boxes along the rows (GATED: gate box, up box)
  constexpr int W_BYTES = G::W_BYTES, XBOX_BYTES = G::XBOX_BYTES, STAGE_BYTES = G::STAGE_BYTES, STAGES = G::STAGES;
  extern __shared__ unsigned char smem_raw[];
  // the swizzle pattern repeats every 1024 bytes: stages start on a 1024-byte boundary
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE_BYTES);
  float* red = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 2 * STAGES * 8);   // (GATED has none of it:
  const unsigned full0 = gt_smem(bars), empty0 = gt_smem(bars + STAGES);                  //  its place holds the
  const unsigned scale_bar = gt_smem(bars + 2 * STAGES);                                   //  row factors' barrier)
  const unsigned stage0 = gt_smem(smem);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == GT_CONSUMERS * 32) {   // the producer's maps
    asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      gt_mbar_init(full0 + 8 * s, 1);
      gt_mbar_init(empty0 + 8 * s, GT_CONSUMERS);
    }
    if (SPLIT && MODE == GT_MODE_GATED) gt_mbar_init(scale_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  LL_PDL_TRIGGER();
  [[maybe_unused]] constexpr int TL_KERNEL = MODE == GT_MODE_QKV_ROPE ? 0 : MODE == GT_MODE_GATED ? 3 : MODE == GT_MODE_WIDE ? 5 : (sizeof(OutT) == 2 ? 2 : 4);
  LL_TIMELINE_STAMP(p.status, TL_KERNEL, 0);

  const int kchunks = p.K / S::KC;
  const int tok0 = BLOCKS ? (int)blockIdx.y * 8 * MT : 0;   // the first token of this CTA's block

  // ---- the rows' factors of the norm before a GATED product (SPLIT): a warp of its own adds the units' sums of
  // squares of each token in a fixed order while the others stream and multiply, and the consumers find
  // 1 / sqrt(mean + eps) in shared memory when they come to their epilogue.  Lanes: 2 MT consecutive ones hold
  // the 8 MT tokens of a unit as 16-byte pieces, so 16 / MT units are on their way at once. ----
  __shared__ float row_scale[(SPLIT && MODE == GT_MODE_GATED) ? GT_SUMSQ_ROWS : 1];
  if (SPLIT && MODE == GT_MODE_GATED && warp == GT_CONSUMERS + 1) {
    LL_PDL_WAIT();
    constexpr int LPU = 2 * MT, UPAR = 32 / LPU;   // lanes a unit, units at once
    const int piece = lane % LPU, usub = lane / LPU;
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int un = usub; un < p.sumsq_units; un += UPAR) {
      const float4 v = *reinterpret_cast<const float4*>(p.sumsq_in + (size_t)un * GT_SUMSQ_ROWS + 4 * piece);
      tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
    }
#pragma unroll
    for (int d = LPU; d < 32; d <<= 1) {   // the units' groups of lanes meet (the same order in every CTA and launch)
      tot.x += __shfl_xor_sync(0xffffffffu, tot.x, d);
      tot.y += __shfl_xor_sync(0xffffffffu, tot.y, d);
      tot.z += __shfl_xor_sync(0xffffffffu, tot.z, d);
      tot.w += __shfl_xor_sync(0xffffffffu, tot.w, d);
    }
    if (usub == 0) {
      row_scale[4 * piece] = 1.0f / sqrtf(tot.x * p.norm_inv_n + p.norm_eps);
      row_scale[4 * piece + 1] = 1.0f / sqrtf(tot.y * p.norm_inv_n + p.norm_eps);
      row_scale[4 * piece + 2] = 1.0f / sqrtf(tot.z * p.norm_inv_n + p.norm_eps);
      row_scale[4 * piece + 3] = 1.0f / sqrtf(tot.w * p.norm_inv_n + p.norm_eps);
    }
    __syncwarp();
    if (lane == 0) gt_mbar_arrive(scale_bar);   // (an arrival releases what the warp wrote before it)
    return;
  }

  if (warp == GT_CONSUMERS) {
    // ------------------------------ producer ------------------------------
    // The weights do not depend on the kernel before this one, so streaming starts at once.  The token
    // rows do: their boxes follow after griddepcontrol.wait, first for the stages already under way.
    if (lane == 0) {
      int uu = blockIdx.x, kc = 0, kc_end = 0, y[RBOXES];
      auto open_unit = [&]() {   // rows and k range of work unit uu
        if (uu >= p.units) return;
        const int u = uu / p.ksplit, kp = uu - u * p.ksplit;
        if (MODE == GT_MODE_WIDE) {
          y[0] = u * 64;
        } else if (MODE == GT_MODE_GATED) {
          y[0] = u * 32;                 // gate rows of the unit's 32 features
          y[RBOXES - 1] = p.N + u * 32;  // their up rows
        } else if (MODE == GT_MODE_QKV_ROPE) {
          const int upr = p.hd / 16;                  // units per head
          const int head = u / upr, i0 = (u - head * upr) * 8;
          y[0] = head * p.hd + i0;                    // 8 features of the first half of the head
          y[RBOXES - 1] = y[0] + p.hd / 2;            // their partners in the second half
        } else {
          y[0] = u * 16;
        }
        kc = kp * p.cpp;
        kc_end = min(kchunks, (kp + 1) * p.cpp);
      };
      auto advance = [&]() {
        if (++kc >= kc_end) {
          uu += gridDim.x;
          open_unit();
        }
      };
      auto issue_w = [&](int s) {
#pragma unroll
        for (int kb = 0; kb < KBOXES; ++kb)
#pragma unroll
          for (int rb = 0; rb < RBOXES; ++rb)
            gt_tma_load(stage0 + s * STAGE_BYTES + (kb * RBOXES + rb) * BOX_BYTES, &wmap, kc * S::KC + kb * 64, y[rb],
                        full0 + 8 * s);
      };
      auto issue_x = [&](int s, int k) {
#pragma unroll
        for (int kb = 0; kb < KBOXES; ++kb)
          gt_tma_load(stage0 + s * STAGE_BYTES + W_BYTES + kb * XBOX_BYTES, &xmap, k * S::KC + kb * 64, tok0, full0 + 8 * s);
      };
      open_unit();
      int early_kc[STAGES];
      int early = 0;
      for (; early < STAGES && uu < p.units; ++early) {   // the ring's first round: weights now
        gt_mbar_expect_tx(full0 + 8 * early, STAGE_BYTES);
        issue_w(early);
        early_kc[early] = kc;
        advance();
      }
      LL_PDL_WAIT();
      for (int s = 0; s < early; ++s) issue_x(s, early_kc[s]);   // their token rows once those exist
      for (long it = early; uu < p.units; ++it) {
        const int s = (int)(it % STAGES);
        const unsigned ph = (unsigned)((it / STAGES) & 1);
        gt_mbar_wait(empty0 + 8 * s, ph ^ 1, p.status);
        gt_mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
        issue_w(s);
        issue_x(s, kc);
        advance();
      }
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  const int g = lane >> 2, c = lane & 3;
  // the token rows are written by the kernel before this one; the producer warp does not wait (it
  // only reads weights), the consumers do, so no CTA exits before the kernel before has finished
  LL_PDL_WAIT();
  LL_TIMELINE_STAMP(p.status, TL_KERNEL, 1);
  // k boxes of a stage this warp works on, and where its two A rows sit inside a box
  constexpr bool KSPLIT_WARPS = (MODE == GT_MODE_NARROW || MODE == GT_MODE_QKV_ROPE);  // warps split k
  constexpr int MYBOXES = KSPLIT_WARPS ? 1 : KBOXES;
  const int kb0 = KSPLIT_WARPS ? warp : 0;
  unsigned row_off[2];  // byte offset of row g / row g + 8 of this warp's tile inside a k box
  if (MODE == GT_MODE_WIDE) {
    row_off[0] = (16 * warp + g) * 128;
    row_off[1] = (16 * warp + g + 8) * 128;
  } else if (MODE == GT_MODE_GATED) {
    row_off[0] = (8 * warp + g) * 128;               // gate box
    row_off[1] = BOX_BYTES + (8 * warp + g) * 128;   // up box
  } else {
    row_off[0] = g * 128;
    row_off[1] = (g + 8) * 128;
  }
  // 16-byte chunk q of a 128-byte row r sits at chunk q ^ (r & 7); all rows used here have r & 7 == g
  const unsigned sw = (unsigned)g;

  long it = 0;
  for (int uu = blockIdx.x; uu < p.units; uu += gridDim.x) {
    const int u = uu / p.ksplit, kp = uu - u * p.ksplit;
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    // QKV_ROPE: what the unit's epilogue reads from global memory (bias, the token's position and cache slot,
    // its cos and sin) is asked for now, so that it has arrived when the MMAs are done
    constexpr int EP_ITEMS = (MODE == GT_MODE_QKV_ROPE) ? (8 * 8 * MT + GT_CONSUMERS * 32 - 1) / (GT_CONSUMERS * 32) : 1;
    float ep_b0[EP_ITEMS], ep_b1[EP_ITEMS], ep_cs[EP_ITEMS], ep_sn[EP_ITEMS];
    long ep_slot[EP_ITEMS];
    if (MODE == GT_MODE_QKV_ROPE) {
      const int upr = p.hd / 16, half = p.hd / 2;
      const int head = u / upr, i0 = (u - head * upr) * 8;
#pragma unroll
      for (int e = 0; e < EP_ITEMS; ++e) {
        const int idx = tid + e * GT_CONSUMERS * 32;
        const int t = idx >> 3, j = idx & 7;
        ep_b0[e] = ep_b1[e] = 0.f;
        ep_cs[e] = 1.f;
        ep_sn[e] = 0.f;
        ep_slot[e] = -1;
        if (idx < 8 * 8 * MT && tok0 + t < p.M) {
          const int f0 = head * p.hd + i0 + j;
          if (p.bias) {
            ep_b0[e] = p.bias[f0];
            ep_b1[e] = p.bias[f0 + half];
          }
          if (head < p.nh + p.nkv) {
            int pos = p.positions[tok0 + t];
            if (pos < 0 || pos >= p.max_pos) {
              set_status(p.status, LL_ERR_POSITION_RANGE);
              pos = 0;
            }
            ep_cs[e] = p.cos_sin[(size_t)pos * p.hd + i0 + j];
            ep_sn[e] = p.cos_sin[(size_t)pos * p.hd + half + i0 + j];
          }
          if (head >= p.nh && p.slot_map) ep_slot[e] = (long)p.slot_map[tok0 + t];
        }
      }
    }
    // NARROW into the residual stream: the residual values and the norm's weights of this thread's places in the
    // unit's epilogue (token idx / 16, feature idx % 16) are asked for now, too
    constexpr bool FUSE_OK = SPLIT && MODE == GT_MODE_NARROW && sizeof(OutT) == 2;
    float fr_res[MT], fr_w[MT];
    if (FUSE_OK) {
#pragma unroll
      for (int e = 0; e < MT; ++e) {
        const int idx = tid + e * GT_CONSUMERS * 32;
        const int t = idx >> 4, n = u * 16 + (idx & 15);
        const bool ok = tok0 + t < p.M && n < p.N;
        fr_res[e] = ok ? __bfloat162float(p.res[(size_t)(tok0 + t) * p.res_stride + n]) : 0.f;
        fr_w[e] = ok ? p.norm_w[n] : 0.f;
      }
    }
    const int kc_end = min(kchunks, (kp + 1) * p.cpp);
    for (int kc = kp * p.cpp; kc < kc_end; ++kc, ++it) {
      const int s = (int)(it % STAGES);
      const unsigned ph = (unsigned)((it / STAGES) & 1);
      uint4 xv[MYBOXES][2][MT];
      gt_mbar_wait(full0 + 8 * s, ph, p.status);
      // token row 8 j + g of the stage's x box: its 16-byte chunk 4 i + c sits at chunk (4 i + c) ^ g
#pragma unroll
      for (int b = 0; b < MYBOXES; ++b)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < MT; ++j)
            xv[b][i][j] = gt_lds16(stage0 + s * STAGE_BYTES + W_BYTES + (kb0 + b) * XBOX_BYTES + (8 * j + g) * 128 +
                                   (((unsigned)(4 * i + c) ^ sw) * 16));
#pragma unroll
      for (int b = 0; b < MYBOXES; ++b) {
        const unsigned box = stage0 + s * STAGE_BYTES + (kb0 + b) * RBOXES * BOX_BYTES;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const unsigned chunk = ((unsigned)(4 * i + c) ^ sw) * 16;
          const uint4 wa = gt_lds16(box + row_off[0] + chunk);
          const uint4 wb = gt_lds16(box + row_off[1] + chunk);
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            gt_mma(acc[j], wa.x, wb.x, wa.y, wb.y, xv[b][i][j].x, xv[b][i][j].y);
            gt_mma(acc[j], wa.z, wb.z, wa.w, wb.w, xv[b][i][j].z, xv[b][i][j].w);
          }
        }
      }
      __syncwarp();
      if (lane == 0) gt_mbar_arrive(empty0 + 8 * s);
    }
    // ---- the unit's results ----
    OutT* out = reinterpret_cast<OutT*>(p.out) + (size_t)kp * p.M * p.out_stride;  // this part's [M, N] block
    if (MODE == GT_MODE_WIDE) {
      const int fa = u * 64 + 16 * warp + g, fb = fa + 8;
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        const int t0 = 8 * j + 2 * c, t1 = t0 + 1;
        if (fa < p.N) {
          if (t0 < p.M) out[(size_t)t0 * p.out_stride + fa] = gt_out<OutT>(acc[j][0]);
          if (t1 < p.M) out[(size_t)t1 * p.out_stride + fa] = gt_out<OutT>(acc[j][1]);
        }
        if (fb < p.N) {
          if (t0 < p.M) out[(size_t)t0 * p.out_stride + fb] = gt_out<OutT>(acc[j][2]);
          if (t1 < p.M) out[(size_t)t1 * p.out_stride + fb] = gt_out<OutT>(acc[j][3]);
        }
      }
    } else if (MODE == GT_MODE_GATED) {
      const int f = u * 32 + 8 * warp + g;
      if (SPLIT) gt_mbar_wait(scale_bar, 0, p.status);   // the rows' factors are in shared memory (long since)
      if (f < p.N) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int t = 8 * j + 2 * c + h;
            if (t < p.M) {
              // gate and up are rounded to bfloat16 first, as the unfused path does between product and activation
              const float rs = SPLIT ? row_scale[t] : 1.0f;
              const float gt = __bfloat162float(__float2bfloat16_rn(acc[j][h] * rs));
              const float up = __bfloat162float(__float2bfloat16_rn(acc[j][2 + h] * rs));
              out[(size_t)t * p.out_stride + f] = gt_out<OutT>(gt / (1.0f + expf(-gt)) * up);
            }
          }
        }
      }
    } else {
      constexpr int TOK = 8 * MT;
      float* r = red + (size_t)warp * 16 * TOK;
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        r[g * TOK + 8 * j + 2 * c] = acc[j][0];
        r[g * TOK + 8 * j + 2 * c + 1] = acc[j][1];
        r[(g + 8) * TOK + 8 * j + 2 * c] = acc[j][2];
        r[(g + 8) * TOK + 8 * j + 2 * c + 1] = acc[j][3];
      }
      gt_consumer_sync();
      if (MODE == GT_MODE_QKV_ROPE) {
        // rows 0..7: features i0 + j of the head, rows 8..15: their partners i0 + j + hd/2
        const int upr = p.hd / 16, half = p.hd / 2;
        const int head = u / upr, i0 = (u - head * upr) * 8;
#pragma unroll
        for (int e = 0; e < EP_ITEMS; ++e) {
          const int idx = tid + e * GT_CONSUMERS * 32;
          const int t = idx >> 3, j = idx & 7;
          if (idx >= 8 * TOK || tok0 + t >= p.M) continue;
          float x0 = 0.f, x1 = 0.f;
#pragma unroll
          for (int wi = 0; wi < GT_CONSUMERS; ++wi) {
            x0 += red[((size_t)wi * 16 + j) * TOK + t];
            x1 += red[((size_t)wi * 16 + j + 8) * TOK + t];
          }
          // the unfused path rounds the projection to bfloat16 before bias and rotation: the same here
          x0 = __bfloat162float(__float2bfloat16_rn(x0)) + ep_b0[e];
          x1 = __bfloat162float(__float2bfloat16_rn(x1)) + ep_b1[e];
          const int f0 = head * p.hd + i0 + j;
          if (head < p.nh + p.nkv) {
            const float r0v = x0 * ep_cs[e] - x1 * ep_sn[e], r1v = x0 * ep_sn[e] + x1 * ep_cs[e];
            x0 = r0v;
            x1 = r1v;
          }
          const bf16 o0 = __float2bfloat16_rn(x0), o1 = __float2bfloat16_rn(x1);
          if (head < p.nh) {
            bf16* q = reinterpret_cast<bf16*>(p.out) + (size_t)(tok0 + t) * p.out_stride + f0;
            q[0] = o0;
            q[half] = o1;
          } else {
            long slot = ep_slot[e];
            if (slot >= p.num_slots) {
              set_status(p.status, LL_ERR_SLOT_RANGE);
              slot = -1;
            }
            if (slot >= 0) {
              const bool is_k = head < p.nh + p.nkv;
              const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
              const long page = slot / p.page_size;
              const int off = (int)(slot - page * p.page_size);
              bf16* dst = (is_k ? p.k_cache : p.v_cache) + (((size_t)page * p.nkv + kvh) * p.page_size + off) * p.hd +
                          i0 + j;
              dst[0] = o0;
              dst[half] = o1;
            }
          }
        }
      } else if (FUSE_OK) {
        // h += product (both rounded as the separate kernels round them: the product to bfloat16, then the sum);
        // out = h * w, what the product after the norm multiplies; the 16 lanes of a token add their squares
#pragma unroll
        for (int e = 0; e < MT; ++e) {
          const int idx = tid + e * GT_CONSUMERS * 32;
          const int t = idx >> 4, f = idx & 15;
          const bool ok = tok0 + t < p.M && u * 16 + f < p.N;
          float sum = 0.f;
#pragma unroll
          for (int wi = 0; wi < GT_CONSUMERS; ++wi) sum += red[((size_t)wi * 16 + f) * TOK + t];
          float hn = 0.f;
          if (ok) {
            hn = __bfloat162float(__float2bfloat16_rn(fr_res[e] + __bfloat162float(__float2bfloat16_rn(sum))));
            p.res[(size_t)(tok0 + t) * p.res_stride + u * 16 + f] = __float2bfloat16_rn(hn);
            out[(size_t)(tok0 + t) * p.out_stride + u * 16 + f] = gt_out<OutT>(hn * fr_w[e]);
          }
          float sq = hn * hn;
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          sq += __shfl_xor_sync(0xffffffffu, sq, 8);
          if (f == 0) p.sumsq_out[(size_t)u * GT_SUMSQ_ROWS + tok0 + t] = sq;   // (rows beyond M hold 0)
        }
      } else {
        for (int idx = tid; idx < 16 * TOK; idx += GT_CONSUMERS * 32) {
          const int t = idx >> 4, f = idx & 15;
          if (tok0 + t < p.M && u * 16 + f < p.N) {
            float sum = 0.f;
#pragma unroll
            for (int wi = 0; wi < GT_CONSUMERS; ++wi) sum += red[((size_t)wi * 16 + f) * TOK + t];
            out[(size_t)(tok0 + t) * p.out_stride + u * 16 + f] = gt_out<OutT>(sum);
          }
        }
      }
      gt_consumer_sync();
    }
  }
  LL_TIMELINE_STAMP(p.status, TL_KERNEL, 2);
}

typedef CUresult (*gt_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static gt_encode_fn gt_encoder() {
  static gt_encode_fn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (gt_encode_fn)ptr;
  }
  return fn;
}

// Tensor map of a bfloat16 matrix [rows, K] (rows row_stride elements apart; 0: K) with boxes of box_rows rows
// x 64 k, 128-byte swizzle.  Rows beyond the matrix read as zeros.
static int gt_make_map(CUtensorMap* map, const void* w, long rows, long K, int box_rows, long row_stride = 0) {
  gt_encode_fn enc = gt_encoder();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)(row_stride > 0 ? row_stride : K) * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int MODE, int MT, typename OutT, bool SPLIT, bool BLOCKS = false>
static int gt_launch(const GtParams& p, const void* w, int sm_count, cudaStream_t stream) {
  using S = GtShape<MODE>;
  using G = GtStage<MODE, MT>;
  CUtensorMap map, xmap;
  const long w_rows = (MODE == GT_MODE_GATED) ? 2l * p.N : p.N;
  int rc = gt_make_map(&map, w, w_rows, p.K, S::BOX_ROWS);
  if (rc != 0) return rc;
  rc = gt_make_map(&xmap, p.x, p.M, p.K, 8 * MT, p.x_stride);   // token rows: boxes of 8 MT rows, zeros beyond M
  if (rc != 0) return rc;
  const size_t smem = 1024 + (size_t)G::STAGES * G::STAGE_BYTES + 2 * G::STAGES * 8 + 8 +   // (+ the row factors' barrier)
                      ((MODE == GT_MODE_NARROW || MODE == GT_MODE_QKV_ROPE) ? sizeof(float) * GT_CONSUMERS * 16 * 8 * MT : 0);
  cudaFuncSetAttribute(gemm_stream_kernel<MODE, MT, OutT, SPLIT, BLOCKS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  // two CTAs an SM (one an SM, so that the next product's CTAs could move in early, was measured slower)
  const int blocks = BLOCKS ? (p.M + 8 * MT - 1) / (8 * MT) : 1;
  const int room = 2 * sm_count / blocks;
  const int grid = p.units < room ? p.units : room;
  const int threads = GT_THREADS + ((SPLIT && MODE == GT_MODE_GATED) ? 32 : 0);
  ll_launch(gemm_stream_kernel<MODE, MT, OutT, SPLIT, BLOCKS>, dim3(grid, blocks), dim3(threads), smem, stream, p, map, xmap);
  return LL_LAUNCH_RESULT();
}

template <int MODE, typename OutT, bool SPLIT = false>
static int gt_dispatch_m(const GtParams& p, const void* w, int sm_count, cudaStream_t stream) {
  if (p.M <= 8) return gt_launch<MODE, 1, OutT, SPLIT>(p, w, sm_count, stream);
  if (p.M <= 16) return gt_launch<MODE, 2, OutT, SPLIT>(p, w, sm_count, stream);
  if constexpr ((MODE == GT_MODE_NARROW || MODE == GT_MODE_QKV_ROPE) && sizeof(OutT) == 2) {
    // 17 to 32 tokens of a small product (a unit a CTA in both blocks at once): two blocks of 16 tokens, which
    // stream the weights twice (the second time from L2) but keep six stages in the ring where tiles of 32 tokens
    // leave four (a decode step at batch 17 1.62 -> 1.55 ms, 24 1.61 -> 1.52, 32 1.66 -> 1.56; two blocks of 8 for
    // 9 to 16 tokens: no difference; with k = 2,048, the o projection of the 3B sizes: none either, or 1 % worse)
    if (p.M > 16 && p.M <= 32 && p.ksplit == 1 && 2 * p.units <= 2 * sm_count && p.K <= 1536)
      return gt_launch<MODE, 2, OutT, SPLIT, true>(p, w, sm_count, stream);
  }
  if (p.M <= 32) return gt_launch<MODE, 4, OutT, SPLIT>(p, w, sm_count, stream);
  if constexpr ((MODE == GT_MODE_NARROW || MODE == GT_MODE_QKV_ROPE) && sizeof(OutT) == 2) {
    if (p.M <= 64 && p.ksplit == 1) return gt_launch<MODE, 4, OutT, SPLIT, true>(p, w, sm_count, stream);
  }
  return (int)cudaErrorInvalidValue;
}

// mode: 0 wide, 1 gated, 2 narrow.  x: bfloat16 [M, K] with row stride x_stride; w: bfloat16
// [N, K] contiguous (gated: [2 N, K]); out: [M, N] bfloat16, or float32 with out_f32 = 1
// (not for gated).  ksplit > 1 cuts the k range into that many parts, each a work unit of
// its own: out must then be float32 [ksplit, M, N] (out_stride = N) and receives partial
// sums that the caller adds (the fused residual-and-norm kernel does).
// sm_count: SMs of the device (the grid is at most two CTAs an SM).
extern "C" int ll_gemm_stream(void* out, long out_stride, int out_f32, const void* x, long x_stride, const void* w,
                              int M, int N, int K, int mode, int ksplit, int sm_count, int* status,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (x_stride % 8) != 0 || sm_count <= 0 || ksplit < 1) return (int)cudaErrorInvalidValue;
  // (33 to 64 tokens: units of 16 features to bfloat16 only, in two blocks of tokens)
  if (M > 32 && (mode != GT_MODE_NARROW || out_f32 || ksplit != 1)) return (int)cudaErrorInvalidValue;
  if (ksplit > 1 && (!out_f32 || mode == GT_MODE_GATED)) return (int)cudaErrorInvalidValue;
  GtParams p = {};
  p.x = (const bf16*)x;
  p.out = out;
  p.x_stride = x_stride;
  p.out_stride = out_stride;
  p.M = M;
  p.N = N;
  p.K = K;
  p.status = status;
  if (mode == GT_MODE_WIDE) {
    if (K % 128) return (int)cudaErrorInvalidValue;
    p.cpp = (K / 128 + ksplit - 1) / ksplit;
    p.ksplit = (K / 128 + p.cpp - 1) / p.cpp;
    if (p.ksplit != ksplit) return (int)cudaErrorInvalidValue;  // the caller's partial buffer would not fit
    p.units = ((N + 63) / 64) * p.ksplit;
    return out_f32 ? gt_dispatch_m<GT_MODE_WIDE, float>(p, w, sm_count, stream)
                   : gt_dispatch_m<GT_MODE_WIDE, bf16>(p, w, sm_count, stream);
  }
  if (mode == GT_MODE_GATED) {
    if (K % 128 || out_f32) return (int)cudaErrorInvalidValue;
    p.cpp = K / 128;
    p.ksplit = 1;
    p.units = (N + 31) / 32;
    return gt_dispatch_m<GT_MODE_GATED, bf16>(p, w, sm_count, stream);
  }
  if (mode == GT_MODE_NARROW) {
    if (K % 256) return (int)cudaErrorInvalidValue;
    p.cpp = (K / 256 + ksplit - 1) / ksplit;
    p.ksplit = (K / 256 + p.cpp - 1) / p.cpp;
    if (p.ksplit != ksplit) return (int)cudaErrorInvalidValue;
    p.units = ((N + 15) / 16) * p.ksplit;
    return out_f32 ? gt_dispatch_m<GT_MODE_NARROW, float>(p, w, sm_count, stream)
                   : gt_dispatch_m<GT_MODE_NARROW, bf16>(p, w, sm_count, stream);
  }
  return (int)cudaErrorInvalidValue;
}

// The product before a norm and the product after it, with the norm split between them (see GtParams).
// ll_gemm_stream_into_norm: res[M, N] += x W^T (bfloat16, rounded as a separate product and sum would be), out[M, N] =
// res * norm_w, sumsq[N / 16][64] = the sums of squares of each row's 16 values of a unit.  K % 256 == 0, N % 16 == 0.
// ll_gemm_stream_gated_scaled: the gated product of rows that are only multiplied by the norm's weight yet; each
// row of the result is scaled by 1 / sqrt(sum over units of sumsq[unit][row] / hidden + eps) before the activation.
extern "C" int ll_gemm_stream_into_norm(void* out, long out_stride, void* res, long res_stride, const float* norm_w,
                                        float* sumsq, const void* x, long x_stride, const void* w, int M, int N, int K,
                                        int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K % 256) != 0 || (N % 16) != 0 || (x_stride % 8) != 0 || sm_count <= 0 || res == nullptr ||
      norm_w == nullptr || sumsq == nullptr)
    return (int)cudaErrorInvalidValue;
  GtParams p = {};
  p.x = (const bf16*)x;
  p.out = out;
  p.x_stride = x_stride;
  p.out_stride = out_stride;
  p.M = M;
  p.N = N;
  p.K = K;
  p.status = status;
  p.cpp = K / 256;
  p.ksplit = 1;
  p.units = N / 16;
  p.res = (bf16*)res;
  p.res_stride = res_stride;
  p.norm_w = norm_w;
  p.sumsq_out = sumsq;
  return gt_dispatch_m<GT_MODE_NARROW, bf16, true>(p, w, sm_count, stream);
}

extern "C" int ll_gemm_stream_gated_scaled(void* out, long out_stride, const void* x, long x_stride, const void* w,
                                           int M, int N, int K, const float* sumsq, int sumsq_units, float eps,
                                           int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K <= 0 || (K % 128) != 0 || (x_stride % 8) != 0 || sm_count <= 0 || sumsq == nullptr || sumsq_units <= 0)
    return (int)cudaErrorInvalidValue;
  GtParams p = {};
  p.x = (const bf16*)x;
  p.out = out;
  p.x_stride = x_stride;
  p.out_stride = out_stride;
  p.M = M;
  p.N = N;
  p.K = K;
  p.status = status;
  p.cpp = K / 128;
  p.ksplit = 1;
  p.units = (N + 31) / 32;
  p.sumsq_in = sumsq;
  p.sumsq_units = sumsq_units;
  p.norm_eps = eps;
  p.norm_inv_n = 1.0f / (float)K;
  return gt_dispatch_m<GT_MODE_GATED, bf16, true>(p, w, sm_count, stream);
}

// The fused q|k|v projection of an attention layer (mode QKV_ROPE): qkv = x W^T (+ bias), q and k
// rotated by the token's position (half-split pairs over the whole head), q written to
// out[t, head * hd + i] (out: bfloat16 [M, >= nh * hd], row stride out_stride), k and v written into the
// cache plane at slot_map[t].  w: bfloat16 [(nh + 2 nkv) hd, K]; K % 256 == 0; hd % 16 == 0; M <= 64 (more than 32: two blocks of tokens).
extern "C" int ll_gemm_stream_qkv_rope(void* out, long out_stride, const void* x, long x_stride, const void* w, int M,
                                       int K, const float* bias, const int* positions, const float* cos_sin,
                                       int max_pos, int nh, int nkv, int hd, const int* slot_map, void* k_cache,
                                       void* v_cache, int page_size, long num_slots, int sm_count, int* status,
                                       cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 64 || K <= 0 || (K % 256) != 0 || (x_stride % 8) != 0 || sm_count <= 0 || hd <= 0 || (hd % 16) != 0 ||
      nh <= 0 || nkv <= 0 || positions == nullptr || cos_sin == nullptr)
    return (int)cudaErrorInvalidValue;
  GtParams p = {};
  p.x = (const bf16*)x;
  p.out = out;
  p.x_stride = x_stride;
  p.out_stride = out_stride;
  p.M = M;
  p.N = (nh + 2 * nkv) * hd;
  p.K = K;
  p.status = status;
  p.cpp = K / 256;
  p.ksplit = 1;
  p.units = (nh + 2 * nkv) * (hd / 16);
  p.bias = bias;
  p.positions = positions;
  p.cos_sin = cos_sin;
  p.max_pos = max_pos;
  p.nh = nh;
  p.nkv = nkv;
  p.hd = hd;
  p.slot_map = slot_map;
  p.k_cache = (bf16*)k_cache;
  p.v_cache = (bf16*)v_cache;
  p.page_size = page_size;
  p.num_slots = num_slots;
  return gt_dispatch_m<GT_MODE_QKV_ROPE, bf16>(p, w, sm_count, stream);
}
