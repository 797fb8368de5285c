// Matrix product for many tokens (portions of prompts) on the fifth-generation tensor cores, two SMs a tile:
// y[M, N] = x[M, K] * W[N, K]^T, bfloat16, float32 accumulation in tensor memory, and the gated
// feed-forward's silu(x Wg^T) * (x Wu^T) with the activation in the epilogue, so that the gate and up
// products never go to memory (a library product writes them and a second kernel reads them back:
// 110 MB of traffic a layer at 2,048 tokens of the 1.5B sizes).
//
// The tokens are the M side of the MMA here (a token is a lane of tensor memory, its features are columns),
// so a thread of the epilogue holds gate and up of the same token and feature side by side.
//
// A tile is 256 tokens x 256 columns, made by a pair of CTAs on two SMs (a thread-block cluster of two,
// tcgen05 with cta_group::2): each CTA brings 128 token rows (A) and 128 weight rows (B) of every 64-wide
// k block into its own shared memory by TMA (no multicast: the pair's two halves of B are different rows)
// and holds the accumulator rows of its own 128 tokens in its own tensor memory; the even CTA of the pair
// issues the MMAs (256 x 256 x 16), which read both CTAs' shared memory and write both tensor memories.
// In gated mode the even CTA's weight rows are 128 gate features and the odd CTA's the up rows of the same
// features: columns 0..127 of the accumulator are gate, 128..255 up.
// In q|k|v mode a tile's 256 columns are whole heads (head size 64, 128 or 256), and the epilogue does what
// follows the projection: bias, the half-split rotation of q and k by the token's position (both halves of a
// head are columns of the same lane), q to its output, k and v into the token's slot of the paged cache.  The
// q|k|v row never goes to memory and one kernel stands for two.
//
// Roles in a CTA (320 threads):
//   warp 0    producer: one thread keeps a ring of six 32 KB stages filled (four in q|k|v mode, whose epilogue
//             takes the room of two for its staging tile); both CTAs' copies complete on the even CTA's
//             `full` barrier of the stage;
//   warp 1    MMA: in the even CTA one thread issues the MMAs of a stage when it is full, and a
//             tcgen05.commit hands the stage back to both producers; the accumulator is double-buffered
//             (2 x 256 columns), so the MMAs of the next tile run while this one's epilogue reads;
//   warps 2-9 epilogue: tensor memory -> registers -> activation -> 16-byte stores of the thread's own row
//             (q|k|v mode: -> shared memory, then rows finished by consecutive threads); a warp reads the 32
//             lanes that its number modulo 4 gives, so two warps share a token row and each takes half of the
//             tile's columns (a pair with one tile has nothing to hide its epilogue behind).
// Tiles go to the pairs round-robin, tokens fastest, so the pairs that run together share weight rows in L2.
//
// Every mbarrier wait is bounded (about two seconds of clock): a wait that runs out records
// LL_ERR_WAIT_TIMEOUT and the kernel carries on to its end, frees its tensor memory and returns.  The two
// CTAs' tensor-memory allocations must be at the same columns; the kernel checks that and otherwise records
// LL_ERR_TMEM_PAIR and computes nothing.
//
// Needs K % 8 == 0 and 16-byte aligned rows; rows beyond M or N and k beyond K are zero-filled by TMA.
#include <cuda.h>

#include "common.cuh"

#define LL_ERR_WAIT_TIMEOUT 5
#define LL_ERR_TMEM_PAIR 7
#define GP_THREADS 320
#define GP_STAGES 6
#define GP_A_BYTES (128 * 128)
#define GP_STAGE_BYTES (2 * GP_A_BYTES)
#define GP_MODE_PLAIN 0
#define GP_MODE_GATED 1
#define GP_MODE_QKV 2
#define GP_SMEM (1024 + GP_STAGES * GP_STAGE_BYTES + (2 * GP_STAGES + 4) * 8 + 16)

__device__ __forceinline__ unsigned gp_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gp_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gp_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrive on a barrier of a CTA of the cluster (the address comes from gp_mapa)
__device__ __forceinline__ void gp_mbar_arrive_cluster(unsigned bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ bool gp_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// `dead` is the calling thread's memory of a wait that ran out: after the first one it waits no more.
__device__ __forceinline__ void gp_mbar_wait(unsigned bar, unsigned parity, int* status, bool& dead) {
  if (dead || gp_mbar_try(bar, parity)) return;
  const long long t0 = clock64();
  while (!gp_mbar_try(bar, parity)) {
    if (clock64() - t0 > 4000000000ll) {
      set_status(status, LL_ERR_WAIT_TIMEOUT);
      dead = true;
      return;
    }
  }
}
__device__ __forceinline__ unsigned gp_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void gp_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster
__device__ __forceinline__ unsigned gp_mapa(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ unsigned gp_ld_cluster(unsigned addr_cluster) {
  unsigned v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr_cluster) : "memory");
  return v;
}
// TMA box into this CTA's shared memory; its bytes complete on a barrier that may be the pair's other CTA's
__device__ __forceinline__ void gp_tma_load(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the 128-byte
// swizzle (what TMA writes): groups of 8 rows are 1024 bytes apart; 16 elements of k are 32 bytes.
__device__ __forceinline__ unsigned long long gp_desc(unsigned smem_addr) {
  return (unsigned long long)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void gp_mma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                       unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair when the MMAs issued so far are done
__device__ __forceinline__ void gp_commit_pair(unsigned bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void gp_ld32_issue(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// (the registers are tied to the wait so that no use of them can be scheduled before it)
__device__ __forceinline__ void gp_ld_wait(unsigned (&a)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
                 "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(a[16]),
                 "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]), "+r"(a[22]), "+r"(a[23]), "+r"(a[24]),
                 "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]), "+r"(a[29]), "+r"(a[30]), "+r"(a[31])
               :
               : "memory");
}
__device__ __forceinline__ void gp_ld_wait2(unsigned (&a)[32], unsigned (&b)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]), "+r"(a[8]),
                 "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]), "+r"(a[15]), "+r"(a[16]),
                 "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]), "+r"(a[22]), "+r"(a[23]), "+r"(a[24]),
                 "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]), "+r"(a[29]), "+r"(a[30]), "+r"(a[31]), "+r"(b[0]),
                 "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]),
                 "+r"(b[10]), "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]), "+r"(b[16]), "+r"(b[17]),
                 "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]), "+r"(b[24]), "+r"(b[25]),
                 "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31])
               :
               : "memory");
}

struct GpParams {
  bf16* out;
  long out_stride;
  int M, N, K;      // tokens, output features (gated: the intermediate size; W has 2 N rows), inner size
  int m_tiles;      // tiles of 256 tokens
  int tiles;        // m_tiles x column tiles (plain: 256 features a tile, gated: 128)
  int vec_ok;       // the output takes 16-byte pieces (aligned base and stride, N a multiple of 8)
  int* status;
  // q|k|v mode only: what follows the projection (N = (nh + 2 nkv) hd; out is q [M, nh hd])
  const float* bias;      // float32 [N] or null
  const int* positions;   // int32 [M]
  const float* cos_sin;   // float32 [max_pos, hd]: cos of the hd/2 angles, then sin
  int max_pos, nh, nkv, hd;
  const int* slot_map;    // int32 [M] or null (no cache write); slot = page * page_size + offset, -1 skips
  bf16* k_cache;          // [num_pages, nkv, page_size, hd]
  bf16* v_cache;
  int page_size;
  long num_slots;
};

// 32 accumulator columns -> 32 bfloat16 features of the thread's row, from column f0 on
__device__ __forceinline__ void gp_store32(const GpParams& p, bf16* row, int f0, const float (&v)[32]) {
  if (p.vec_ok && f0 + 32 <= p.N) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 pk;
      unsigned* w = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
        w[j] = *reinterpret_cast<const unsigned*>(&h);
      }
      *reinterpret_cast<uint4*>(row + f0 + 8 * q) = pk;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (f0 + i < p.N) row[f0 + i] = __float2bfloat16_rn(v[i]);
  }
}

// 32 values -> 32 bfloat16 at dst (16-byte aligned)
__device__ __forceinline__ void gp_put32(bf16* dst, const float (&v)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 pk;
    unsigned* w = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
      w[j] = *reinterpret_cast<const unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(dst + 8 * q) = pk;
  }
}
// The q|k|v epilogue works in two steps, because a thread that owns a token row (a lane of tensor memory) would
// read its own row of the cos/sin table and write its own rows of q and of the cache: 32 different lines an
// instruction.  Step 1: the accumulator tile goes to shared memory, rounded to bfloat16 (as the unfused path
// sees the product), [128 rows][256 columns], the 16-byte pieces of every 128 bytes XOR-swizzled by the row.
// Step 2: consecutive threads take consecutive pieces of a row, as the stand-alone rotation kernel does.
#define GP_STG_BYTES (128 * 512)
__device__ __forceinline__ unsigned gp_stg_offset(int row, int piece) {   // piece: 8 columns
  return (unsigned)(row * 512 + (((piece & ~7) | ((piece ^ row) & 7)) << 4));
}
// step 1 for 32 columns of the thread's row
__device__ __forceinline__ void gp_stage32(unsigned char* stg, int row, int col0, const unsigned (&a)[32]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 pk;
    unsigned* w = reinterpret_cast<unsigned*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(a[8 * q + 2 * j]), __uint_as_float(a[8 * q + 2 * j + 1]));
      w[j] = *reinterpret_cast<const unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(stg + gp_stg_offset(row, (col0 >> 3) + q)) = pk;
  }
}
__device__ __forceinline__ void gp_unpack8(const uint4& a, float (&x)[8]) {
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(a2[k]);
    x[2 * k] = f.x;
    x[2 * k + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 gp_pack8(const float (&x)[8]) {
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);
  return o;
}
// step 2 for the CTA's 128 rows.  A work item is 8 columns of the first half of a head and their 8 partners in
// the second half; a row has 16 of them, and epilogue thread e (of 256) takes item e % 16 of the rows
// e / 16 + 16 k, k = 0..7: the same head and columns in eight rows.  What it needs from global memory for
// that (bias, the rows' positions and cache slots) does not depend on the product and is read while the MMAs
// of the tile still run (gp_qkv_prepare); the rows' cos and sin are asked for one row ahead.
struct GpQkvPrep {
  int pos[8];
  int slot[8];
  float b0[8], b1[8];
};
__device__ __forceinline__ void gp_qkv_prepare(const GpParams& p, int e, int row0, int head0, GpQkvPrep& w) {
  const int hd = p.hd, half = hd >> 1, per_head = half >> 3;
  const int pi = e & 15, hl = pi / per_head, i0 = (pi - hl * per_head) << 3, h = head0 + hl;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int row = row0 + (e >> 4) + 16 * k;
    w.pos[k] = row < p.M ? p.positions[row] : 0;
    w.slot[k] = (row < p.M && p.slot_map != nullptr) ? p.slot_map[row] : -1;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) w.b0[j] = w.b1[j] = 0.f;
  if (p.bias != nullptr && h < p.nh + 2 * p.nkv) {
    const float* bb = p.bias + (size_t)h * hd + i0;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const float4 x = __ldg(reinterpret_cast<const float4*>(bb) + q);
      const float4 y = __ldg(reinterpret_cast<const float4*>(bb + half) + q);
      w.b0[4 * q] = x.x; w.b0[4 * q + 1] = x.y; w.b0[4 * q + 2] = x.z; w.b0[4 * q + 3] = x.w;
      w.b1[4 * q] = y.x; w.b1[4 * q + 1] = y.y; w.b1[4 * q + 2] = y.z; w.b1[4 * q + 3] = y.w;
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (w.pos[k] < 0 || w.pos[k] >= p.max_pos) {
      set_status(p.status, LL_ERR_POSITION_RANGE);
      w.pos[k] = 0;
    }
    if ((long)w.slot[k] >= p.num_slots) {
      set_status(p.status, LL_ERR_SLOT_RANGE);
      w.slot[k] = -1;
    }
  }
}
__device__ __forceinline__ void gp_qkv_finish(const GpParams& p, const unsigned char* stg, int e, int row0, int head0,
                                              const GpQkvPrep& w) {
  const int hd = p.hd, half = hd >> 1, per_head = half >> 3;
  const int pi = e & 15, hl = pi / per_head, i0 = (pi - hl * per_head) << 3, h = head0 + hl;
  if (h >= p.nh + 2 * p.nkv) return;
  const bool rotate = h < p.nh + p.nkv;   // q or k head; v heads: bias and store
  const int piece = (hl * hd + i0) >> 3;
  float4 cs[4];                           // cos (2) and sin (2) of the row in hand
  auto ask = [&](int k, float4 (&t)[4]) {
    const float* src = p.cos_sin + (size_t)w.pos[k] * hd + i0;
    t[0] = __ldg(reinterpret_cast<const float4*>(src));
    t[1] = __ldg(reinterpret_cast<const float4*>(src) + 1);
    t[2] = __ldg(reinterpret_cast<const float4*>(src + half));
    t[3] = __ldg(reinterpret_cast<const float4*>(src + half) + 1);
  };
  if (rotate) ask(0, cs);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int r = (e >> 4) + 16 * k, row = row0 + r;
    float4 nxt[4];
    if (rotate && k + 1 < 8) ask(k + 1, nxt);
    bf16* dst = nullptr;
    if (row < p.M) {
      if (h < p.nh) {
        dst = p.out + (size_t)row * p.out_stride + (size_t)h * hd;
      } else if (w.slot[k] >= 0) {
        const int page = w.slot[k] / p.page_size;
        const int off = w.slot[k] - page * p.page_size;
        dst = rotate ? p.k_cache + (((size_t)page * p.nkv + (h - p.nh)) * p.page_size + off) * hd
                     : p.v_cache + (((size_t)page * p.nkv + (h - p.nh - p.nkv)) * p.page_size + off) * hd;
      }
    }
    if (dst != nullptr) {
      float x0[8], x1[8];
      gp_unpack8(*reinterpret_cast<const uint4*>(stg + gp_stg_offset(r, piece)), x0);
      gp_unpack8(*reinterpret_cast<const uint4*>(stg + gp_stg_offset(r, piece + (half >> 3))), x1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        x0[j] += w.b0[j];
        x1[j] += w.b1[j];
      }
      if (rotate) {
        const float c[8] = {cs[0].x, cs[0].y, cs[0].z, cs[0].w, cs[1].x, cs[1].y, cs[1].z, cs[1].w};
        const float sn[8] = {cs[2].x, cs[2].y, cs[2].z, cs[2].w, cs[3].x, cs[3].y, cs[3].z, cs[3].w};
        float o0[8], o1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o0[j] = x0[j] * c[j] - x1[j] * sn[j];
          o1[j] = x0[j] * sn[j] + x1[j] * c[j];
        }
        *reinterpret_cast<uint4*>(dst + i0) = gp_pack8(o0);
        *reinterpret_cast<uint4*>(dst + i0 + half) = gp_pack8(o1);
      } else {
        *reinterpret_cast<uint4*>(dst + i0) = gp_pack8(x0);
        *reinterpret_cast<uint4*>(dst + i0 + half) = gp_pack8(x1);
      }
    }
    if (rotate && k + 1 < 8) {
#pragma unroll
      for (int j = 0; j < 4; ++j) cs[j] = nxt[j];
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(GP_THREADS)
gemm_pair_kernel(const GpParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
  // (q|k|v mode gives two of the six stages' room to its epilogue's staging tile)
  constexpr int STAGES = (MODE == GP_MODE_QKV) ? GP_STAGES - GP_STG_BYTES / GP_STAGE_BYTES : GP_STAGES;
  constexpr int STAGE_BYTES = GP_STAGE_BYTES, A_BYTES = GP_A_BYTES;
  constexpr int COLS = (MODE == GP_MODE_GATED) ? 128 : 256;   // output features a tile
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + GP_STAGES * STAGE_BYTES);
  unsigned char* stg = smem + STAGES * STAGE_BYTES;   // q|k|v mode only
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * GP_STAGES + 4);
  const unsigned stage0 = gp_smem(smem);
  const unsigned full0 = gp_smem(bars), empty0 = gp_smem(bars + GP_STAGES);
  const unsigned acc_full0 = gp_smem(bars + 2 * GP_STAGES), acc_empty0 = gp_smem(bars + 2 * GP_STAGES + 2);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = gp_cluster_rank();   // 0: issues the MMAs and owns the `full` and `acc_empty` barriers
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;   // the pair is a cluster of two along x
  if (tid == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
  }
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      gp_mbar_init(full0 + 8 * s, 1);    // the even CTA's producer announces both CTAs' bytes
      gp_mbar_init(empty0 + 8 * s, 1);   // one commit
    }
    for (int b = 0; b < 2; ++b) {
      gp_mbar_init(acc_full0 + 8 * b, 1);    // one commit
      gp_mbar_init(acc_empty0 + 8 * b, 16);  // the eight epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // all of this SM's tensor memory: two accumulators of 256 columns; both CTAs take part
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gp_smem(tmem_slot)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  gp_cluster_sync();   // both CTAs' barriers are initialised and both allocations are known
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = *tmem_slot;
  const bool paired = gp_ld_cluster(gp_mapa(gp_smem(tmem_slot), rank ^ 1u)) == tmem;
  if (!paired && tid == 0) set_status(p.status, LL_ERR_TMEM_PAIR);
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();

  bool dead = false;
  const int kboxes = (p.K + 63) / 64;
  if (paired) {
    if (warp == 0) {
      // ------------------------------ producer ------------------------------
      if (lane == 0) {
        long it = 0;
        for (int t = pair; t < p.tiles; t += pairs) {
          const int mt = t % p.m_tiles, nt = t / p.m_tiles;
          const int x_row = mt * 256 + (int)rank * 128;
          const int w_row = (MODE == GP_MODE_GATED) ? (int)rank * p.N + nt * 128 : nt * 256 + (int)rank * 128;
          for (int kc = 0; kc < kboxes; ++kc, ++it) {
            const int s = (int)(it % STAGES);
            const unsigned ph = (unsigned)((it / STAGES) & 1);
            if (it >= STAGES) gp_mbar_wait(empty0 + 8 * s, ph ^ 1, p.status, dead);
            if (rank == 0) gp_mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
            const unsigned bar = gp_mapa(full0 + 8 * s, 0);
            gp_tma_load(stage0 + s * STAGE_BYTES, &xmap, kc * 64, x_row, bar);
            gp_tma_load(stage0 + s * STAGE_BYTES + A_BYTES, &wmap, kc * 64, w_row, bar);
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issue (even CTA) ------------------------------
      if (lane == 0 && rank == 0) {
        // instruction descriptor: float32 accumulate, bfloat16 A and B, both K-major, N = 256, M = 256 (the pair's)
        constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
        long it = 0;
        int tl = 0;
        for (int t = pair; t < p.tiles; t += pairs, ++tl) {
          const int b = tl & 1;
          // both CTAs' epilogues of the tile before last must have read this accumulator
          gp_mbar_wait(acc_empty0 + 8 * b, (unsigned)(((tl >> 1) & 1) ^ 1), p.status, dead);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const unsigned acc = tmem + (unsigned)(b * 256);
          for (int kc = 0; kc < kboxes; ++kc, ++it) {
            const int s = (int)(it % STAGES);
            const unsigned ph = (unsigned)((it / STAGES) & 1);
            gp_mbar_wait(full0 + 8 * s, ph, p.status, dead);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned a_addr = stage0 + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16)
              gp_mma(acc, gp_desc(a_addr + 32 * k16), gp_desc(b_addr + 32 * k16), IDESC, (kc > 0 || k16 > 0) ? 1u : 0u);
            gp_commit_pair(empty0 + 8 * s);   // the stage is free in both CTAs once these MMAs have read it
          }
          gp_commit_pair(acc_full0 + 8 * b);  // the tile's accumulator is complete once all its MMAs are done
        }
      }
    } else {
      // ------------------------------ epilogue (warps 2..9) ------------------------------
      const int ew = warp & 3;          // the 32 tensor-memory lanes this warp may read: 32 ew .. 32 ew + 31
      const int eh = (warp - 2) >> 2;   // which half of the tile's columns it takes
      const unsigned acc_empty_lead = gp_mapa(acc_empty0, 0);
      int tl = 0;
      for (int t = pair; t < p.tiles; t += pairs, ++tl) {
        const int mt = t % p.m_tiles, nt = t / p.m_tiles;
        const int b = tl & 1;
        const int row = mt * 256 + (int)rank * 128 + 32 * ew + lane;
        GpQkvPrep prep;
        if (MODE == GP_MODE_QKV) gp_qkv_prepare(p, tid - 64, mt * 256 + (int)rank * 128, nt * (256 / p.hd), prep);
        gp_mbar_wait(acc_full0 + 8 * b, (unsigned)((tl >> 1) & 1), p.status, dead);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned taddr = tmem + ((unsigned)(32 * ew) << 16) + (unsigned)(b * 256);
        if (MODE == GP_MODE_QKV) {
          const int r = 32 * ew + lane;
#pragma unroll 1
          for (int c = eh * 4; c < eh * 4 + 4; ++c) {
            unsigned a[32];
            gp_ld32_issue(taddr + 32 * c, a);
            gp_ld_wait(a);
            gp_stage32(stg, r, 32 * c, a);
          }
        } else {
        bf16* out_row = p.out + (size_t)(row < p.M ? row : 0) * p.out_stride;
#pragma unroll 1
        for (int c = eh * (COLS / 64); c < (eh + 1) * (COLS / 64); ++c) {
          float v[32];
          if (MODE == GP_MODE_GATED) {
            unsigned g[32], u[32];
            gp_ld32_issue(taddr + 32 * c, g);
            gp_ld32_issue(taddr + 128 + 32 * c, u);
            gp_ld_wait2(g, u);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              // gate and up rounded to bfloat16 first, as the unfused path does between product and activation
              const float gt = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[i])));
              const float uv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
              // (x * rcp(y) instead of the IEEE division: that one's chain of dependent instructions with a
              //  branch an element, on the one warp a scheduler has here, made the epilogue twice as long as the MMAs)
              v[i] = __fdividef(gt, 1.0f + __expf(-gt)) * uv;
            }
          } else {
            unsigned a[32];
            gp_ld32_issue(taddr + 32 * c, a);
            gp_ld_wait(a);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(a[i]);
          }
          if (row < p.M) gp_store32(p, out_row, nt * COLS + 32 * c, v);
        }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) gp_mbar_arrive_cluster(acc_empty_lead + 8 * b);
        if (MODE == GP_MODE_QKV) {
          asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps: the staged tile is complete
          gp_qkv_finish(p, stg, tid - 64, mt * 256 + (int)rank * 128, nt * (256 / p.hd), prep);
          asm volatile("bar.sync 1, 256;" ::: "memory");   // it may be overwritten by the next tile
        }
      }
    }
  }
  // ---- everyone is done, in both CTAs (nobody's shared or tensor memory is still in use): free ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  gp_cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

typedef CUresult (*gp_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static gp_encode_fn gp_encoder() {
  static gp_encode_fn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (gp_encode_fn)ptr;
  }
  return fn;
}

// Tensor map of a bfloat16 matrix [rows, K] with row stride `stride` elements: boxes of 128 rows x 64 k.
static int gp_make_map(CUtensorMap* map, const void* base, long rows, long K, long stride) {
  gp_encode_fn enc = gp_encoder();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// Pairs of CTAs that can be resident at once (a pair needs two SMs of one GPU processing cluster)
template <int MODE>
static int gp_max_pairs(int sm_count) {
  static int cached = -1;
  if (cached < 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count & ~1, 1, 1);
    cfg.blockDim = dim3(GP_THREADS);
    cfg.dynamicSmemBytes = GP_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<MODE>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    cached = n < sm_count / 2 ? n : sm_count / 2;
  }
  return cached;
}

template <int MODE>
static int gp_launch(GpParams& p, const void* w, const void* x, long x_stride, int sm_count, cudaStream_t stream) {
  constexpr bool GATED = MODE == GP_MODE_GATED;
  CUtensorMap wmap, xmap;
  int rc = gp_make_map(&wmap, w, GATED ? 2l * p.N : (long)p.N, p.K, p.K);
  if (rc == 0) rc = gp_make_map(&xmap, x, p.M, p.K, x_stride);
  if (rc != 0) return rc;
  cudaFuncSetAttribute(gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GP_SMEM);
  const int cols = GATED ? 128 : 256;
  p.m_tiles = (p.M + 255) / 256;
  p.tiles = p.m_tiles * ((p.N + cols - 1) / cols);
  const int most = gp_max_pairs<MODE>(sm_count);
  const int pairs = p.tiles < most ? p.tiles : most;
  // a pair is a cluster of two CTAs along x (what a kernel with cta_group::2 instructions is launched as)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GP_THREADS);
  cfg.dynamicSmemBytes = GP_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = ll_pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE>, p, wmap, xmap);
  return LL_LAUNCH_RESULT();
}

// x: bfloat16 [M, K] (row stride x_stride, a multiple of 8); w: bfloat16 [N, K] contiguous (gated: [2 N, K],
// gate rows first); out: bfloat16 [M, N] (gated: silu(gate) * up).  Any M; meant for hundreds of tokens and more.
extern "C" int ll_gemm_pair(void* out, long out_stride, const void* x, long x_stride, const void* w, int M, int N,
                            int K, int gated, int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (x_stride % 8) != 0 || sm_count < 2) return (int)cudaErrorInvalidValue;
  GpParams p;
  p.out = reinterpret_cast<bf16*>(out);
  p.out_stride = out_stride;
  p.M = M;
  p.N = N;
  p.K = K;
  p.status = status;
  p.vec_ok = ((uintptr_t)out % 16 == 0 && out_stride % 8 == 0 && N % 8 == 0) ? 1 : 0;
  p.bias = nullptr;
  p.positions = nullptr;
  p.cos_sin = nullptr;
  p.slot_map = nullptr;
  p.k_cache = p.v_cache = nullptr;
  p.max_pos = p.nh = p.nkv = p.hd = p.page_size = 0;
  p.num_slots = 0;
  return gated ? gp_launch<GP_MODE_GATED>(p, w, x, x_stride, sm_count, stream)
               : gp_launch<GP_MODE_PLAIN>(p, w, x, x_stride, sm_count, stream);
}

// The q|k|v projection of an attention layer with what follows it: qkv = x W^T (+ bias), q and k rotated by
// the token's position (half-split pairs, whole head), q -> q_out [M, nh hd] (bfloat16, row stride q_stride),
// k and v -> the cache plane at slot_map[token] (null: no cache write).  w: [(nh + 2 nkv) hd, K]; head size 64,
// 128 or 256; cos_sin: float32 [max_pos, hd]; bias: float32 or null.
extern "C" int ll_gemm_pair_qkv_rope(void* q_out, long q_stride, const void* x, long x_stride, const void* w, int M, int K,
                                     const float* bias, const int* positions, const float* cos_sin, int max_pos, int nh,
                                     int nkv, int hd, const int* slot_map, void* k_cache, void* v_cache, int page_size,
                                     long num_slots, int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (x_stride % 8) != 0 || sm_count < 2 || (hd != 64 && hd != 128 && hd != 256) || nh <= 0 ||
      nkv <= 0 || positions == nullptr || cos_sin == nullptr || (q_stride % 8) != 0 || (uintptr_t)q_out % 16 != 0 ||
      (bias != nullptr && (uintptr_t)bias % 16 != 0) || (uintptr_t)cos_sin % 16 != 0 ||
      (slot_map != nullptr && (k_cache == nullptr || v_cache == nullptr || page_size <= 0 || (uintptr_t)k_cache % 16 != 0 ||
                               (uintptr_t)v_cache % 16 != 0)))
    return (int)cudaErrorInvalidValue;
  GpParams p;
  p.out = reinterpret_cast<bf16*>(q_out);
  p.out_stride = q_stride;
  p.M = M;
  p.N = (nh + 2 * nkv) * hd;
  p.K = K;
  p.status = status;
  p.vec_ok = 1;
  p.bias = bias;
  p.positions = positions;
  p.cos_sin = cos_sin;
  p.max_pos = max_pos;
  p.nh = nh;
  p.nkv = nkv;
  p.hd = hd;
  p.slot_map = slot_map;
  p.k_cache = reinterpret_cast<bf16*>(k_cache);
  p.v_cache = reinterpret_cast<bf16*>(v_cache);
  p.page_size = page_size;
  p.num_slots = num_slots;
  return gp_launch<GP_MODE_QKV>(p, w, x, x_stride, sm_count, stream);
}
