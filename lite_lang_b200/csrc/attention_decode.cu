// Decode attention on tensor cores, transposed: one new token per request, bfloat16.
//
// attention_mma.cu puts the (token, head) rows on the M side of mma.sync.m16n8k16; with one token a
// request only `group` of its 16 rows carry a query head.  Here the product is transposed: the 16 keys
// of a tile are the M side and the group's query heads (at most 8) the N side,
//     S^T[16 keys x 8 heads] = K[16 x hd] Q^T[hd x 8],      O^T[hd x 8 heads] += V^T[hd x 16 keys] P^T[16 x 8],
// which halves the MMAs, the accumulator registers and the softmax work per tile (8 columns instead of
// 16 rows) and leaves room for three CTAs an SM.  P^T moves from the accumulator layout to the B-operand
// layout with two movmatrix transposes.  Keys and values come through a ring of DEPTH tiles a warp in
// shared memory, filled with cp.async DEPTH tiles ahead (loads straight into registers kept too few bytes
// in flight: the compiler holds them back behind the softmax of the tile before); the ring's first round
// is asked for before the wait for the kernel before this one, which writes the new token's row only.
// They are read from the ring with 16-byte loads by the same freedom as in attention_mma.cu: the contraction index is mapped to 8
// contiguous head dimensions per thread (Q K^T), and the output rows of an MMA tile are mapped so that a
// thread's eight values of a key row serve four tiles (P V; two keys are paired by a byte permute).  The
// 16-byte chunks of a row are XOR-swizzled by the row so that both read patterns are conflict-free.
//
// One CTA (4 or 8 warps) works on one (entry, kv head, split of the keys); its warps take the split's 16-key
// tiles in turn and are merged through shared memory.  The splits of an (entry, kv head) are the CTAs of
// one thread-block cluster (1, 2, 4 or 8) and merge through distributed shared memory: every CTA
// finishes a slice of the head dimensions, which the others send to it with stores into its shared memory
// before the cluster's one barrier.  No scratch memory, no counters, nothing spins (the cluster
// barrier is the hardware's; every CTA of a cluster reaches it, early exits are the same for all of them).
// A variant (OUTER) for very few requests with very long contexts gives an (entry, kv head) several such clusters,
// each with a range of the keys; their slices of the result meet in scratch memory, where the last CTA of a
// slice to arrive (a counter, no spinning) adds them up.
//
// Head sizes 64 and 128, groups of at most 8 query heads, pages of a multiple of 16 tokens.
#include "common.cuh"

#define AD_TILE 16
#define AD_HEADS 8
#define AD_BT_CACHE 256

struct AttnDecodeParams {
  const bf16* q;
  long q_stride;
  bf16* out;
  long out_stride;
  const bf16* k_cache;
  const bf16* v_cache;
  const int* block_table;
  int bt_stride;
  const int* ctx_len;
  const int* req_slot;
  int n_entries;
  int nh, nkv, group;
  int page_size, num_pages;
  int window;
  float scale_log2;
  int nsplit;
  // (after `status`:) Few requests with very long contexts: `nouter` clusters a (entry, kv head), each with a range of the keys of its
  // own; a cluster's CTAs leave their slices of its partial result (unnormalised sums, maximum and sum of every
  // head) in scratch memory, and the last of the `nouter` CTAs of a slice to arrive (a counter a slice, zero
  // between launches) adds them up and writes the output.
  int* status;
  int nouter;
  float* scratch;     // [entries * nkv * nouter][nsplit][AD_HEADS][HD / nsplit + 2]
  int* counters;      // [entries * nkv * nsplit]
};

__device__ __forceinline__ void ad_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ad_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned ad_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ uint4 ad_ldg16(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// transpose of an 8x8 matrix of 16-bit values held one row-pair per thread
__device__ __forceinline__ unsigned ad_movmatrix(unsigned x) {
  unsigned y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ void ad_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned ad_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in CTA `rank` of the cluster, of what is at `local` in this CTA's shared memory
__device__ __forceinline__ unsigned ad_peer_addr(const void* local, unsigned rank) {
  unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
  return ra;
}
__device__ __forceinline__ void ad_st_peer(unsigned addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void ad_st_peer2(unsigned addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void ad_st_peer4(unsigned addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// OUTER: several clusters a (entry, kv head) (see AttnDecodeParams; a variant of its own, so that the ordinary
// kernel carries none of its code: with it in, a decode step at batch 1 to 16 was 3 to 5 % slower)
template <int HD, int NW, int DEPTH, bool OUTER>
__global__ void __launch_bounds__(NW * 32) attn_decode_kernel(const AttnDecodeParams p) {
  constexpr int KS = HD / 32;   // 16-byte loads per key row and thread for Q K^T
  constexpr int VS = HD / 64;   // 16-byte loads per value row and thread
  constexpr int MT = HD / 16;   // MMA row tiles of O^T
  // (the warps' partial outputs, [NW][AD_HEADS][HD + 4] floats, are laid over the ring of tiles when the loop is over)
  __shared__ float sm_m[NW][AD_HEADS];
  __shared__ float sm_l[NW][AD_HEADS];
  __shared__ int sm_bt[AD_BT_CACHE];
  // what the other CTAs of the cluster send for the slice of dims that this CTA finishes: [sender][head][dim of
  // the slice] (8 HD values whatever the cluster's size), and every sender's maximum and sum per head
  __shared__ __align__(16) float rx_o[AD_HEADS * HD];
  __shared__ float rx_m[8][AD_HEADS];
  __shared__ float rx_l[8][AD_HEADS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int e = blockIdx.x, kvh = blockIdx.y;
  const int split = OUTER ? (int)(blockIdx.z % p.nsplit) : (int)blockIdx.z;
  [[maybe_unused]] const int outer = OUTER ? (int)(blockIdx.z / p.nsplit) : 0;
  if (e >= p.n_entries) return;
  LL_PDL_TRIGGER();   // the kernel after this one may move in and fetch its weights while this one works
  LL_TIMELINE_STAMP(p.status, 1, 0);
  // What the step's index arrays say (slot, context length, block table) was uploaded before the step's
  // first kernel and is read before the wait for the kernel before this one; q and the new token's key
  // and value are that kernel's output and are read after it.
  const int slot = p.req_slot[e];
  const int ctx = p.ctx_len[e];
  const int pos = ctx;  // position of the new token; it looks at keys lo..pos
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int t_first = lo / AD_TILE, t_last = pos / AD_TILE;
  const int ntiles = t_last - t_first + 1;
  // (OUTER: the tiles of this cluster first, then of this CTA among them)
  const int tpo = OUTER ? (ntiles + p.nouter - 1) / p.nouter : ntiles;
  const int o_begin = OUTER ? t_first + outer * tpo : t_first;
  const int o_end = OUTER ? min(t_last + 1, o_begin + tpo) : t_last + 1;
  const int tps = OUTER ? (max(o_end - o_begin, 0) + p.nsplit - 1) / p.nsplit : (ntiles + p.nsplit - 1) / p.nsplit;
  const int t_begin = o_begin + split * tps;
  const int t_end = OUTER ? max(t_begin, min(o_end, t_begin + tps)) : min(t_last + 1, t_begin + tps);
  const int* bt = p.block_table + (size_t)max(slot, 0) * p.bt_stride;
  const int nt_split = t_end - t_begin;
  const bool bt_cached = nt_split <= AD_BT_CACHE;
  if (bt_cached && slot >= 0)
    for (int i = tid; i < nt_split; i += (NW * 32)) sm_bt[i] = bt[((t_begin + i) * AD_TILE) / p.page_size];
  __syncthreads();
  // ---- the warp's ring of tiles in shared memory ----
  // A warp's tiles (16 keys: 16 rows of K and of V, HD * 2 bytes each) are copied into its own ring of
  // DEPTH stages with cp.async, 16 bytes a lane and instruction, DEPTH tiles ahead of the one being
  // worked on: with a few hundred keys a split the loop is a chain of memory latencies, and the ring
  // shortens it by that factor; with many requests it keeps enough bytes in flight for the bandwidth.
  // The 16-byte piece j of row r sits at piece j ^ swizzle(r), chosen so that the fragment reads below
  // (K: rows g, g + 8, pieces 4 s + c; V: rows 2 c (+1, +8, +9), pieces 8 h + g) hit all banks once.
  constexpr int ROW_BYTES = HD * 2, CH = HD / 8;           // pieces a row
  constexpr int TILE_BYTES = AD_TILE * ROW_BYTES;           // K (or V) of a tile
  extern __shared__ __align__(16) unsigned char ad_ring[];
  unsigned char* my_ring = ad_ring + (size_t)warp * DEPTH * 2 * TILE_BYTES;
  const unsigned ring_addr = (unsigned)__cvta_generic_to_shared(my_ring);
  auto tile_base = [&](int t) -> long {   // < 0: the table's entry is no page of the pool
    const int key0 = t * AD_TILE;
    const int page = bt_cached ? sm_bt[t - t_begin] : bt[key0 / p.page_size];
    if (page < 0 || page >= p.num_pages) return -1;
    return (((long)page * p.nkv + kvh) * p.page_size + (key0 % p.page_size)) * HD;
  };
  auto issue_tile = [&](int stage, int t) {   // the whole warp; always one group, empty beyond the split's end
    const long tb = (t < t_end) ? tile_base(t) : -1;
    if (tb >= 0) {
      const unsigned kdst = ring_addr + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
#pragma unroll
      for (int i = 0; i < AD_TILE * CH / 32; ++i) {
        const int idx = lane + 32 * i, r = idx / CH, j = idx % CH;
        const bf16* ksrc = p.k_cache + tb + (long)r * HD + 8 * j;
        const bf16* vsrc = p.v_cache + tb + (long)r * HD + 8 * j;
        const unsigned kd = kdst + r * ROW_BYTES + ((j ^ (4 * (r & 1))) << 4);
        const unsigned vd = vdst + r * ROW_BYTES + ((j ^ (2 * ((r >> 1) & 3))) << 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kd), "l"(ksrc) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vd), "l"(vsrc) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // The kernel before this one writes the new token's key and value only: every tile but the one that holds
  // position `pos` was written by earlier steps and may be asked for before that kernel has finished.  The
  // ring's first round goes out here (with few keys a split that is all of them: the loop below then finds its
  // tiles in shared memory instead of meeting a memory latency a tile), and each lane asks L2 for one of the
  // warp's later tiles (K and V, contiguous within a page), so that those meet L2's latency instead of
  // memory's; the last tile is left alone.  L2 is only asked while the step's keys and values are a small part
  // of it (few requests, where the loop is a chain of latencies; with many, the loop is bound by bandwidth and
  // L2 could not hold what was asked for).
  constexpr unsigned TILE_B = AD_TILE * HD * 2;
  int filled = 0;   // tiles of the ring's first round that are under way
  if (slot >= 0) {
    for (; filled < DEPTH; ++filled) {
      const int t = t_begin + warp + filled * NW;
      if (t >= t_end || t == t_last) break;
      issue_tile(filled, t);
    }
    if ((long)gridDim.x * gridDim.y * gridDim.z * nt_split * 2 * TILE_B <= (48l << 20)) {
      for (int t = t_begin + warp + (DEPTH + lane) * NW; t < t_end; t += 32 * NW) {
        if (t == t_last) continue;
        const long off = tile_base(t);
        if (off < 0) continue;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.k_cache + off), "r"(TILE_B) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.v_cache + off), "r"(TILE_B) : "memory");
      }
    }
  }
  LL_PDL_WAIT();
  LL_TIMELINE_STAMP(p.status, 1, 1);
  // ---- Q^T fragments: thread (g, c) holds head g, dims 32 s + 8 c .. + 7 ----
  uint4 qf[KS];
  {
    const bool hv = g < p.group;
    const bf16* qr = p.q + (size_t)e * p.q_stride + (size_t)(kvh * p.group + (hv ? g : 0)) * HD + 8 * c;
#pragma unroll
    for (int s = 0; s < KS; ++s) qf[s] = hv ? ad_ldg16(qr + 32 * s) : make_uint4(0, 0, 0, 0);
  }
  if (slot < 0) {  // padding entry of a captured step: zeros, no reads (the same for the whole cluster)
    if (split == 0 && (!OUTER || outer == 0))
      for (int i = tid; i < p.group * HD; i += (NW * 32))
        p.out[(size_t)e * p.out_stride + (size_t)kvh * p.group * HD + i] = __float2bfloat16_rn(0.f);
    return;
  }
  // The cluster's merge below writes into the other CTAs' shared memory, which needs them to have started:
  // every CTA says so here and checks it only when it gets there (by then it costs nothing).
  if (p.nsplit > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  auto lds16 = [&](unsigned addr) -> uint4 {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
  };

  float o_acc[MT][4];  // O^T tile (h, jj): rows = dims 64 h + 8 g + jj and + 4, columns = heads 2c, 2c + 1
#pragma unroll
  for (int t = 0; t < MT; ++t) o_acc[t][0] = o_acc[t][1] = o_acc[t][2] = o_acc[t][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // heads 2c and 2c + 1

  // tiles t_begin + warp, + NW, ...: the rest of the ring's first round (the tile with the new token, and
  // empty groups beyond the split's end, so that group i is tile i's)
  for (; filled < DEPTH; ++filled) issue_tile(filled, t_begin + warp + filled * NW);
  int it = 0;
  for (int t = t_begin + warp; t < t_end; t += NW, ++it) {
    const int stage = it % DEPTH;
    asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");   // this lane's copies of tile `it` are in
    __syncwarp();                                                           // and so are the other lanes'
    const long tb = tile_base(t);
    if (tb < 0) {   // (nothing was copied; the stage takes the tile DEPTH ahead like any other)
      if (lane == 0) set_status(p.status, LL_ERR_PAGE_RANGE);
      issue_tile(stage, t + DEPTH * NW);
      continue;
    }
    const unsigned kst = ring_addr + stage * 2 * TILE_BYTES, vst = kst + TILE_BYTES;
    uint4 ka[KS], kb[KS], vv[VS][4];
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      ka[s] = lds16(kst + g * ROW_BYTES + (((4 * s + c) ^ (4 * (g & 1))) << 4));          // key g
      kb[s] = lds16(kst + (g + 8) * ROW_BYTES + (((4 * s + c) ^ (4 * (g & 1))) << 4));    // key g + 8
    }
    // ---- S^T = K Q^T: rows = keys g and g + 8, columns = heads 2c, 2c + 1 ----
    float s_acc[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      ad_mma(s_acc, ka[s].x, kb[s].x, ka[s].y, kb[s].y, qf[s].x, qf[s].y);
      ad_mma(s_odd, ka[s].z, kb[s].z, ka[s].w, kb[s].w, qf[s].z, qf[s].w);
    }
    // ---- scale, mask, online softmax per head (column) ----
    const int key0 = t * AD_TILE;
    const bool boundary = (key0 + AD_TILE - 1 > pos) || (key0 < lo);
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      float v = (s_acc[x] + s_odd[x]) * p.scale_log2;
      if (boundary) {
        const int j = key0 + g + 8 * (x >> 1);
        if (j > pos || j < lo) v = -INFINITY;
      }
      s_acc[x] = v;
      tmax[x & 1] = fmaxf(tmax[x & 1], v);
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 4));
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 8));
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 16));
      const float m_new = fmaxf(m_run[i], tmax[i]);
      msafe[i] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[i] = ad_exp2(m_run[i] - msafe[i]);
      m_run[i] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float pv = ad_exp2(s_acc[x] - msafe[x & 1]);
      s_acc[x] = pv;
      psum[x & 1] += pv;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
    // P^T as the B operand: (keys 2c, 2c+1 | 2c+8, 2c+9; head g) from (key g | g+8; heads 2c, 2c+1)
    const unsigned b0 = ad_movmatrix(ad_pack(s_acc[0], s_acc[1]));
    const unsigned b1 = ad_movmatrix(ad_pack(s_acc[2], s_acc[3]));
#pragma unroll
    for (int h = 0; h < VS; ++h) {
      const unsigned sw = (unsigned)(2 * (c & 3));   // rows 2 c, 2 c + 1, 2 c + 8, 2 c + 9 share the swizzle
      const unsigned piece = ((unsigned)(8 * h + g) ^ sw) << 4;
      vv[h][0] = lds16(vst + (2 * c) * ROW_BYTES + piece);
      vv[h][1] = lds16(vst + (2 * c + 1) * ROW_BYTES + piece);
      vv[h][2] = lds16(vst + (2 * c + 8) * ROW_BYTES + piece);
      vv[h][3] = lds16(vst + (2 * c + 9) * ROW_BYTES + piece);
    }
    // the stage's rows are in registers: it takes the tile DEPTH ahead
    __syncwarp();
    issue_tile(stage, t + DEPTH * NW);
    // keys that the token may not see have probability 0 by selection, but what their rows of V hold (left by an
    // earlier owner of the page, possibly Inf or NaN) would still spoil the product: zeros by selection too
    if (boundary) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = key0 + 2 * c + (i & 1) + 8 * (i >> 1);
        if (j > pos || j < lo) {
#pragma unroll
          for (int h = 0; h < VS; ++h) vv[h][i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    // ---- O^T = O^T * alpha + V^T P^T ----
    const bool rescale = (alpha[0] != 1.f) || (alpha[1] != 1.f);
#pragma unroll
    for (int h = 0; h < VS; ++h) {
      const unsigned* w0 = reinterpret_cast<const unsigned*>(&vv[h][0]);
      const unsigned* w1 = reinterpret_cast<const unsigned*>(&vv[h][1]);
      const unsigned* w2 = reinterpret_cast<const unsigned*>(&vv[h][2]);
      const unsigned* w3 = reinterpret_cast<const unsigned*>(&vv[h][3]);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int T = h * 4 + jj;
        // element jj of a 16-byte load is word jj / 2, half jj % 2; element 4 + jj is word 2 + jj / 2
        const unsigned sel = (jj & 1) ? 0x7632u : 0x5410u;
        const unsigned a0 = __byte_perm(w0[jj >> 1], w1[jj >> 1], sel);          // dim 8g+jj,   keys 2c, 2c+1
        const unsigned a1 = __byte_perm(w0[2 + (jj >> 1)], w1[2 + (jj >> 1)], sel);  // dim 8g+4+jj, keys 2c, 2c+1
        const unsigned a2 = __byte_perm(w2[jj >> 1], w3[jj >> 1], sel);          // dim 8g+jj,   keys 2c+8, 2c+9
        const unsigned a3 = __byte_perm(w2[2 + (jj >> 1)], w3[2 + (jj >> 1)], sel);
        if (rescale) {
          o_acc[T][0] *= alpha[0];
          o_acc[T][1] *= alpha[1];
          o_acc[T][2] *= alpha[0];
          o_acc[T][3] *= alpha[1];
        }
        ad_mma(o_acc[T], a0, a1, a2, a3, b0, b1);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  LL_TIMELINE_STAMP(p.status, 1, 3);   // (the tile loop is over)

  // ---- merge the four warps (rows of the merge = heads) ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 4);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 8);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 16);
  }
  // every warp is done with its ring (its last copies were waited for in the loop): the partial outputs go there
  static_assert(sizeof(float) * NW * AD_HEADS * (HD + 4) <= (size_t)NW * DEPTH * 2 * TILE_BYTES, "sm_o fits the ring");
  float (*sm_o)[AD_HEADS][HD + 4] = reinterpret_cast<float (*)[AD_HEADS][HD + 4]>(ad_ring);
  __syncthreads();
  if (g == 0) {
    sm_m[warp][2 * c] = m_run[0];
    sm_m[warp][2 * c + 1] = m_run[1];
    sm_l[warp][2 * c] = l_run[0];
    sm_l[warp][2 * c + 1] = l_run[1];
  }
#pragma unroll
  for (int T = 0; T < MT; ++T) {
    const int h = T >> 2, jj = T & 3;
    const int d0 = 64 * h + 8 * g + jj, d1 = d0 + 4;
    sm_o[warp][2 * c][d0] = o_acc[T][0];
    sm_o[warp][2 * c + 1][d0] = o_acc[T][1];
    sm_o[warp][2 * c][d1] = o_acc[T][2];
    sm_o[warp][2 * c + 1][d1] = o_acc[T][3];
  }
  __syncthreads();
  constexpr int CPR = (NW * 32) / AD_HEADS;  // 16 threads per head
  constexpr int DPT = HD / CPR;               // 8 or 4 dims per thread
  const int row = tid / CPR, dbase = (tid % CPR) * DPT;
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < NW; ++w) M = fmaxf(M, sm_m[w][row]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f, wgt[NW];
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    wgt[w] = ad_exp2(sm_m[w][row] - Ms);
    L += sm_l[w][row] * wgt[w];
  }
  float acc[DPT];
#pragma unroll
  for (int d = 0; d < DPT; ++d) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) a += sm_o[w][row][dbase + d] * wgt[w];
    acc[d] = a;
  }
  if (p.nsplit == 1) {
    if (row < p.group) {
      bf16* orow = p.out + (size_t)e * p.out_stride + (size_t)(kvh * p.group + row) * HD + dbase;
      const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
      for (int d = 0; d < DPT; d += 2)
        *reinterpret_cast<unsigned*>(orow + d) = ad_pack(acc[d] * inv, acc[d + 1] * inv);
    }
    LL_TIMELINE_STAMP(p.status, 1, 2);
    return;
  }
  // ---- the splits are the CTAs of one cluster: each finishes a slice of the dims of all heads ----
  // Every CTA sends each of its partial sums to the CTA that finishes that dim (stores into the peer's shared
  // memory, which nobody waits for one by one), then one cluster barrier, then everybody reads only its own
  // shared memory: nothing of a CTA is read by another one after the barrier, so it may leave at once.
  const int cs = p.nsplit;
  const unsigned rank = ad_cluster_rank();
  const int slice = HD / cs;                     // dims a CTA finishes: 8 .. 64 (a multiple of DPT)
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // (the arrive is above the tile loop)
  {
    const unsigned owner = (unsigned)(dbase / slice);
    const int ds = dbase - (int)owner * slice;
    const unsigned dst = ad_peer_addr(&rx_o[((int)rank * AD_HEADS + row) * slice + ds], owner);
    if (DPT == 8) {
      ad_st_peer4(dst, acc[0], acc[1], acc[2], acc[3]);
      ad_st_peer4(dst + 16, acc[DPT - 4], acc[DPT - 3], acc[DPT - 2], acc[DPT - 1]);
    } else if (DPT == 4) {
      ad_st_peer4(dst, acc[0], acc[1], acc[2], acc[3]);
    } else {
      ad_st_peer2(dst, acc[0], acc[1]);
    }
    // a head's maximum and sum go to every CTA: the head's CPR threads share the cs receivers among them
    const int j = tid % CPR;
    if (j < cs) {
      ad_st_peer(ad_peer_addr(&rx_m[rank][row], (unsigned)j), M);
      ad_st_peer(ad_peer_addr(&rx_l[rank][row], (unsigned)j), L);
    }
  }
  ad_cluster_sync();
  const int outputs = AD_HEADS * slice;          // 64 .. 512
  const int per = max(1, outputs / (NW * 32));  // 1 .. 4 consecutive dims of one head per thread
  const bool worker = tid * per < outputs;
  const int o0 = worker ? tid * per : 0;
  const int row2 = o0 / slice, dl = o0 - row2 * slice;
  float Mg = -INFINITY;
#pragma unroll
  for (int sI = 0; sI < 8; ++sI)
    if (sI < cs) Mg = fmaxf(Mg, rx_m[sI][row2]);
  const float Mgs = (Mg == -INFINITY) ? 0.f : Mg;
  float Lg = 0.f, fin[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int sI = 0; sI < 8; ++sI)
    if (sI < cs) {
      const float ws = ad_exp2(rx_m[sI][row2] - Mgs);
      Lg += rx_l[sI][row2] * ws;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < per) fin[k] += rx_o[(sI * AD_HEADS + row2) * slice + dl + k] * ws;
    }
  if (OUTER) {
    // ---- several clusters a (entry, kv head): the slice's partial results meet in scratch memory ----
    __shared__ int sm_last;
    const int pair = e * p.nkv + kvh;
    const int rec = AD_HEADS * (slice + 2);     // floats of a slice's record: [head][slice dims, maximum, sum]
    float* mine = p.scratch + (((size_t)pair * p.nouter + outer) * cs + rank) * rec;
    if (worker) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < per) mine[row2 * (slice + 2) + dl + k] = fin[k];
      if (dl == 0) {
        mine[row2 * (slice + 2) + slice] = Mg;
        mine[row2 * (slice + 2) + slice + 1] = Lg;
      }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* cnt = p.counters + (size_t)pair * cs + rank;
      const int old = atomicAdd(cnt, 1);
      sm_last = old == p.nouter - 1;
      if (sm_last) *cnt = 0;     // ready for the next launch
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    if (worker && row2 < p.group) {
      const float* base = p.scratch + ((size_t)pair * p.nouter * cs + rank) * rec + row2 * (slice + 2);
      float Mt = -INFINITY;
      for (int o = 0; o < p.nouter; ++o) Mt = fmaxf(Mt, __ldcg(base + (size_t)o * cs * rec + slice));
      const float Mts = (Mt == -INFINITY) ? 0.f : Mt;
      float Lt = 0.f, tot[4] = {0.f, 0.f, 0.f, 0.f};
      for (int o = 0; o < p.nouter; ++o) {
        const float* r = base + (size_t)o * cs * rec;
        const float wo = ad_exp2(__ldcg(r + slice) - Mts);
        Lt += __ldcg(r + slice + 1) * wo;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < per) tot[k] += __ldcg(r + dl + k) * wo;
      }
      bf16* o2 = p.out + (size_t)e * p.out_stride + (size_t)(kvh * p.group + row2) * HD + (int)rank * slice + dl;
      const float inv = Lt > 0.f ? 1.0f / Lt : 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < per) o2[k] = __float2bfloat16_rn(tot[k] * inv);
    }
    return;
  }
  if (worker && row2 < p.group) {
    bf16* o2 = p.out + (size_t)e * p.out_stride + (size_t)(kvh * p.group + row2) * HD + (int)rank * slice + dl;
    const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (k < per) o2[k] = __float2bfloat16_rn(fin[k] * inv);
  }
  LL_TIMELINE_STAMP(p.status, 1, 2);
}

// One new token per entry: q row e (head h at q + e*q_stride + h*hd) attends to the cached keys of
// the request in req_slot[e] up to position ctx_len[e] (its own key is already in the cache).
// nouter clusters a (entry, kv head) (1; more only with nsplit >= 2: scratch is then float32
// [n_entries * nkv * nouter * nsplit * 8 * (hd / nsplit + 2)], counters int32 [n_entries * nkv * nsplit], zero, left zero).
// nsplit in {1, 2, 4, 8}: CTAs per (entry, kv head) and cluster, launched as one cluster; warps in {4, 8}: warps a CTA
// (they take the split's 16-key tiles in turn); depth: tiles of a warp's ring, 2..4 for 4 warps, 2 or 3 for 8
// (0: 3, but 2 for 8 warps in clusters).  Measured in a decode step at batch 8 (4 warps, 17 tiles a CTA): rings
// of 3 tiles 1.108 ms, of 2 tiles 1.125-1.157 ms, of 4 tiles (128 KB a CTA, which no longer sits beside the
// products around it while they stream their weights ahead) 1.24-1.27 ms.
extern "C" int ll_attn_decode(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int bt_stride, const int* ctx_len,
                              const int* req_slot, int n_entries, int nh, int nkv, int hd, int page_size,
                              int num_pages, int window, float scale, int nsplit, int warps, int depth, int nouter,
                              float* scratch, int* counters, int* status, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if ((hd != 64 && hd != 128) || page_size % AD_TILE != 0 || nkv <= 0 || nh % nkv != 0 || nkv > 65535)
    return (int)cudaErrorInvalidValue;
  if (nh / nkv > AD_HEADS || !(nsplit == 1 || nsplit == 2 || nsplit == 4 || nsplit == 8) || !(warps == 4 || warps == 8))
    return (int)cudaErrorInvalidValue;
  if ((q_stride % 8) != 0 || (out_stride % 2) != 0) return (int)cudaErrorInvalidValue;
  AttnDecodeParams p;
  p.q = (const bf16*)q;
  p.q_stride = q_stride;
  p.out = (bf16*)out;
  p.out_stride = out_stride;
  p.k_cache = (const bf16*)k_cache;
  p.v_cache = (const bf16*)v_cache;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.ctx_len = ctx_len;
  p.req_slot = req_slot;
  p.n_entries = n_entries;
  p.nh = nh;
  p.nkv = nkv;
  p.group = nh / nkv;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (nouter < 1 || nouter > 64 || (nouter > 1 && (nsplit < 2 || scratch == nullptr || counters == nullptr)))
    return (int)cudaErrorInvalidValue;
  p.nsplit = nsplit;
  p.nouter = nouter;
  p.scratch = scratch;
  p.counters = counters;
  p.status = status;
  dim3 grid(n_entries, nkv, nsplit * nouter);
  if (depth == 0) depth = (warps == 4 || nsplit == 1) ? 3 : 2;
  if (!((warps == 4 && depth >= 2 && depth <= 4) || (warps == 8 && (depth == 2 || depth == 3))))
    return (int)cudaErrorInvalidValue;
  const size_t ring = (size_t)warps * depth * 2 * AD_TILE * hd * 2;
#define AD_LAUNCH(HD_, NW_, DEPTH_)                                                                                  \
  do {                                                                                                               \
    cudaFuncSetAttribute(attn_decode_kernel<HD_, NW_, DEPTH_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring); \
    ll_launch_cluster(attn_decode_kernel<HD_, NW_, DEPTH_, false>, grid, dim3(NW_ * 32), ring, stream, nsplit, p);          \
  } while (0)
#define AD_PICK(HD_)                                       \
  do {                                                     \
    if (warps == 4 && depth == 2) AD_LAUNCH(HD_, 4, 2);    \
    else if (warps == 4 && depth == 3) AD_LAUNCH(HD_, 4, 3); \
    else if (warps == 4) AD_LAUNCH(HD_, 4, 4);             \
    else if (depth == 2) AD_LAUNCH(HD_, 8, 2);             \
    else AD_LAUNCH(HD_, 8, 3);                             \
  } while (0)
  if (nouter > 1) {   // (8 warps, rings of two tiles: what the plan of few requests with long contexts uses)
    if (warps != 8 || depth != 2) return (int)cudaErrorInvalidValue;
    if (hd == 64) {
      cudaFuncSetAttribute(attn_decode_kernel<64, 8, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring);
      ll_launch_cluster(attn_decode_kernel<64, 8, 2, true>, grid, dim3(256), ring, stream, nsplit, p);
    } else {
      cudaFuncSetAttribute(attn_decode_kernel<128, 8, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring);
      ll_launch_cluster(attn_decode_kernel<128, 8, 2, true>, grid, dim3(256), ring, stream, nsplit, p);
    }
    return LL_LAUNCH_RESULT();
  }
  if (hd == 64) AD_PICK(64);
  else AD_PICK(128);
#undef AD_PICK
#undef AD_LAUNCH
  return LL_LAUNCH_RESULT();
}
