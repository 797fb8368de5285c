// Paged attention on tensor cores for bfloat16: decode (split over the keys) and prompt
// portions with one kernel.
//
// Work item = (block of 16 query rows, kv head, split of the keys).  A query row is a
// (new token, query head of the kv head's group) pair of one entry of the step, rows
// ordered token-major, so the 16 rows of a block share the kv head's keys and values:
// they are read once per group, not once per query head as in the reference's decode
// kernel (litelang/kernel/develop_flash_attn/flash_decoding.py:7-114).  For a decoded
// token the block holds the group's heads (the rest of the 16 rows is padding); for a
// portion of a prompt it holds consecutive tokens' heads with a causal limit per row.
//
// The four warps of a CTA take the 16-key tiles of the work item's key range in turn.
// Each warp keeps its own running maximum, sum and accumulator (online softmax,
// float32) and the warps are merged through shared memory at the end.  With more than
// one split the CTA's result goes to scratch memory and the CTA that arrives last
// (a counter per row block and kv head) merges the splits; nothing spins.
//
// Data path: keys and values go from global memory straight into the registers that
// mma.sync.m16n8k16 wants, in 16-byte loads.  That works because a dot product does
// not care about the order of its terms: the contraction index of an MMA step is
// mapped onto head dimensions (for Q K^T) so that each thread's four B values are 8
// contiguous bytes... concretely thread (g = lane / 4, c = lane % 4) loads dims
// [32 s + 8 c, 32 s + 8 c + 8) of key g of the tile and uses them for MMA steps 2 s
// and 2 s + 1; Q is loaded with the same mapping.  For P V each thread loads, for its
// four keys (2c, 2c+1, 2c+8, 2c+9), dims [64 h + 8 g, 64 h + 8 g + 8) and pairs the
// values of two keys with a byte permute; output column n of MMA tile (h, j) is then
// head dimension 64 h + 8 n + j.
//
// Takes head sizes 64 and 128, page sizes that are multiples of 16, any group size and
// any number of heads.  Other shapes, and float32, go to the generic kernel.
#include "common.cuh"

// 4 or 8 warps a CTA (template parameter NW): 8 when the step has so few row blocks that four warps
// an SM could not hide instruction latency (a lone warp per scheduler spends about as long on the
// arithmetic of a tile as on waiting for its keys).
#define AM_ROWS 16
#define AM_TILE 16

struct AttnMmaParams {
  const bf16* q;
  long q_stride;
  bf16* out;
  long out_stride;
  const bf16* k_cache;
  const bf16* v_cache;
  const int* block_table;
  int bt_stride;
  const int* cu_q;
  const int* ctx_len;
  const int* req_slot;
  int n_entries;
  int nh, nkv, group;
  int page_size, num_pages;
  int window;
  float scale_log2;  // softmax scale times log2(e)
  int nsplit;
  int all_single;  // every entry brings one token and a group fits a row block: entry = blockIdx.x
  int cluster;     // the nsplit CTAs of a (row block, kv head) are one thread-block cluster (nsplit 2, 4, 8 or 16)
  float* scratch_o;   // [row blocks * nkv * nsplit][16][HD]
  float* scratch_ml;  // [row blocks * nkv * nsplit][16][2]
  int* counters;      // [row blocks * nkv], zero before and after every launch
  int* status;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// volatile: the loads stay where they are written, between the MMAs (also volatile), so that the
// next tile's keys really are requested before the softmax of this one
__device__ __forceinline__ uint4 ldg16(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// ---- thread-block cluster: hardware barrier and reads of another CTA's shared memory ----
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_peer(const float* local, unsigned rank) {
  unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

#define AM_BT_CACHE 256

template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32) attn_mma_kernel(const AttnMmaParams p) {
  constexpr int AM_WARPS = NW, AM_THREADS = NW * 32;
  constexpr int KS = HD / 32;  // 16-byte key loads per thread and key row
  constexpr int VS = HD / 64;  // 16-byte value loads per thread and key row
  constexpr int NT = HD / 8;   // MMA column tiles of the output
  extern __shared__ float sm_dyn[];
  float (*sm_o)[AM_ROWS][HD + 4] = reinterpret_cast<float (*)[AM_ROWS][HD + 4]>(sm_dyn);
  float (*sm_m)[AM_ROWS] = reinterpret_cast<float (*)[AM_ROWS]>(sm_dyn + AM_WARPS * AM_ROWS * (HD + 4));
  float (*sm_l)[AM_ROWS] = sm_m + AM_WARPS;
  __shared__ int sm_last;
  __shared__ int sm_bt[AM_BT_CACHE];

  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.y, split = blockIdx.z;

  // ---- which entry does this row block belong to ----
  int e = 0, base = 0, ql = 0, tok0;
  if (p.all_single) {  // decode: no search, and one memory round trip less
    e = blockIdx.x;
    base = e;
    ql = 1;
    tok0 = e;
    if (e >= p.n_entries) return;
  } else {
    for (; e < p.n_entries; ++e) {
      ql = p.cu_q[e + 1] - p.cu_q[e];
      const int nb = (ql * p.group + AM_ROWS - 1) / AM_ROWS;
      if ((int)blockIdx.x < base + nb) break;
      base += nb;
    }
    if (e >= p.n_entries) return;
    tok0 = p.cu_q[e];
  }
  const int r0 = ((int)blockIdx.x - base) * AM_ROWS;
  const int slot = p.req_slot[e];
  const int ctx = p.ctx_len[e];
  const int total_rows = ql * p.group;

  // rows of this thread: g and g + 8
  int tokr[2], headr[2];
  bool validr[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + g + 8 * i;
    validr[i] = r < total_rows;
    const int rr = validr[i] ? r : r0;
    tokr[i] = rr / p.group;
    headr[i] = kvh * p.group + (rr - tokr[i] * p.group);
  }
  // ---- Q fragments (issued before anything waits for the slot and the context length) ----
  uint4 qa[KS], qb[KS];
  {
    const bf16* qra = p.q + (size_t)(tok0 + tokr[0]) * p.q_stride + (size_t)headr[0] * HD + 8 * c;
    const bf16* qrb = p.q + (size_t)(tok0 + tokr[1]) * p.q_stride + (size_t)headr[1] * HD + 8 * c;
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      qa[s] = validr[0] ? ldg16(qra + 32 * s) : make_uint4(0, 0, 0, 0);
      qb[s] = validr[1] ? ldg16(qrb + 32 * s) : make_uint4(0, 0, 0, 0);
    }
  }

  if (slot < 0) {  // padding entry of a captured step: zeros, no reads, counters untouched
    if (split == 0 && warp == 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (validr[i]) {
          bf16* o = p.out + (size_t)(tok0 + tokr[i]) * p.out_stride + (size_t)headr[i] * HD;
          for (int d = c; d < HD; d += 4) o[d] = __float2bfloat16_rn(0.f);
        }
    }
    return;
  }
  int posr[2], lor[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    posr[i] = ctx + tokr[i];
    lor[i] = p.window > 0 ? max(0, posr[i] - p.window + 1) : 0;
  }
  // key range of the whole block: from the first row's lower limit to the last valid row's position
  const int first_tok = r0 / p.group;
  const int last_row = min(total_rows, r0 + AM_ROWS) - 1;
  const int last_tok = last_row / p.group;
  const int j_lo = p.window > 0 ? max(0, ctx + first_tok - p.window + 1) : 0;
  const int j_hi = ctx + last_tok;
  const int lo_max = p.window > 0 ? max(0, ctx + last_tok - p.window + 1) : 0;  // largest lower limit of a row
  const int p_min = ctx + first_tok;                                            // smallest position of a row
  const int t_first = j_lo / AM_TILE, t_last = j_hi / AM_TILE;
  const int ntiles = t_last - t_first + 1;
  const int tps = (ntiles + p.nsplit - 1) / p.nsplit;
  const int t_begin = t_first + split * tps;
  const int t_end = min(t_last + 1, t_begin + tps);

  float o_acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o_acc[t][0] = o_acc[t][1] = o_acc[t][2] = o_acc[t][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  uint4 kk[2][KS], vv[VS][4];

  // the block-table entries of this CTA's tiles, fetched in one go: the tile loop then depends on
  // one memory round trip per tile (the keys), not two
  const int nt_split = t_end - t_begin;
  const bool bt_cached = nt_split <= AM_BT_CACHE;
  if (bt_cached) {
    for (int i = tid; i < nt_split; i += AM_THREADS) sm_bt[i] = bt[((t_begin + i) * AM_TILE) / p.page_size];
    __syncthreads();
  }

  auto tile_base = [&](int t) -> long {  // element offset of key 0 of tile t for this kv head, or -1
    const int key0 = t * AM_TILE;
    const int page = bt_cached ? sm_bt[t - t_begin] : bt[key0 / p.page_size];
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) set_status(p.status, LL_ERR_PAGE_RANGE);
      return -1;
    }
    return (((long)page * p.nkv + kvh) * p.page_size + (key0 % p.page_size)) * HD;
  };
  auto load_k = [&](long tb) {
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int s = 0; s < KS; ++s) kk[u][s] = ldg16(p.k_cache + tb + (long)(8 * u + g) * HD + 32 * s + 8 * c);
  };
  auto load_v = [&](long tb) {
#pragma unroll
    for (int h = 0; h < VS; ++h) {
      vv[h][0] = ldg16(p.v_cache + tb + (long)(2 * c) * HD + 64 * h + 8 * g);
      vv[h][1] = ldg16(p.v_cache + tb + (long)(2 * c + 1) * HD + 64 * h + 8 * g);
      vv[h][2] = ldg16(p.v_cache + tb + (long)(2 * c + 8) * HD + 64 * h + 8 * g);
      vv[h][3] = ldg16(p.v_cache + tb + (long)(2 * c + 9) * HD + 64 * h + 8 * g);
    }
  };

  int t = t_begin + warp;
  long tb = (t < t_end) ? tile_base(t) : -1;
  if (t < t_end && tb >= 0) {
    load_k(tb);
    load_v(tb);
  }
  for (; t < t_end; t += AM_WARPS) {
    const int t_next = t + AM_WARPS;
    const long tb_next = (t_next < t_end) ? tile_base(t_next) : -1;
    if (tb < 0) {  // a page that is not there: nothing of this tile counts
      tb = tb_next;
      if (tb >= 0) {
        load_k(tb);
        load_v(tb);
      }
      continue;
    }
    // ---- S = Q K^T ----
    float s_acc[2][4], s_odd[2][4];  // two chains per column tile: an MMA waits ~30 cycles for the one before
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      s_acc[u][0] = s_acc[u][1] = s_acc[u][2] = s_acc[u][3] = 0.f;
      s_odd[u][0] = s_odd[u][1] = s_odd[u][2] = s_odd[u][3] = 0.f;
    }
#pragma unroll
    for (int s = 0; s < KS; ++s)
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        mma_bf16_16816(s_acc[u], qa[s].x, qb[s].x, qa[s].y, qb[s].y, kk[u][s].x, kk[u][s].y);
        mma_bf16_16816(s_odd[u], qa[s].z, qb[s].z, qa[s].w, qb[s].w, kk[u][s].z, kk[u][s].w);
      }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int x = 0; x < 4; ++x) s_acc[u][x] += s_odd[u][x];
    if (tb_next >= 0) load_k(tb_next);  // the key registers are free again: fetch the next tile's keys
    // ---- scale, mask, online softmax ----
    const int key0 = t * AM_TILE;
    const bool boundary = (key0 + AM_TILE - 1 > p_min) || (key0 < lo_max);
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int i = x >> 1;  // 0: row g, 1: row g + 8
        float v = s_acc[u][x] * p.scale_log2;
        if (boundary) {
          const int j = key0 + 8 * u + 2 * c + (x & 1);
          if (j > posr[i] || j < lor[i]) v = -INFINITY;  // padding rows act as copies of the first row
        }
        s_acc[u][x] = v;
        tmax[i] = fmaxf(tmax[i], v);
      }
    float alpha[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
      tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
      const float m_new = fmaxf(m_run[i], tmax[i]);
      msafe[i] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[i] = fast_exp2(m_run[i] - msafe[i]);
      m_run[i] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int i = x >> 1;
        const float pv = fast_exp2(s_acc[u][x] - msafe[i]);
        s_acc[u][x] = pv;
        psum[i] += pv;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
    const unsigned pa0 = pack_bf16(s_acc[0][0], s_acc[0][1]);
    const unsigned pa1 = pack_bf16(s_acc[0][2], s_acc[0][3]);
    const unsigned pa2 = pack_bf16(s_acc[1][0], s_acc[1][1]);
    const unsigned pa3 = pack_bf16(s_acc[1][2], s_acc[1][3]);
    // keys outside what any row of the block may see have probability 0 by selection, but what their rows of V
    // hold (left by an earlier owner of the page, possibly Inf or NaN) would still spoil the product: zeros too
    if (key0 + AM_TILE - 1 > j_hi || key0 < j_lo) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = key0 + 2 * c + (i & 1) + 8 * (i >> 1);
        if (j > j_hi || j < j_lo) {
#pragma unroll
          for (int h = 0; h < VS; ++h) vv[h][i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    // ---- O = O * alpha + P V ----
#pragma unroll
    for (int h = 0; h < VS; ++h) {
      const unsigned* w0 = reinterpret_cast<const unsigned*>(&vv[h][0]);
      const unsigned* w1 = reinterpret_cast<const unsigned*>(&vv[h][1]);
      const unsigned* w2 = reinterpret_cast<const unsigned*>(&vv[h][2]);
      const unsigned* w3 = reinterpret_cast<const unsigned*>(&vv[h][3]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int T = h * 8 + j;
        const unsigned sel = (j & 1) ? 0x7632u : 0x5410u;
        const unsigned b0 = __byte_perm(w0[j >> 1], w1[j >> 1], sel);
        const unsigned b1 = __byte_perm(w2[j >> 1], w3[j >> 1], sel);
        o_acc[T][0] *= alpha[0];
        o_acc[T][1] *= alpha[0];
        o_acc[T][2] *= alpha[1];
        o_acc[T][3] *= alpha[1];
        mma_bf16_16816(o_acc[T], pa0, pa1, pa2, pa3, b0, b1);
      }
    }
    if (tb_next >= 0) load_v(tb_next);
    tb = tb_next;
  }

  // ---- merge the four warps ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  if (c == 0) {
    sm_m[warp][g] = m_run[0];
    sm_m[warp][g + 8] = m_run[1];
    sm_l[warp][g] = l_run[0];
    sm_l[warp][g + 8] = l_run[1];
  }
#pragma unroll
  for (int T = 0; T < NT; ++T) {
    const int h = T >> 3, j = T & 7;
    const int d0 = 64 * h + 16 * c + j, d1 = d0 + 8;
    sm_o[warp][g][d0] = o_acc[T][0];
    sm_o[warp][g][d1] = o_acc[T][1];
    sm_o[warp][g + 8][d0] = o_acc[T][2];
    sm_o[warp][g + 8][d1] = o_acc[T][3];
  }
  __syncthreads();
  // thread -> (row, HD/8 contiguous dims)
  constexpr int CPR = AM_THREADS / AM_ROWS;  // threads per row: 8 or 16
  constexpr int DPT = HD / CPR;
  const int row = tid / CPR, dbase = (tid % CPR) * DPT;
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, sm_m[w][row]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f, wgt[AM_WARPS];
#pragma unroll
  for (int w = 0; w < AM_WARPS; ++w) {
    wgt[w] = fast_exp2(sm_m[w][row] - Ms);
    L += sm_l[w][row] * wgt[w];
  }
  float acc[DPT];
#pragma unroll
  for (int d = 0; d < DPT; ++d) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < AM_WARPS; ++w) a += sm_o[w][row][dbase + d] * wgt[w];
    acc[d] = a;
  }
  const int r = r0 + row;
  const bool rvalid = r < total_rows;
  const int rtok = rvalid ? r / p.group : 0;
  const int rhead = kvh * p.group + (rvalid ? r - rtok * p.group : 0);
  bf16* orow = p.out + (size_t)(tok0 + rtok) * p.out_stride + (size_t)rhead * HD + dbase;

  if (p.nsplit == 1) {
    if (rvalid) {
      const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
      for (int d = 0; d < DPT; d += 2)
        *reinterpret_cast<unsigned*>(orow + d) = pack_bf16(acc[d] * inv, acc[d + 1] * inv);
    }
    return;
  }
  if (p.cluster) {
    // ---- several splits as one cluster: every CTA parks its result in its own shared memory and
    // finishes a slice of the head dimensions of all rows from its peers' shared memory ----
    __syncthreads();  // sm_o, sm_m, sm_l have been read by everyone
#pragma unroll
    for (int d = 0; d < DPT; ++d) sm_o[0][row][dbase + d] = acc[d];
    if ((tid % CPR) == 0) {
      sm_m[0][row] = M;
      sm_l[0][row] = L;
    }
    cluster_sync_all();
    const int cs = p.nsplit;
    const unsigned rank = cluster_rank();
    const int slice = HD / cs;                      // dims this CTA finishes
    const int outputs = AM_ROWS * slice;
    const int per = max(1, outputs / AM_THREADS);   // outputs a thread: 1..8, consecutive dims of one row
    const int o0 = min(tid * per, outputs - per);   // (with more threads than outputs the last ones repeat)
    const int row2 = o0 / slice, d0 = (int)rank * slice + (o0 - row2 * slice);
    float ms[16], ls[16], Mg = -INFINITY;
#pragma unroll
    for (int sI = 0; sI < 16; ++sI) {
      if (sI < cs) {
        ms[sI] = ld_peer(&sm_m[0][row2], sI);
        ls[sI] = ld_peer(&sm_l[0][row2], sI);
        Mg = fmaxf(Mg, ms[sI]);
      }
    }
    const float Mgs = (Mg == -INFINITY) ? 0.f : Mg;
    float Lg = 0.f, fin[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) fin[k] = 0.f;
#pragma unroll
    for (int sI = 0; sI < 16; ++sI) {
      if (sI < cs) {
        const float ws = fast_exp2(ms[sI] - Mgs);
        Lg += ls[sI] * ws;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (k < per) fin[k] += ld_peer(&sm_o[0][row2][d0 + k], sI) * ws;
      }
    }
    const int r2 = r0 + row2;
    if (r2 < total_rows) {
      const int tok2 = r2 / p.group;
      const int head2 = kvh * p.group + (r2 - tok2 * p.group);
      bf16* o2 = p.out + (size_t)(tok0 + tok2) * p.out_stride + (size_t)head2 * HD + d0;
      const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < per) o2[k] = __float2bfloat16_rn(fin[k] * inv);
    }
    cluster_sync_all();  // nobody leaves while its shared memory may still be read
    return;
  }
  // ---- several splits: park the partial result, the last CTA to arrive merges ----
  const size_t item = ((size_t)blockIdx.x * p.nkv + kvh);
  float* so = p.scratch_o + ((item * p.nsplit + split) * AM_ROWS + row) * HD + dbase;
#pragma unroll
  for (int d = 0; d < DPT; ++d) so[d] = acc[d];
  if ((tid % CPR) == 0) {
    float* sml = p.scratch_ml + ((item * p.nsplit + split) * AM_ROWS + row) * 2;
    sml[0] = M;
    sml[1] = L;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int arrived = atomicAdd(p.counters + item, 1);
    sm_last = (arrived == p.nsplit - 1);
  }
  __syncthreads();
  if (!sm_last) return;
  __threadfence();
  // maxima of all splits first (independent loads), then the weighted sum
  float Mg = -INFINITY;
  {
    const float* mlbase = p.scratch_ml + (item * p.nsplit * AM_ROWS + row) * 2;
    int s = 0;
    for (; s + 4 <= p.nsplit; s += 4) {
      const float m0 = __ldcg(mlbase + (size_t)(s + 0) * AM_ROWS * 2);
      const float m1 = __ldcg(mlbase + (size_t)(s + 1) * AM_ROWS * 2);
      const float m2 = __ldcg(mlbase + (size_t)(s + 2) * AM_ROWS * 2);
      const float m3 = __ldcg(mlbase + (size_t)(s + 3) * AM_ROWS * 2);
      Mg = fmaxf(fmaxf(Mg, fmaxf(m0, m1)), fmaxf(m2, m3));
    }
    for (; s < p.nsplit; ++s) Mg = fmaxf(Mg, __ldcg(mlbase + (size_t)s * AM_ROWS * 2));
  }
  const float Mgs = (Mg == -INFINITY) ? 0.f : Mg;
  float Lg = 0.f;
#pragma unroll
  for (int d = 0; d < DPT; ++d) acc[d] = 0.f;
  for (int s0 = 0; s0 < p.nsplit; s0 += 4) {
    float v[4][DPT], ms[4], ls[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int s = min(s0 + k, p.nsplit - 1);
      const float* sml = p.scratch_ml + ((item * p.nsplit + s) * AM_ROWS + row) * 2;
      const float* po = p.scratch_o + ((item * p.nsplit + s) * AM_ROWS + row) * HD + dbase;
      const float2 mlv = __ldcg(reinterpret_cast<const float2*>(sml));
      ms[k] = mlv.x;
      ls[k] = mlv.y;
#pragma unroll
      for (int d = 0; d < DPT; d += 4) {
        const float4 x = __ldcg(reinterpret_cast<const float4*>(po + d));
        v[k][d] = x.x;
        v[k][d + 1] = x.y;
        v[k][d + 2] = x.z;
        v[k][d + 3] = x.w;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (s0 + k < p.nsplit) {
        const float ws = fast_exp2(ms[k] - Mgs);
        Lg += ls[k] * ws;
#pragma unroll
        for (int d = 0; d < DPT; ++d) acc[d] += v[k][d] * ws;
      }
    }
  }
  if (rvalid) {
    const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
    for (int d = 0; d < DPT; d += 2)
      *reinterpret_cast<unsigned*>(orow + d) = pack_bf16(acc[d] * inv, acc[d + 1] * inv);
  }
  if (tid == 0) p.counters[item] = 0;  // ready for the next launch
}

// Sizes of the scratch memory for a launch with `row_blocks` row blocks.
extern "C" long ll_attn_mma_scratch_floats(int row_blocks, int nkv, int nsplit, int hd) {
  return (long)row_blocks * nkv * nsplit * AM_ROWS * (hd + 2);
}

extern "C" int ll_attn_mma_ex(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                              const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh, int nkv,
                              int hd, int page_size, int num_pages, int window, float scale, int nsplit,
                              int all_single, int use_cluster, int warps, float* scratch, int* counters,
                              int* status, cudaStream_t stream);

// q: query rows, head h of token t at q + t*q_stride + h*hd (bfloat16); out likewise.
// cu_q / ctx_len / req_slot describe the entries; row_blocks = sum over entries of
// ceil(q_len * group / 16), counted by the caller.  scratch: float32, at least
// ll_attn_mma_scratch_floats() elements (unused when nsplit == 1); counters: int32
// [row_blocks * nkv], zero at the first launch (the kernel leaves them zero).
extern "C" int ll_attn_mma(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                           const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                           const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh, int nkv,
                           int hd, int page_size, int num_pages, int window, float scale, int nsplit, float* scratch,
                           int* counters, int* status, cudaStream_t stream) {
  return ll_attn_mma_ex(out, out_stride, q, q_stride, k_cache, v_cache, block_table, bt_stride, cu_q, ctx_len, req_slot,
                        n_entries, row_blocks, nh, nkv, hd, page_size, num_pages, window, scale, nsplit, 0, 0, 4, scratch,
                        counters, status, stream);
}

// The same with a promise and a choice.  all_single != 0 says that every entry brings exactly one
// token (a decode step), which saves the kernel the search for its entry.  use_cluster != 0 (nsplit
// 2, 4, 8 or 16) launches the splits of a row block as one thread-block cluster that merges them through
// distributed shared memory; scratch and counters are then not used.  warps: 4 or 8 warps a CTA.
extern "C" int ll_attn_mma_ex(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                              const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh, int nkv,
                              int hd, int page_size, int num_pages, int window, float scale, int nsplit,
                              int all_single, int use_cluster, int warps, float* scratch, int* counters,
                              int* status, cudaStream_t stream) {
  if (warps != 4 && warps != 8) return (int)cudaErrorInvalidValue;
  if (row_blocks <= 0 || n_entries <= 0) return 0;
  if ((hd != 64 && hd != 128) || page_size % AM_TILE != 0 || nkv <= 0 || nh % nkv != 0 || nsplit < 1 ||
      nsplit > 65535 || nkv > 65535)
    return (int)cudaErrorInvalidValue;
  if ((q_stride % 8) != 0 || (out_stride % 2) != 0) return (int)cudaErrorInvalidValue;
  AttnMmaParams p;
  p.q = (const bf16*)q;
  p.q_stride = q_stride;
  p.out = (bf16*)out;
  p.out_stride = out_stride;
  p.k_cache = (const bf16*)k_cache;
  p.v_cache = (const bf16*)v_cache;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.cu_q = cu_q;
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
  p.nsplit = nsplit;
  p.all_single = (row_blocks == n_entries && p.group <= AM_ROWS && all_single) ? 1 : 0;
  if (use_cluster && !(nsplit == 2 || nsplit == 4 || nsplit == 8 || nsplit == 16)) return (int)cudaErrorInvalidValue;
  p.cluster = use_cluster ? 1 : 0;
  p.scratch_o = scratch;
  p.scratch_ml = scratch ? scratch + (long)row_blocks * nkv * nsplit * AM_ROWS * hd : nullptr;
  p.counters = counters;
  p.status = status;
  if (nsplit > 1 && !use_cluster && (scratch == nullptr || counters == nullptr)) return (int)cudaErrorInvalidValue;
  dim3 grid(row_blocks, nkv, nsplit);
  const int cz = use_cluster ? nsplit : 1;
  const size_t smem = sizeof(float) * ((size_t)warps * AM_ROWS * (hd + 4) + 2 * warps * AM_ROWS);
  if (cz > 8) {  // clusters of 16 are beyond the portable size: allowed per kernel
    if (hd == 64 && warps == 4) cudaFuncSetAttribute(attn_mma_kernel<64, 4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (hd == 64 && warps == 8) cudaFuncSetAttribute(attn_mma_kernel<64, 8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (hd == 128 && warps == 4) cudaFuncSetAttribute(attn_mma_kernel<128, 4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (hd == 128 && warps == 8) cudaFuncSetAttribute(attn_mma_kernel<128, 8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  }
  if (hd == 64 && warps == 4) {
    ll_launch_cluster(attn_mma_kernel<64, 4>, grid, dim3(128), smem, stream, cz, p);
  } else if (hd == 64) {
    ll_launch_cluster(attn_mma_kernel<64, 8>, grid, dim3(256), smem, stream, cz, p);
  } else if (warps == 4) {
    ll_launch_cluster(attn_mma_kernel<128, 4>, grid, dim3(128), smem, stream, cz, p);
  } else {
    cudaFuncSetAttribute(attn_mma_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch_cluster(attn_mma_kernel<128, 8>, grid, dim3(256), smem, stream, cz, p);
  }
  return LL_LAUNCH_RESULT();
}
