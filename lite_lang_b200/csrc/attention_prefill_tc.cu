// Paged attention for portions of prompts on the fifth-generation tensor cores (tcgen05), bfloat16,
// head size 64 or 128, pages of 8, 16, 32 or a multiple of 64 tokens.
//
// A CTA works on up to 128 query rows of one kv head: floor(128 / group) consecutive tokens of one entry
// times the group's query heads (row = token * group + head), so the keys and values are read once for
// the whole group.  It walks the keys the rows may see in blocks of 64:
//   S  = Q K^T      tcgen05.mma 128 x 64 x head size, both operands K-major from shared memory, S in
//                   tensor memory (two buffers);
//   softmax         four warps, one row per thread: the row comes out of tensor memory with tcgen05.ld,
//                   the running maximum and sum stay in registers (float32, exp2 with the scale folded in),
//                   P goes to shared memory as bfloat16 in the 128-byte swizzled K-major form;
//   O += P V       tcgen05.mma 128 x head size x 64, V as the MN-major operand straight from the cache
//                   rows, accumulated in tensor memory over all blocks.  The probabilities are taken
//                   against a reference maximum per row that follows the true maximum only when that has
//                   grown by more than 2^8: then the row's thread scales its row of O in tensor memory
//                   (tcgen05.ld / st) and its sum.  In between, P is at most 2^8, exact enough in bfloat16
//                   as before, and nothing has to be rescaled.
// Two CTAs fit an SM (half of its shared memory and tensor memory each), so that one's softmax runs
// beside the other's MMAs.
// Roles: warp 0 loads (one thread: Q once through a 3-d tensor map [token, head, head size]; K and V
// of a block page by page through 2-d maps over the cache plane, into a ring of two stages), warp 1
// issues the MMAs (one thread; S a whole block ahead of the softmax, so that the tensor cores work
// while the softmax threads do), warps 2..5 are the softmax rows.  All hand-offs are mbarriers: TMA
// completes the "full" ones, tcgen05.commit the ones the tensor cores free, the softmax warps arrive
// on the rest.  Every wait is bounded; one that runs out records LL_ERR_WAIT_TIMEOUT, stops waiting in
// that thread and lets the kernel run to its end, where tensor memory is freed.
//
// Masked places: a key after the row's position, or before its window, gets probability 0 by selection
// (never by arithmetic on what was read).  Pages that a window has given back (table entry -1) and pages
// beyond the context are read from page 0 instead and are always masked.  What such places hold is
// whatever an earlier owner of the page left there, possibly Inf or NaN, and 0 x NaN is NaN in P V: so in
// a block with keys that none of the CTA's rows may see (the last block of the rows, the first one of a
// window), the softmax warps overwrite those keys' rows of V in shared memory with zeros before the
// product is issued.  A table entry of a key that a row does see must name a page of the pool; one that
// does not sets LL_ERR_PAGE_RANGE.
#include "tc05.cuh"

#define AT_THREADS 192
#define AT_KB 64  // keys a block
#define AT_KS 2   // stages of K and of V

struct AttnTcParams {
  bf16* out;
  long out_stride;
  const int* block_table;
  int bt_stride;
  const int* cu_q;
  const int* ctx_len;
  const int* req_slot;
  int n_entries, nkv, group, tpb;   // tpb: tokens a CTA (floor(128 / group))
  int page_size, num_pages, window;
  int box_rows;                     // keys a K/V box: min(page_size, 64)
  float scale_log2;
  // the key blocks of a row block may be split over up to nsplit CTAs (long contexts, few row blocks):
  // partial results (unnormalised O, reference maximum, sum) meet in scratch memory, the last CTA to
  // arrive (a counter per row block and kv head, left at zero again) merges them
  int nsplit, row_blocks, split_len;
  float* scratch;      // [row blocks * nkv * nsplit][HD + 2][128]
  int* counters;       // [row blocks * nkv], zero between launches
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 2)
attn_prefill_tc_kernel(const AttnTcParams p, const __grid_constant__ CUtensorMap qmap,
                       const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
  constexpr int HB = HD / 64;                  // 64-wide boxes along the head size
  constexpr int Q_BYTES = 128 * HD * 2;        // also the output rows on their way out
  constexpr int KV_BYTES = AT_KB * HD * 2;     // K (or V) of a block
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int P_BYTES = 128 * AT_KB * 2;
  constexpr int TMEM_COLS = 256;               // S: 2 x 64 columns, O: HD columns (half an SM's tensor memory)
  constexpr unsigned IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AT_KB >> 3) << 17) | ((128u >> 4) << 24);
  constexpr unsigned IDESC_PV =
      (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((128u >> 4) << 24);

  // the swizzled tiles need 1024-byte alignment in the shared window; there is no static shared memory
  // in this kernel, so the dynamic part starts aligned (checked below, refused otherwise)
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;
  unsigned char* kv_s = q_s + Q_BYTES;
  unsigned char* p_s = kv_s + AT_KS * STAGE_BYTES;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(p_s + P_BYTES);
  // barriers: q_full, k_full[KS], k_empty[KS], v_full[KS], v_empty[KS], s_full[2], s_empty[2], p_full, pv_done
  const unsigned q_full = at_smem(bars);
  const unsigned k_full0 = at_smem(bars + 1), k_empty0 = k_full0 + 8 * AT_KS;
  const unsigned v_full0 = k_full0 + 16 * AT_KS, v_empty0 = k_full0 + 24 * AT_KS;
  const unsigned s_full0 = k_full0 + 32 * AT_KS, s_empty0 = s_full0 + 16, p_full = s_full0 + 32;
  const unsigned pv_done = s_full0 + 40;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 1 + 4 * AT_KS + 6);
  unsigned* merge_flag = tmem_slot + 1;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // ---- which rows: row block rb of the step.  Order of the CTAs (the hardware starts them in the order of
  // their number, and one that has to wait holds back all after it): first split 0 of every row block, the
  // heavier, later blocks of an entry first, the kv heads side by side; then split 1 of every row block, and
  // so on.  The CTAs without work (splits that a short row block does not have) are the last of each round,
  // and nearly all of them the last of the grid. ----
  const int kvh = blockIdx.x % p.nkv;
  const int l2 = blockIdx.x / p.nkv;
  const int split = l2 / p.row_blocks;
  const int rb_step = p.row_blocks - 1 - l2 % p.row_blocks;   // row block within the step (names its scratch and counter)
  int rb = rb_step;
  int entry = -1, qlen = 0;
  for (int e = 0; e < p.n_entries; ++e) {
    const int ql = p.cu_q[e + 1] - p.cu_q[e];
    const int nb = (ql + p.tpb - 1) / p.tpb;
    if (rb < nb) {
      entry = e;
      qlen = ql;
      break;
    }
    rb -= nb;
  }
  if (entry < 0) return;
  if ((at_smem(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(p.status, LL_ERR_SMEM_ALIGN);
    return;
  }
  const int slot = p.req_slot[entry];
  if (slot < 0) return;
  const int tok0 = p.cu_q[entry] + rb * p.tpb;              // first token (row of q and out) of this CTA
  const int ntok = min(p.tpb, qlen - rb * p.tpb);
  const int pos0 = p.ctx_len[entry] + rb * p.tpb;           // its position (ctx_len: tokens cached before the step)
  const int hi = pos0 + ntok - 1;
  const int lo_min = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int nblk_all = hi / AT_KB - lo_min / AT_KB + 1;      // key blocks the rows may see
  // splits that have work: about split_len blocks each (the host chooses that length so that the step's CTAs
  // just fit the SMs at once), none empty; the same for every CTA of the row block
  int eff = min(p.nsplit, max(1, (nblk_all + p.split_len - 1) / p.split_len));
  const int per = (nblk_all + eff - 1) / eff;
  eff = (nblk_all + per - 1) / per;
  if (split >= eff) return;
  const int kb_lo = lo_min / AT_KB + split * per;             // this CTA's first block
  const int nblk = min(per, nblk_all - split * per);

  if (tid == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&qmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
  }
  if (tid == 0) {
    at_mbar_init(q_full, 1);
    for (int s = 0; s < 4 * AT_KS; ++s) at_mbar_init(k_full0 + 8 * s, 1);
    for (int b = 0; b < 2; ++b) {
      at_mbar_init(s_full0 + 8 * b, 1);
      at_mbar_init(s_empty0 + 8 * b, 4);
    }
    at_mbar_init(p_full, 4);
    at_mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(tmem_slot)),
                 "r"((unsigned)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  AT_FENCE_BEFORE();
  __syncthreads();
  AT_FENCE_AFTER();
  const unsigned tmem = *tmem_slot;
  const unsigned tmem_s = tmem, tmem_o = tmem + 2 * AT_KB;
  LL_PDL_WAIT();   // q and the new keys and values come from the kernel before
  LL_PDL_TRIGGER();
  bool dead = false;

  if (warp == 0) {
    // ------------------------------ loads ------------------------------
    // Lane b < boxes owns the b-th box (page, or part of a page) of every block: it looks its page up
    // one block ahead and issues that box's copies; lane 0 also does the waiting and the byte counts.
    if (lane == 0) {
      at_mbar_expect_tx(q_full, (unsigned)(HB * 64 * p.group * p.tpb * 2));
      for (int h = 0; h < HB; ++h)
        at_tma_3d(at_smem(q_s) + h * (Q_BYTES / HB), &qmap, h * 64, kvh * p.group, tok0, q_full);
    }
    const int* bt = p.block_table + (size_t)slot * p.bt_stride;
    const int boxes = AT_KB / p.box_rows;
    auto page_of = [&](int j) -> int {   // cache row of this lane's box of block j
      const int kp = (kb_lo + j) * AT_KB + lane * p.box_rows;
      const int lp = kp / p.page_size;
      const bool mine = lane < boxes && j < nblk;
      int page = (mine && lp < p.bt_stride) ? bt[lp] : -1;
      if (page < 0 || page >= p.num_pages) {   // given back or beyond the context: masked, and V zeroed, below
        if (mine && (page >= p.num_pages || (kp <= hi && kp + p.box_rows - 1 >= lo_min)))
          set_status(p.status, LL_ERR_PAGE_RANGE);   // a key that a row sees has no page of the pool
        page = 0;
      }
      return (page * p.nkv + kvh) * p.page_size + kp % p.page_size;
    };
    // order of the copies: K(0), K(1), then V(j) before K(j + 2), the order in which the MMAs want them
    auto load = [&](int j, int row, bool is_v) {
      const int s = j % AT_KS;
      const unsigned full = (is_v ? v_full0 : k_full0) + 8 * s;
      if (lane == 0) {
        at_mbar_wait((is_v ? v_empty0 : k_empty0) + 8 * s, (unsigned)(((j / AT_KS) & 1) ^ 1), p.status, dead);
        at_mbar_expect_tx(full, KV_BYTES);
      }
      __syncwarp();
      if (lane < boxes) {
        const unsigned dst = at_smem(kv_s) + s * STAGE_BYTES + (is_v ? KV_BYTES : 0) + lane * p.box_rows * 128;
        for (int h = 0; h < HB; ++h) at_tma_2d(dst + h * (KV_BYTES / HB), is_v ? &vmap : &kmap, h * 64, row, full);
      }
    };
    int row0 = page_of(0), row1 = page_of(1);   // cache rows of blocks j and j + 1
    load(0, row0, false);
    if (nblk > 1) load(1, row1, false);
    for (int j = 0; j < nblk; ++j) {
      const int row2 = page_of(j + 2);
      load(j, row0, true);
      if (j + 2 < nblk) load(j + 2, row2, false);
      row0 = row1;
      row1 = row2;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issue ------------------------------
    if (lane == 0) {
      auto mma_s = [&](int j) {   // S[j % 2] = Q K(j)^T
        const int s = j % AT_KS, b = j & 1;
        at_mbar_wait(k_full0 + 8 * s, (unsigned)((j / AT_KS) & 1), p.status, dead);
        at_mbar_wait(s_empty0 + 8 * b, (unsigned)(((j >> 1) & 1) ^ 1), p.status, dead);
        AT_FENCE_AFTER();
        const unsigned k_addr = at_smem(kv_s) + s * STAGE_BYTES;
#pragma unroll
        for (int k16 = 0; k16 < HD / 16; ++k16) {
          const unsigned off = (k16 / 4) * (Q_BYTES / HB) + (k16 % 4) * 32;
          const unsigned koff = (k16 / 4) * (KV_BYTES / HB) + (k16 % 4) * 32;
          at_mma(tmem_s + b * AT_KB, at_desc_k(at_smem(q_s) + off), at_desc_k(k_addr + koff), IDESC_S, k16 > 0 ? 1u : 0u);
        }
        at_commit(s_full0 + 8 * b);
        at_commit(k_empty0 + 8 * s);   // the K stage is free once these MMAs have read it
      };
      at_mbar_wait(q_full, 0, p.status, dead);
      // S runs a whole block ahead of the softmax: S(j + 2) is issued as soon as P(j) has gone into O, into
      // the buffer whose S(j) the softmax warps read long ago, so S(j + 1) is complete when they want it
      // however far apart the four warps have drifted
      mma_s(0);
      if (nblk > 1) mma_s(1);
      for (int j = 0; j < nblk; ++j) {
        const int s = j % AT_KS;
        at_mbar_wait(v_full0 + 8 * s, (unsigned)((j / AT_KS) & 1), p.status, dead);
        at_mbar_wait(p_full, (unsigned)(j & 1), p.status, dead);
        AT_FENCE_AFTER();
        const unsigned v_addr = at_smem(kv_s) + s * STAGE_BYTES + KV_BYTES;
        const unsigned p_addr = at_smem(p_s);
#pragma unroll
        for (int k16 = 0; k16 < AT_KB / 16; ++k16)   // 16 keys a step: 32 bytes along P's rows, 2048 bytes down V
          at_mma(tmem_o, at_desc_k(p_addr + k16 * 32), at_desc_mn(v_addr + k16 * 2048, KV_BYTES / HB), IDESC_PV,
                 (j > 0 || k16 > 0) ? 1u : 0u);
        at_commit(pv_done);            // P may be written again; O holds the blocks up to j
        at_commit(v_empty0 + 8 * s);
        if (j + 2 < nblk) mma_s(j + 2);
      }
    }
  } else {
    // ------------------------------ softmax rows (warps 2..5) ------------------------------
    const int ew = warp & 3;                 // tensor-memory lanes 32 ew .. 32 ew + 31
    const int r = 32 * ew + lane;            // row of the tile
    const int t = r / p.group, g = r - t * p.group;
    const bool row_ok = r < p.tpb * p.group && t < ntok;
    const int prow = row_ok ? pos0 + t : -1;                                  // position of the row's token
    const int lo_row = (p.window > 0 && prow >= 0) ? max(0, prow - p.window + 1) : 0;
    const unsigned lane_addr = (unsigned)(32 * ew) << 16;
    float m_ref = -INFINITY, l_run = 0.f;   // reference maximum (scaled, log2 units) and sum against it

    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      const int k0 = (kb_lo + j) * AT_KB;
      at_mbar_wait(s_full0 + 8 * b, (unsigned)((j >> 1) & 1), p.status, dead);
      AT_FENCE_AFTER();
      float sv[AT_KB];
      {
        unsigned ra[32], rb[32];      // both halves of the row are on their way before the one wait
        at_ld32_issue(tmem_s + lane_addr + b * AT_KB, ra);
        at_ld32_issue(tmem_s + lane_addr + b * AT_KB + 32, rb);
        at_ld_wait(ra, rb);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          sv[i] = __uint_as_float(ra[i]);
          sv[32 + i] = __uint_as_float(rb[i]);
        }
      }
      AT_FENCE_BEFORE();
      __syncwarp();
      if (lane == 0) at_mbar_arrive(s_empty0 + 8 * b);
      // mask by selection; maximum of the row's part
      if ((k0 + AT_KB - 1 > prow) || (k0 < lo_row)) {
#pragma unroll
        for (int i = 0; i < AT_KB; ++i)
          if (k0 + i > prow || k0 + i < lo_row) sv[i] = -INFINITY;
      }
      // (the softmax warps are bound by instruction issue: packed float32 pairs for the scaling and the sums,
      // three-input maxima, one MUFU instruction per exponential)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < AT_KB; i += 8) {
        mx4[0] = at_max3(mx4[0], sv[i], sv[i + 1]);
        mx4[1] = at_max3(mx4[1], sv[i + 2], sv[i + 3]);
        mx4[2] = at_max3(mx4[2], sv[i + 4], sv[i + 5]);
        mx4[3] = at_max3(mx4[3], sv[i + 6], sv[i + 7]);
      }
      const float mxs = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const bool grow = mxs > m_ref + 8.0f;          // also the first keys a row sees (m_ref = -inf)
      const float factor = grow ? at_ex2(m_ref - mxs) : 1.0f;   // m_ref = -inf: 0 (O and the sum are 0 then)
      if (grow) m_ref = mxs;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // the row of P in registers: 64 bfloat16 = 8 pieces of 16 bytes
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_use, -m_use);
      unsigned pw[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float2 a = __ffma2_rn(make_float2(sv[2 * i], sv[2 * i + 1]), sc2, nm2);
        const float2 e = make_float2(at_ex2(a.x), at_ex2(a.y));
        sum2[i & 1] = __fadd2_rn(sum2[i & 1], e);
        const __nv_bfloat162 h = __floats2bfloat162_rn(e.x, e.y);
        pw[i] = *reinterpret_cast<const unsigned*>(&h);
      }
      const float2 st = __fadd2_rn(sum2[0], sum2[1]);
      l_run = l_run * factor + (st.x + st.y);
      // the block before must be in O, and P read, before either is touched
      if (j > 0) {
        at_mbar_wait(pv_done, (unsigned)((j - 1) & 1), p.status, dead);
        AT_FENCE_AFTER();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            float v[32];
            at_ld32(tmem_o + lane_addr + c0, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= factor;
            at_st32(tmem_o + lane_addr + c0, v);
          }
        }
      }
      // keys that no row of the CTA may see: their rows of V (128 bytes for each 64 head-size elements, whole
      // rows, so the swizzle does not matter) become zeros before the product reads them
      if (k0 + AT_KB - 1 > hi || k0 < lo_min) {
        const int s = j % AT_KS;
        at_mbar_wait(v_full0 + 8 * s, (unsigned)((j / AT_KS) & 1), p.status, dead);
        unsigned char* v_s = kv_s + s * STAGE_BYTES + KV_BYTES;
        for (int idx = tid - 64; idx < AT_KB * HB * 8; idx += 128) {
          const int kk = idx / (HB * 8), rest = idx - kk * (HB * 8);
          if (k0 + kk > hi || k0 + kk < lo_min)
            *reinterpret_cast<uint4*>(v_s + (rest >> 3) * (KV_BYTES / HB) + kk * 128 + ((rest & 7) << 4)) =
                make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // piece c of the row goes to (c ^ (r & 7)) of the swizzled 128-byte row
      unsigned char* prow_s = p_s + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow_s + ((c ^ (r & 7)) << 4)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is read by the tensor cores
      AT_FENCE_BEFORE();                                             // and so is the rescaled O
      __syncwarp();
      if (lane == 0) at_mbar_arrive(p_full);
    }
    at_mbar_wait(pv_done, (unsigned)((nblk - 1) & 1), p.status, dead);
    AT_FENCE_AFTER();
    // ---- the splits of a row block meet in scratch memory; the last one to arrive goes on ----
    bool finish = true;
    float inv;
    const size_t part0 = ((size_t)rb_step * p.nkv + kvh) * p.nsplit;     // this row block's first partial
    constexpr int PSTRIDE = (HD + 2) * 128;   // floats a partial: column-major [HD + 2][128 rows] (O, maximum, sum),
                                              // so that a warp's 32 rows read and write 128 contiguous bytes
    if (eff > 1) {
      float* mine = p.scratch + (part0 + split) * PSTRIDE + r;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float v[32];
        at_ld32(tmem_o + lane_addr + c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) mine[(size_t)(c0 + i) * 128] = v[i];
      }
      mine[(size_t)HD * 128] = m_ref;
      mine[(size_t)(HD + 1) * 128] = l_run;
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (tid == 64) {
        const int old = atomicAdd(p.counters + rb_step * p.nkv + kvh, 1);
        const bool last = old == eff - 1;
        if (last) p.counters[rb_step * p.nkv + kvh] = 0;     // ready for the next launch
        *merge_flag = last ? 1u : 0u;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      finish = *merge_flag != 0u;
      if (finish) {
        // The last one to arrive adds the others' partial results to its own, which is still in tensor memory.
        // Each comes with one bulk copy into the shared memory of the K/V rings and P (free now: every MMA of
        // this CTA is done) and is added there; reading them from global memory piece by piece was a chain of
        // 4 x splits trips to L2.  Online merge: the running maximum and sum are rescaled as the partials come.
        __threadfence();
        float* part_s = reinterpret_cast<float*>(kv_s);
        static_assert(PSTRIDE * 4 <= AT_KS * STAGE_BYTES + P_BYTES, "a partial fits the freed shared memory");
        float m_cur = m_ref, l_cur = l_run;
        int round = 0;
        for (int q = 0; q < eff; ++q) {
          if (q == split) continue;
          asm volatile("bar.sync 1, 128;" ::: "memory");   // everybody is done with what the region held before
          if (tid == 64) {
            asm volatile("fence.proxy.async;" ::: "memory");
            at_mbar_expect_tx(q_full, (unsigned)(PSTRIDE * 4));
            at_bulk_load(at_smem(part_s), p.scratch + (part0 + q) * PSTRIDE, (unsigned)(PSTRIDE * 4), q_full);
          }
          at_mbar_wait(q_full, (unsigned)((round + 1) & 1), p.status, dead);   // (phase 0 was the Q tile)
          const float mq = part_s[HD * 128 + r], lq = part_s[(HD + 1) * 128 + r];
          const float m_new = fmaxf(m_cur, mq);
          const float sc_old = (m_cur == -INFINITY) ? 0.f : exp2f(m_cur - m_new);
          const float sc_q = (mq == -INFINITY) ? 0.f : exp2f(mq - m_new);
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            float v[32];
            at_ld32(tmem_o + lane_addr + c0, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = fmaf(part_s[(c0 + i) * 128 + r], sc_q, v[i] * sc_old);
            at_st32(tmem_o + lane_addr + c0, v);
          }
          l_cur = l_cur * sc_old + lq * sc_q;
          m_cur = m_new;
          ++round;
        }
        inv = l_cur > 0.f ? 1.0f / l_cur : 0.f;
      }
    } else {
      inv = l_run > 0.f ? 1.0f / l_run : 0.f;
    }
    // ---- normalise; rows leave through shared memory (the Q tile is no longer read) ----
    if (finish) {
      unsigned char* orow = q_s + r * (HD * 2);
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float v[32];
        at_ld32(tmem_o + lane_addr + c0, v);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int c = c0 / 8 + cc;
          unsigned w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * cc + 2 * i] * inv, v[8 * cc + 2 * i + 1] * inv);
            w[i] = *reinterpret_cast<const unsigned*>(&h);
          }
          *reinterpret_cast<uint4*>(orow + (((c & ~7) | ((c ^ r) & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int e = tid - 64;
    constexpr int CPR = HD / 8;   // 16-byte pieces a row
    for (int idx = e; finish && idx < 128 * CPR; idx += 128) {
      const int rr = idx / CPR, c = idx % CPR;
      const int tt = rr / p.group, gg = rr - tt * p.group;
      if (rr < p.tpb * p.group && tt < ntok) {
        const uint4 v = *reinterpret_cast<const uint4*>(q_s + rr * (HD * 2) + (((c & ~7) | ((c ^ rr) & 7)) << 4));
        *reinterpret_cast<uint4*>(p.out + (size_t)(tok0 + tt) * p.out_stride + (size_t)(kvh * p.group + gg) * HD + 8 * c) = v;
      }
    }
    (void)g;
  }
  // ---- everyone is done: free the tensor memory ----
  AT_FENCE_BEFORE();
  __syncthreads();
  if (warp == 1) {
    AT_FENCE_AFTER();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)TMEM_COLS) : "memory");
  }
}

typedef CUresult (*at_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static at_encode_fn at_encoder() {
  static at_encode_fn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (at_encode_fn)ptr;
  }
  return fn;
}

// Arguments as ll_attn_prefill (attention_prefill.cu), but the row blocks are counted differently:
// row_blocks = sum over the entries of ceil(q_len / floor(128 / group)); num_tokens is the number of rows of q.
// nsplit in 1..8: CTAs a row block's key blocks may be split over, each taking about split_len blocks of 64 keys; with nsplit > 1, scratch is float32
// [row_blocks * nkv * nsplit * (hd + 2) * 128] and counters int32 [row_blocks * nkv], zero at the first launch
// (the kernel leaves them zero).
extern "C" int ll_attn_prefill_tc(void* out, long out_stride, const void* q, long q_stride, int num_tokens,
                                  const void* k_cache, const void* v_cache, const int* block_table, int bt_stride,
                                  const int* cu_q, const int* ctx_len, const int* req_slot, int n_entries,
                                  int row_blocks, int nh, int nkv, int hd, int page_size, int num_pages, int window,
                                  float scale, int nsplit, int split_len, float* scratch, int* counters,
                                  int* status, cudaStream_t stream) {
  if (row_blocks <= 0 || n_entries <= 0) return 0;
  if ((hd != 64 && hd != 128) || nkv <= 0 || nh % nkv != 0 || nkv > 65535 || nh / nkv > 128)
    return (int)cudaErrorInvalidValue;
  if (!(page_size == 8 || page_size == 16 || page_size == 32 || (page_size > 0 && page_size % 64 == 0)))
    return (int)cudaErrorInvalidValue;
  if ((q_stride % 8) != 0 || (out_stride % 8) != 0 || ((uintptr_t)q % 16) != 0 || ((uintptr_t)out % 16) != 0)
    return (int)cudaErrorInvalidValue;
  if (nsplit < 1 || nsplit > 8 || split_len < 1 || (nsplit > 1 && (scratch == nullptr || counters == nullptr || ((uintptr_t)scratch % 16) != 0)))
    return (int)cudaErrorInvalidValue;
  at_encode_fn enc = at_encoder();
  if (enc == nullptr) return (int)cudaErrorNotSupported;
  AttnTcParams p;
  p.out = (bf16*)out;
  p.out_stride = out_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.cu_q = cu_q;
  p.ctx_len = ctx_len;
  p.req_slot = req_slot;
  p.n_entries = n_entries;
  p.nkv = nkv;
  p.group = nh / nkv;
  p.tpb = 128 / p.group;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.window = window;
  p.box_rows = page_size < 64 ? page_size : 64;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.nsplit = nsplit;
  p.scratch = scratch;
  p.counters = counters;
  p.status = status;

  CUtensorMap qmap, kmap, vmap;
  const cuuint32_t estr3[3] = {1, 1, 1};
  {
    const cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nh, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)p.group, (cuuint32_t)p.tpb};
    if (enc(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr3,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  for (int which = 0; which < 2; ++which) {
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)num_pages * nkv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)p.box_rows};
    if (enc(which ? &vmap : &kmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_cache : k_cache),
            dims, strides, box, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return (int)cudaErrorInvalidValue;
  }
  const size_t smem = (size_t)128 * hd * 2 + (size_t)AT_KS * 2 * AT_KB * hd * 2 + 128 * AT_KB * 2 + 256;
  p.row_blocks = row_blocks;
  p.split_len = split_len;
  dim3 grid(row_blocks * nsplit * nkv);
  if (hd == 64) {
    cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(attn_prefill_tc_kernel<64>, grid, dim3(AT_THREADS), smem, stream, p, qmap, kmap, vmap);
  } else {
    cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(attn_prefill_tc_kernel<128>, grid, dim3(AT_THREADS), smem, stream, p, qmap, kmap, vmap);
  }
  return LL_LAUNCH_RESULT();
}
