// Paged attention on tensor cores for portions of prompts (bfloat16).
//
// The decode kernel (attention_mma.cu) gives every block of 16 query rows its own CTA, which reads the
// keys and values of its range from L2 on its own: fine for one token a request, but for a prompt of
// 2,048 tokens every key is then fetched by hundreds of CTAs and L2 bandwidth becomes the limit.
// Here a CTA of 8 warps works on 128 consecutive query rows (a row = a (token, query head of the kv
// head's group) pair, token-major, as in the decode kernel); every warp owns 16 of them.  The CTA walks
// the keys in stages of 64: all threads copy the stage's keys and values from the pages into shared
// memory with cp.async (double buffered, zero-filled beyond the request's length), and each warp takes
// its MMA operands from there, so a key is fetched once per 128 rows.  A warp works on 32 keys at a time (four
// independent score tiles in flight, one softmax update per 32 keys) and skips 32-key pieces that lie
// entirely after its rows' positions (causal) or before their window.  (64-row CTAs, two an SM, were
// tried against the causal tail and were slower.)
//
// Shared-memory layout: row = key, 16-byte chunk q of a row stored at chunk q ^ (4 * (key & 1)) for
// keys and q ^ (key & 6) for values, which makes the 16-byte reads of the two fragment patterns
// (Q K^T: thread (g, c) reads key g, chunk 4 s + c; P V: key 2c(+1, +8, +9), chunk 8 h + g) free of bank
// conflicts.  The contraction-index trick of the decode kernel carries over unchanged.
//
// Online softmax in float32 with exp2; P rounded to bfloat16 for the second product, as in the
// reference's prefill kernel (litelang/kernel/develop_flash_attn/flash_attn_v2.py:449-501).
// Head sizes 64 and 128, page sizes that are multiples of 16.
#include "common.cuh"

#define AP_WARPS 8
#define AP_THREADS (AP_WARPS * 32)
#define AP_ROWS (16 * AP_WARPS)
#define AP_TK 64

struct AttnPrefillParams {
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
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void ap_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ap_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned ap_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ uint4 ap_lds16(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// 16 bytes global -> shared, asynchronously; src_bytes = 0 writes zeros and reads nothing
__device__ __forceinline__ void ap_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ap_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ap_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int HD>
__global__ void __launch_bounds__(AP_THREADS) attn_prefill_kernel(const AttnPrefillParams p) {
  constexpr int KS = HD / 32, VS = HD / 64, NT = HD / 8;
  constexpr int CPR = HD / 8;                   // 16-byte chunks in a key row
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = AP_TK * ROW_BYTES;  // keys (or values) of one stage
  extern __shared__ __align__(16) unsigned char smem[];  // K[2] | V[2]
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const unsigned k_base = (unsigned)__cvta_generic_to_shared(smem);
  const unsigned v_base = k_base + 2 * TILE_BYTES;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.y;

  // ---- which entry: blocks are handed out from the end, so the ones with the most keys start first ----
  const int rb = (int)gridDim.x - 1 - (int)blockIdx.x;
  int e = 0, base = 0, ql = 0;
  for (; e < p.n_entries; ++e) {
    ql = p.cu_q[e + 1] - p.cu_q[e];
    const int nb = (ql * p.group + AP_ROWS - 1) / AP_ROWS;
    if (rb < base + nb) break;
    base += nb;
  }
  if (e >= p.n_entries) return;
  const int tok0 = p.cu_q[e];
  const int slot = p.req_slot[e];
  const int ctx = p.ctx_len[e];
  const int total_rows = ql * p.group;
  const int r0 = (rb - base) * AP_ROWS;   // first row of the CTA
  const int rw0 = r0 + 16 * warp;          // first row of the warp

  int tokr[2], headr[2];
  bool validr[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rw0 + g + 8 * i;
    validr[i] = r < total_rows;
    const int rr = validr[i] ? r : min(rw0, total_rows - 1);
    tokr[i] = rr / p.group;
    headr[i] = kvh * p.group + (rr - tokr[i] * p.group);
  }
  if (slot < 0) {  // padding entry: zeros, nothing read
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (validr[i]) {
        bf16* o = p.out + (size_t)(tok0 + tokr[i]) * p.out_stride + (size_t)headr[i] * HD;
        for (int d = c; d < HD; d += 4) o[d] = __float2bfloat16_rn(0.f);
      }
    return;
  }
  // ---- Q fragments ----
  uint4 qa[KS], qb[KS];
  {
    const bf16* qra = p.q + (size_t)(tok0 + tokr[0]) * p.q_stride + (size_t)headr[0] * HD + 8 * c;
    const bf16* qrb = p.q + (size_t)(tok0 + tokr[1]) * p.q_stride + (size_t)headr[1] * HD + 8 * c;
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      qa[s] = validr[0] ? *reinterpret_cast<const uint4*>(qra + 32 * s) : make_uint4(0, 0, 0, 0);
      qb[s] = validr[1] ? *reinterpret_cast<const uint4*>(qrb + 32 * s) : make_uint4(0, 0, 0, 0);
    }
  }
  int posr[2], lor[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    posr[i] = ctx + tokr[i];
    lor[i] = p.window > 0 ? max(0, posr[i] - p.window + 1) : 0;
  }
  // key ranges: of the CTA (what is loaded) and of the warp (what it computes on)
  const int cta_last_row = min(total_rows, r0 + AP_ROWS) - 1;
  const int cta_lo = p.window > 0 ? max(0, ctx + r0 / p.group - p.window + 1) : 0;
  const int cta_hi = ctx + cta_last_row / p.group;
  const bool warp_active = rw0 < total_rows;
  const int w_last_row = min(total_rows, rw0 + 16) - 1;
  const int w_first_tok = min(rw0, total_rows - 1) / p.group, w_last_tok = max(w_last_row, 0) / p.group;
  const int w_lo = p.window > 0 ? max(0, ctx + w_first_tok - p.window + 1) : 0;   // smallest lower limit
  const int w_lo_max = p.window > 0 ? max(0, ctx + w_last_tok - p.window + 1) : 0;  // largest lower limit
  const int w_pmin = ctx + w_first_tok, w_hi = ctx + w_last_tok;

  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  const int T_first = cta_lo / AP_TK, T_last = cta_hi / AP_TK;

  // copy stage T (keys [64 T, 64 T + 64)) into buffer buf
  auto load_stage = [&](int buf, int T) {
    constexpr int PER_THREAD = AP_TK * CPR / AP_THREADS;  // 16-byte chunks a thread copies, for K and for V
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
      const int idx = tid + AP_THREADS * i;
      const int key = idx / CPR, chunk = idx - key * CPR;
      const int pos = T * AP_TK + key;
      const bf16* ksrc = p.k_cache;
      const bf16* vsrc = p.v_cache;
      int bytes = 0;
      if (pos <= cta_hi && pos >= cta_lo) {
        const int page = bt[pos / p.page_size];
        if (page >= 0 && page < p.num_pages) {
          const size_t off = (((size_t)page * p.nkv + kvh) * p.page_size + (pos % p.page_size)) * HD + 8 * chunk;
          ksrc += off;
          vsrc += off;
          bytes = 16;
        } else {
          set_status(p.status, LL_ERR_PAGE_RANGE);
        }
      }
      const unsigned kd = k_base + buf * TILE_BYTES + key * ROW_BYTES + ((chunk ^ ((key & 1) << 2)) << 4);
      const unsigned vd = v_base + buf * TILE_BYTES + key * ROW_BYTES + ((chunk ^ (key & 6)) << 4);
      ap_cp_async16(kd, ksrc, bytes);
      ap_cp_async16(vd, vsrc, bytes);
    }
  };

  float o_acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o_acc[t][0] = o_acc[t][1] = o_acc[t][2] = o_acc[t][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  load_stage(0, T_first);
  ap_commit();
  for (int T = T_first; T <= T_last; ++T) {
    const int buf = (T - T_first) & 1;
    if (T < T_last) load_stage(buf ^ 1, T + 1);
    ap_commit();
    ap_wait<1>();      // everything but the newest group has landed: stage T is complete
    __syncthreads();
    if (warp_active) {
#pragma unroll 1
      for (int sub = 0; sub < AP_TK / 32; ++sub) {
        const int key0 = T * AP_TK + 32 * sub;
        if (key0 > w_hi || key0 + 31 < w_lo) continue;  // nothing of this piece is visible to the warp's rows
        const unsigned kt = k_base + buf * TILE_BYTES + (32 * sub) * ROW_BYTES;
        const unsigned vt = v_base + buf * TILE_BYTES + (32 * sub) * ROW_BYTES;
        // ---- S = Q K^T for 32 keys: four column tiles, two accumulation chains each ----
        float s_acc[4][4], s_odd[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s_acc[u][0] = s_acc[u][1] = s_acc[u][2] = s_acc[u][3] = 0.f;
          s_odd[u][0] = s_odd[u][1] = s_odd[u][2] = s_odd[u][3] = 0.f;
        }
#pragma unroll
        for (int s = 0; s < KS; ++s)
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int key = 8 * u + g;   // row inside the piece; 32 * sub and 8 u are even, so key & 1 == g & 1
            const uint4 kk = ap_lds16(kt + key * ROW_BYTES + (((4 * s + c) ^ ((g & 1) << 2)) << 4));
            ap_mma(s_acc[u], qa[s].x, qb[s].x, qa[s].y, qb[s].y, kk.x, kk.y);
            ap_mma(s_odd[u], qa[s].z, qb[s].z, qa[s].w, qb[s].w, kk.z, kk.w);
          }
        // ---- scale, mask, online softmax ----
        const bool boundary = (key0 + 31 > w_pmin) || (key0 < w_lo_max);
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = x >> 1;
            float v = (s_acc[u][x] + s_odd[u][x]) * p.scale_log2;
            if (boundary) {
              const int j = key0 + 8 * u + 2 * c + (x & 1);
              if (j > posr[i] || j < lor[i]) v = -INFINITY;
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
          alpha[i] = ap_exp2(m_run[i] - msafe[i]);
          m_run[i] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = x >> 1;
            const float pv = ap_exp2(s_acc[u][x] - msafe[i]);
            s_acc[u][x] = pv;
            psum[i] += pv;
          }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
        unsigned pa[2][4];  // P as the A operand of the two 16-key steps
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          pa[ks][0] = ap_pack(s_acc[2 * ks][0], s_acc[2 * ks][1]);
          pa[ks][1] = ap_pack(s_acc[2 * ks][2], s_acc[2 * ks][3]);
          pa[ks][2] = ap_pack(s_acc[2 * ks + 1][0], s_acc[2 * ks + 1][1]);
          pa[ks][3] = ap_pack(s_acc[2 * ks + 1][2], s_acc[2 * ks + 1][3]);
        }
        // ---- O = O * alpha + P V ----
        if ((alpha[0] != 1.f) || (alpha[1] != 1.f)) {
#pragma unroll
          for (int Tn = 0; Tn < NT; ++Tn) {
            o_acc[Tn][0] *= alpha[0];
            o_acc[Tn][1] *= alpha[0];
            o_acc[Tn][2] *= alpha[1];
            o_acc[Tn][3] *= alpha[1];
          }
        }
#pragma unroll
        for (int h = 0; h < VS; ++h) {
          // the keys of this thread in a 16-key step: 2c, 2c+1, 2c+8, 2c+9; for all of them key & 6 == (2c) & 6
          const unsigned chunk = (((unsigned)(8 * h + g)) ^ (unsigned)((2 * c) & 6)) << 4;
          uint4 vv[2][4];
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            const unsigned vk = vt + (16 * ks) * ROW_BYTES + chunk;
            vv[ks][0] = ap_lds16(vk + (2 * c) * ROW_BYTES);
            vv[ks][1] = ap_lds16(vk + (2 * c + 1) * ROW_BYTES);
            vv[ks][2] = ap_lds16(vk + (2 * c + 8) * ROW_BYTES);
            vv[ks][3] = ap_lds16(vk + (2 * c + 9) * ROW_BYTES);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int Tn = h * 8 + j;
            const unsigned sel = (j & 1) ? 0x7632u : 0x5410u;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const unsigned* w0 = reinterpret_cast<const unsigned*>(&vv[ks][0]);
              const unsigned* w1 = reinterpret_cast<const unsigned*>(&vv[ks][1]);
              const unsigned* w2 = reinterpret_cast<const unsigned*>(&vv[ks][2]);
              const unsigned* w3 = reinterpret_cast<const unsigned*>(&vv[ks][3]);
              const unsigned b0 = __byte_perm(w0[j >> 1], w1[j >> 1], sel);
              const unsigned b1 = __byte_perm(w2[j >> 1], w3[j >> 1], sel);
              ap_mma(o_acc[Tn], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b0, b1);
            }
          }
        }
      }
    }
    __syncthreads();  // the buffer may be overwritten by the copy of stage T + 2
  }
  ap_wait<0>();

  // ---- normalise and write: through shared memory, so that rows go out in 16-byte pieces ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  const float inv0 = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
  const float inv1 = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
  // each warp has 16 rows x HD bfloat16 of staging space (the K buffers are free now: all warps passed
  // the last barrier of the loop)
  bf16* stage = reinterpret_cast<bf16*>(smem) + (size_t)warp * 16 * (HD + 8);
#pragma unroll
  for (int Tn = 0; Tn < NT; ++Tn) {
    const int h = Tn >> 3, j = Tn & 7;
    const int d0 = 64 * h + 16 * c + j, d1 = d0 + 8;
    stage[g * (HD + 8) + d0] = __float2bfloat16_rn(o_acc[Tn][0] * inv0);
    stage[g * (HD + 8) + d1] = __float2bfloat16_rn(o_acc[Tn][1] * inv0);
    stage[(g + 8) * (HD + 8) + d0] = __float2bfloat16_rn(o_acc[Tn][2] * inv1);
    stage[(g + 8) * (HD + 8) + d1] = __float2bfloat16_rn(o_acc[Tn][3] * inv1);
  }
  __syncwarp();
  for (int idx = lane; idx < 16 * CPR; idx += 32) {
    const int row = idx / CPR, chunk = idx - row * CPR;
    const int r = rw0 + row;
    if (r < total_rows) {
      const int tok = r / p.group;
      const int head = kvh * p.group + (r - tok * p.group);
      const uint4 v = *reinterpret_cast<const uint4*>(stage + row * (HD + 8) + 8 * chunk);
      *reinterpret_cast<uint4*>(p.out + (size_t)(tok0 + tok) * p.out_stride + (size_t)head * HD + 8 * chunk) = v;
    }
  }
}

// Arguments as ll_attn_mma (attention_mma.cu), without splits: row_blocks = sum over entries of
// ceil(q_len * group / 128), counted by the caller.
extern "C" int ll_attn_prefill(void* out, long out_stride, const void* q, long q_stride, const void* k_cache,
                               const void* v_cache, const int* block_table, int bt_stride, const int* cu_q,
                               const int* ctx_len, const int* req_slot, int n_entries, int row_blocks, int nh, int nkv,
                               int hd, int page_size, int num_pages, int window, float scale, int* status,
                               cudaStream_t stream) {
  if (row_blocks <= 0 || n_entries <= 0) return 0;
  if ((hd != 64 && hd != 128) || page_size % 16 != 0 || nkv <= 0 || nh % nkv != 0 || nkv > 65535)
    return (int)cudaErrorInvalidValue;
  if ((q_stride % 8) != 0 || (out_stride % 8) != 0) return (int)cudaErrorInvalidValue;
  AttnPrefillParams p;
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
  p.status = status;
  const size_t smem = (size_t)4 * AP_TK * hd * 2;  // K[2] and V[2]
  dim3 grid(row_blocks, nkv);
  if (hd == 64) {
    cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(attn_prefill_kernel<64>, grid, dim3(AP_THREADS), smem, stream, p);
  } else {
    cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(attn_prefill_kernel<128>, grid, dim3(AP_THREADS), smem, stream, p);
  }
  return LL_LAUNCH_RESULT();
}
