// Paged attention with shaped scores on tensor cores (bfloat16): prompt portions and single tokens.
//
// The mechanisms of attention_modulated.cu (a number a head on the scores, the heads' scores mixed by a
// matrix, a window or chunks, a sink, a sigmoid gate a head) on the layout of attention_prefill.cu: a CTA of
// 8 warps works on 128 consecutive rows (a row = a (token, query head of the kv head's group) pair,
// token-major), every warp on 16 of them; the CTA walks the keys in stages of 64 that all threads copy from
// the pages into shared memory with cp.async (double buffered), and the warps take their MMA operands from
// there.  Entries of one token (decode) have few rows and would leave one CTA to walk all their keys: their
// launch splits the keys instead, `span` stages a CTA (blockIdx.z), counted from the first stage that the
// token's mask leaves visible, so that which keys meet in which partial sum depends on the position only.
// The partial results (unnormalised sums, maximum and sum of a row, float32) meet in a second small kernel,
// which also adds the sink and applies the gate.
//
// Mixed heads.  s'_h[j] = sum_a M[h, a] (q_a . k_kv(a)[j]) is one dot product of a longer query with the
// keys of ALL kv heads side by side: with Q'_h = [ sum_{a in group c} M[h, a] q_a  for c = 0 .. nkv-1 ]
// (made in float32 by the kernel that normalises and rotates q, rounded once) and K_cat[j] = [k_0[j] ..
// k_(nkv-1)[j]], s'_h[j] = Q'_h . K_cat[j].  So with a mix the contraction runs over nkv * HD channels, the
// stage holds all kv heads' keys, and the values stay those of the row's own kv head.  Q' fragments are read
// from global memory (L1) where they are used: nkv * HD / 8 registers a thread would not fit.
//
// Scores, masks and the softmax are float32 in the exp2 domain; the sink is a key of score 0: the running
// maximum starts at 0 and the sum at 1.  The softmax weights enter the second product as two bfloat16
// terms (P = hi + lo, sixteen bits of mantissa) accumulated in float32, so that they are not rounded to
// eight bits where the design wants them in 32-bit.
// Head sizes 64 and 128 (keys and values separately), page sizes that are multiples of 16.
//
// Further shapes of the scores, as in attention_modulated.cu: a factor on the query that grows with its position
// (1 + coef ln(floor((p + 1) / every) + 1)); a cap, s <- cap tanh(s / cap); a bias by distance from a table
// [distances, heads], added after the cap; with a window, the request's first `keep` positions stay visible (the
// stages that hold them are walked before the window's: by part 0 where the keys are split); a sink of a learned
// score a head in the place of 0; a sigmoid gate a channel in the place of one a head; a constant on the output.
#include "common.cuh"

#define AS_WARPS 8
#define AS_THREADS (AS_WARPS * 32)
#define AS_ROWS (16 * AS_WARPS)
#define AS_TK 64

struct AttnShapedParams {
  const bf16* q;        // no mix: [tokens] rows of q_stride, head h at h * HD; mix: Q' [tokens, nh, nkv * HD]
  long q_stride;
  const bf16* gate;     // optional: token t, head h at gate[t * gate_stride + h]
  long gate_stride;
  const float* temp;    // optional [nh]
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
  int mask, mask_size, sink;
  float scale_log2;
  int* status;
  int nsplit, span;     // nsplit > 1: every entry brings one token; CTA z takes stages [first + z span, + span)
  float* part;          // [tokens, nh, nsplit, VD + 2]: sums, then the maximum (log2 domain) and the sum
  const float* sink_val;  // optional [nh]: the sink's score (natural units) in the place of 0
  const float* rel;       // optional [nd, nh]: bias of a key min(n, nd - 1) positions back (natural units)
  int nd;
  int keep;               // with mask 1: positions below it stay visible
  float cap_log2, inv_cap_log2;   // cap > 0: scores through cap tanh(s / cap); here cap log2(e) and its inverse
  float qt_coef;
  int qt_every;           // > 0: the query's factor by position
  int gate_channels;      // the gate is a number a channel: token t, head h, channel d at gate[t * gate_stride + h * VD + d]
  float out_scale;
};
#define AS_LOG2E 1.4426950408889634f
// tanh from exp2 and a division: absolute error of a few 1e-7
__device__ __forceinline__ float as_tanh(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.885390081777927f));
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}

__device__ __forceinline__ void as_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float as_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned as_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ uint4 as_lds16(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void as_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void as_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void as_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ int as_first_visible(int mask, int size, int pos) {
  if (mask == 1) return max(0, pos - size + 1);
  if (mask == 2) return (pos / size) * size;
  return 0;
}

template <int HD, int VD, bool MIX>
__global__ void __launch_bounds__(AS_THREADS) attn_shaped_kernel(const AttnShapedParams p) {
  constexpr int KS = HD / 32, VS = VD / 64, NT = VD / 8;
  constexpr int KCPR = HD / 8, VCPR = VD / 8;   // 16-byte chunks in a key row of one kv head, in a value row
  constexpr int KROW = HD * 2, VROW = VD * 2;
  constexpr int VT_BYTES = AS_TK * VROW;
  extern __shared__ __align__(16) unsigned char smem[];  // K[2] | V[2]
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int nkb = MIX ? p.nkv : 1;      // kv heads whose keys a stage holds
  const int kpitch = nkb * KROW;        // bytes from one key to the next in a stage
  const int kt_bytes = AS_TK * kpitch;
  const unsigned k_base = (unsigned)__cvta_generic_to_shared(smem);
  const unsigned v_base = k_base + 2 * kt_bytes;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int kvh = blockIdx.y;
  const int z = blockIdx.z;

  // ---- which entry: blocks are handed out from the end, so the ones with the most keys start first ----
  const int rb = (int)gridDim.x - 1 - (int)blockIdx.x;
  int e = 0, base = 0, ql = 0;
  for (; e < p.n_entries; ++e) {
    ql = p.cu_q[e + 1] - p.cu_q[e];
    const int nb = (ql * p.group + AS_ROWS - 1) / AS_ROWS;
    if (rb < base + nb) break;
    base += nb;
  }
  if (e >= p.n_entries) return;
  const int tok0 = p.cu_q[e];
  const int slot = p.req_slot[e];
  const int ctx = p.ctx_len[e];
  const int total_rows = ql * p.group;
  const int r0 = (rb - base) * AS_ROWS;   // first row of the CTA
  const int rw0 = r0 + 16 * warp;          // first row of the warp
  const bool split = p.nsplit > 1;

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
  if (slot < 0) {  // padding entry: zeros, nothing read (with splits the second kernel writes them)
    if (!split) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (validr[i]) {
          bf16* o = p.out + (size_t)(tok0 + tokr[i]) * p.out_stride + (size_t)headr[i] * VD;
          for (int d = c; d < VD; d += 4) o[d] = __float2bfloat16_rn(0.f);
        }
    }
    return;
  }
  // ---- Q: fragments in registers, or (mixed heads) pointers to the rows of Q' ----
  const size_t qhead = MIX ? (size_t)p.nkv * HD : (size_t)HD;
  const bf16* qra = p.q + (size_t)(tok0 + tokr[0]) * p.q_stride + (size_t)headr[0] * qhead + 8 * c;
  const bf16* qrb = p.q + (size_t)(tok0 + tokr[1]) * p.q_stride + (size_t)headr[1] * qhead + 8 * c;
  uint4 qa[KS], qb[KS];
  if constexpr (!MIX) {
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      qa[s] = *reinterpret_cast<const uint4*>(qra + 32 * s);
      qb[s] = *reinterpret_cast<const uint4*>(qrb + 32 * s);
    }
  }
  int posr[2], lor[2];
  float sc[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    posr[i] = ctx + tokr[i];
    lor[i] = as_first_visible(p.mask, p.mask_size, posr[i]);
    sc[i] = p.scale_log2 * ((!MIX && p.temp) ? p.temp[headr[i]] : 1.0f);
    if (p.qt_every > 0) sc[i] *= 1.0f + p.qt_coef * logf((float)((posr[i] + 1) / p.qt_every) + 1.0f);
  }
  const int keep = p.mask == 1 ? p.keep : 0;
  // key ranges: of the CTA (what is loaded) and of the warp (what it computes on); the first visible key
  // never decreases with the position, so the first row has the smallest and the last row the largest one
  const int cta_last_row = min(total_rows, r0 + AS_ROWS) - 1;
  const int cta_lo = as_first_visible(p.mask, p.mask_size, ctx + r0 / p.group);
  const int cta_hi = ctx + cta_last_row / p.group;
  const bool warp_active = rw0 < total_rows;
  const int w_last_row = min(total_rows, rw0 + 16) - 1;
  const int w_first_tok = min(rw0, total_rows - 1) / p.group, w_last_tok = max(w_last_row, 0) / p.group;
  const int w_lo = as_first_visible(p.mask, p.mask_size, ctx + w_first_tok);
  const int w_lo_max = as_first_visible(p.mask, p.mask_size, ctx + w_last_tok);
  const int w_pmin = ctx + w_first_tok, w_hi = ctx + w_last_tok;

  const int* bt = p.block_table + (size_t)slot * p.bt_stride;
  int T_first = cta_lo / AS_TK, T_last = cta_hi / AS_TK;
  // the stages that hold kept first positions and lie before the window's first stage are walked first
  int nkeep = keep > 0 ? min((keep - 1) / AS_TK + 1, T_first) : 0;
  if (split && z != 0) nkeep = 0;
  if (split) {
    T_first += z * p.span;
    if (T_first > T_last) return;      // the second kernel counts the parts of a row from its position
    if (z < p.nsplit - 1) T_last = min(T_last, T_first + p.span - 1);   // (the last part takes what is left)
  }

  // copy stage T (keys [64 T, 64 T + 64)) into buffer buf
  auto load_stage = [&](int buf, int T) {
    const int kchunks = AS_TK * nkb * KCPR;   // key chunks of a stage: key-major, then kv head, then chunk
    for (int idx = tid; idx < kchunks; idx += AS_THREADS) {
      const int key = idx / (nkb * KCPR);
      const int rem = idx - key * (nkb * KCPR);
      const int kl = rem / KCPR, chunk = rem - kl * KCPR;
      const int pos = T * AS_TK + key;
      const bf16* ksrc = p.k_cache;
      int bytes = 0;
      if (pos <= cta_hi && (pos >= cta_lo || pos < keep)) {
        const int page = bt[pos / p.page_size];
        if (page >= 0 && page < p.num_pages) {
          ksrc += (((size_t)page * p.nkv + (MIX ? kl : kvh)) * p.page_size + (pos % p.page_size)) * HD + 8 * chunk;
          bytes = 16;
        } else {
          set_status(p.status, LL_ERR_PAGE_RANGE);
        }
      }
      as_cp_async16(k_base + buf * kt_bytes + key * kpitch + kl * KROW + ((chunk ^ ((key & 1) << 2)) << 4), ksrc, bytes);
    }
    constexpr int V_PER_THREAD = AS_TK * VCPR / AS_THREADS;
#pragma unroll
    for (int i = 0; i < V_PER_THREAD; ++i) {
      const int idx = tid + AS_THREADS * i;
      const int key = idx / VCPR, chunk = idx - key * VCPR;
      const int pos = T * AS_TK + key;
      const bf16* vsrc = p.v_cache;
      int bytes = 0;
      if (pos <= cta_hi && (pos >= cta_lo || pos < keep)) {
        const int page = bt[pos / p.page_size];
        if (page >= 0 && page < p.num_pages) {
          vsrc += (((size_t)page * p.nkv + kvh) * p.page_size + (pos % p.page_size)) * VD + 8 * chunk;
          bytes = 16;
        }
      }
      as_cp_async16(v_base + buf * VT_BYTES + key * VROW + ((chunk ^ (key & 6)) << 4), vsrc, bytes);
    }
  };

  float o_acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t) o_acc[t][0] = o_acc[t][1] = o_acc[t][2] = o_acc[t][3] = 0.f;
  // the sink is a key of score 0 that every row sees (with splits the second kernel adds it)
  const bool sink_here = p.sink && !split;
  float m_run[2], l_run[2], sink_log2[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    sink_log2[i] = p.sink_val ? p.sink_val[headr[i]] * AS_LOG2E : 0.f;
    m_run[i] = sink_here ? sink_log2[i] : -INFINITY;
    l_run[i] = 0.f;   // (a thread holds a quarter of a row's sum: the sink's term is added after the reduction)
  }
  const int n_stages = nkeep + (T_last - T_first + 1);
  auto stage_T = [&](int n) { return n < nkeep ? n : T_first + (n - nkeep); };

  load_stage(0, stage_T(0));
  as_commit();
  for (int n = 0; n < n_stages; ++n) {
    const int T = stage_T(n);
    const int buf = n & 1;
    if (n + 1 < n_stages) load_stage(buf ^ 1, stage_T(n + 1));
    as_commit();
    as_wait<1>();      // everything but the newest group has landed: stage T is complete
    __syncthreads();
    if (warp_active) {
#pragma unroll 1
      for (int sub = 0; sub < AS_TK / 32; ++sub) {
        const int key0 = T * AS_TK + 32 * sub;
        if (key0 > w_hi || (key0 + 31 < w_lo && key0 >= keep)) continue;  // nothing of this piece is visible to the warp's rows
        const unsigned kt = k_base + buf * kt_bytes + (32 * sub) * kpitch;
        const unsigned vt = v_base + buf * VT_BYTES + (32 * sub) * VROW;
        // the biases of this piece's scores are asked for before the products, whose time covers the table's latency
        float bias_v[4][4];
        if (p.rel) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const int i = x >> 1;
              const int j = key0 + 8 * u + 2 * c + (x & 1);
              bias_v[u][x] = __ldg(p.rel + (size_t)min(max(posr[i] - j, 0), p.nd - 1) * p.nh + headr[i]);
            }
        }
        // ---- S = Q K^T for 32 keys: four column tiles, two accumulation chains each ----
        float s_acc[4][4], s_odd[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s_acc[u][0] = s_acc[u][1] = s_acc[u][2] = s_acc[u][3] = 0.f;
          s_odd[u][0] = s_odd[u][1] = s_odd[u][2] = s_odd[u][3] = 0.f;
        }
        if constexpr (!MIX) {
#pragma unroll
          for (int s = 0; s < KS; ++s)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int key = 8 * u + g;   // row inside the piece; 32 * sub and 8 u are even, so key & 1 == g & 1
              const uint4 kk = as_lds16(kt + key * kpitch + (((4 * s + c) ^ ((g & 1) << 2)) << 4));
              as_mma(s_acc[u], qa[s].x, qb[s].x, qa[s].y, qb[s].y, kk.x, kk.y);
              as_mma(s_odd[u], qa[s].z, qb[s].z, qa[s].w, qb[s].w, kk.z, kk.w);
            }
        } else {
#pragma unroll 1
          for (int kl = 0; kl < p.nkv; ++kl) {
#pragma unroll
            for (int s = 0; s < KS; ++s) {
              qa[s] = __ldg(reinterpret_cast<const uint4*>(qra + kl * HD + 32 * s));
              qb[s] = __ldg(reinterpret_cast<const uint4*>(qrb + kl * HD + 32 * s));
            }
#pragma unroll
            for (int s = 0; s < KS; ++s)
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int key = 8 * u + g;
                const uint4 kk = as_lds16(kt + key * kpitch + kl * KROW + (((4 * s + c) ^ ((g & 1) << 2)) << 4));
                as_mma(s_acc[u], qa[s].x, qb[s].x, qa[s].y, qb[s].y, kk.x, kk.y);
                as_mma(s_odd[u], qa[s].z, qb[s].z, qa[s].w, qb[s].w, kk.z, kk.w);
              }
          }
        }
        // ---- scale, mask, online softmax ----
        const bool boundary = (key0 + 31 > w_pmin) || (key0 < w_lo_max);
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = x >> 1;
            float v = (s_acc[u][x] + s_odd[u][x]) * sc[i];
            if (p.cap_log2 > 0.f) v = p.cap_log2 * as_tanh(v * p.inv_cap_log2);
            if (p.rel) v = fmaf(bias_v[u][x], AS_LOG2E, v);
            if (boundary) {
              const int j = key0 + 8 * u + 2 * c + (x & 1);
              if (j > posr[i] || (j < lor[i] && j >= keep)) v = -INFINITY;
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
          alpha[i] = as_exp2(m_run[i] - msafe[i]);
          m_run[i] = m_new;
        }
        float psum[2] = {0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int i = x >> 1;
            const float pv = as_exp2(s_acc[u][x] - msafe[i]);
            s_acc[u][x] = pv;
            psum[i] += pv;
          }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
        // P as the A operand of the two 16-key steps, in two bfloat16 terms: hi, and what hi lost
        unsigned pa[2][4], pl[2][4];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float a = s_acc[2 * ks + (w >> 1)][2 * (w & 1)], b = s_acc[2 * ks + (w >> 1)][2 * (w & 1) + 1];
            const __nv_bfloat162 hi = __floats2bfloat162_rn(a, b);
            pa[ks][w] = *reinterpret_cast<const unsigned*>(&hi);
            pl[ks][w] = as_pack(a - __low2float(hi), b - __high2float(hi));
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
            const unsigned vk = vt + (16 * ks) * VROW + chunk;
            vv[ks][0] = as_lds16(vk + (2 * c) * VROW);
            vv[ks][1] = as_lds16(vk + (2 * c + 1) * VROW);
            vv[ks][2] = as_lds16(vk + (2 * c + 8) * VROW);
            vv[ks][3] = as_lds16(vk + (2 * c + 9) * VROW);
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
              as_mma(o_acc[Tn], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b0, b1);
              as_mma(o_acc[Tn], pl[ks][0], pl[ks][1], pl[ks][2], pl[ks][3], b0, b1);
            }
          }
        }
      }
    }
    __syncthreads();  // the buffer may be overwritten by the copy of stage T + 2
  }
  as_wait<0>();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  if (split) {
    // ---- this CTA's part of every row: sums as they are, the maximum and the sum of the weights ----
    if (warp_active) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (validr[i]) {
          float* dst = p.part + (((size_t)(tok0 + tokr[i]) * p.nh + headr[i]) * p.nsplit + z) * (VD + 2);
#pragma unroll
          for (int Tn = 0; Tn < NT; ++Tn) {
            const int d0 = 64 * (Tn >> 3) + 16 * c + (Tn & 7);
            dst[d0] = o_acc[Tn][2 * i];
            dst[d0 + 8] = o_acc[Tn][2 * i + 1];
          }
          if (c == 0) {
            dst[VD] = m_run[i];
            dst[VD + 1] = l_run[i];
          }
        }
    }
    return;
  }
  // ---- normalise, gate and write: through shared memory, so that rows go out in 16-byte pieces ----
  float inv[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float l = l_run[i] + (sink_here ? as_exp2(sink_log2[i] - m_run[i]) : 0.f);
    inv[i] = (l > 0.f ? 1.0f / l : 0.f) * p.out_scale;
    if (p.gate && !p.gate_channels) {
      const float gv = __bfloat162float(p.gate[(size_t)(tok0 + tokr[i]) * p.gate_stride + headr[i]]);
      inv[i] *= 1.0f / (1.0f + expf(-gv));
    }
  }
  // each warp has 16 rows x VD bfloat16 of staging space (the buffers are free now: all warps passed the last
  // barrier of the loop)
  bf16* stage = reinterpret_cast<bf16*>(smem) + (size_t)warp * 16 * (VD + 8);
#pragma unroll
  for (int Tn = 0; Tn < NT; ++Tn) {
    const int h = Tn >> 3, j = Tn & 7;
    const int d0 = 64 * h + 16 * c + j, d1 = d0 + 8;
    float ga[2] = {1.f, 1.f}, gb[2] = {1.f, 1.f};      // a gate a channel: before the value's one rounding
    if (p.gate && p.gate_channels) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bf16* gr = p.gate + (size_t)(tok0 + tokr[i]) * p.gate_stride + (size_t)headr[i] * VD;
        ga[i] = 1.0f / (1.0f + expf(-__bfloat162float(gr[d0])));
        gb[i] = 1.0f / (1.0f + expf(-__bfloat162float(gr[d1])));
      }
    }
    stage[g * (VD + 8) + d0] = __float2bfloat16_rn(o_acc[Tn][0] * inv[0] * ga[0]);
    stage[g * (VD + 8) + d1] = __float2bfloat16_rn(o_acc[Tn][1] * inv[0] * gb[0]);
    stage[(g + 8) * (VD + 8) + d0] = __float2bfloat16_rn(o_acc[Tn][2] * inv[1] * ga[1]);
    stage[(g + 8) * (VD + 8) + d1] = __float2bfloat16_rn(o_acc[Tn][3] * inv[1] * gb[1]);
  }
  __syncwarp();
  for (int idx = lane; idx < 16 * VCPR; idx += 32) {
    const int row = idx / VCPR, chunk = idx - row * VCPR;
    const int r = rw0 + row;
    if (r < total_rows) {
      const int tok = r / p.group;
      const int head = kvh * p.group + (r - tok * p.group);
      const uint4 v = *reinterpret_cast<const uint4*>(stage + row * (VD + 8) + 8 * chunk);
      *reinterpret_cast<uint4*>(p.out + (size_t)(tok0 + tok) * p.out_stride + (size_t)head * VD + 8 * chunk) = v;
    }
  }
}

// The parts of a single token's rows meet: out[h] = sum_z O_z 2^(m_z - M) / (sum_z l_z 2^(m_z - M) + sink 2^-M),
// M the largest maximum (0 at least with a sink), times the head's gate.  How many parts a row has follows
// from its position as in the first kernel.  One block a (entry, head), a thread a value channel.
template <int VD>
__global__ void __launch_bounds__(VD) attn_shaped_join_kernel(const AttnShapedParams p) {
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int e = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int tok = p.cu_q[e];
  bf16* o = p.out + (size_t)tok * p.out_stride + (size_t)head * VD;
  if (p.req_slot[e] < 0) {
    o[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const int pos = p.ctx_len[e];
  const int stages = pos / AS_TK - as_first_visible(p.mask, p.mask_size, pos) / AS_TK + 1;
  const int parts = min(p.nsplit, (stages + p.span - 1) / p.span);
  const float* src = p.part + ((size_t)tok * p.nh + head) * p.nsplit * (VD + 2);
  const float sink_log2 = p.sink_val ? p.sink_val[head] * AS_LOG2E : 0.f;
  float M = p.sink ? sink_log2 : -INFINITY;
  for (int zz = 0; zz < parts; ++zz) M = fmaxf(M, src[(size_t)zz * (VD + 2) + VD]);
  float L = (p.sink && M > -INFINITY) ? as_exp2(sink_log2 - M) : 0.f, acc = 0.f;
  for (int zz = 0; zz < parts; ++zz) {
    const float* s = src + (size_t)zz * (VD + 2);
    const float m = s[VD];
    const float w = m > -INFINITY ? as_exp2(m - M) : 0.f;
    L = fmaf(s[VD + 1], w, L);
    acc = fmaf(s[d], w, acc);
  }
  float r = (L > 0.f ? acc / L : 0.f) * p.out_scale;
  if (p.gate)
    r *= 1.0f / (1.0f + expf(-__bfloat162float(p.gate[(size_t)tok * p.gate_stride +
                                                       (p.gate_channels ? (size_t)head * VD + d : (size_t)head)])));
  o[d] = __float2bfloat16_rn(r);
}

// Shared memory of a CTA for these sizes (0: the shape is not taken).
extern "C" long ll_attn_shaped_smem(int nkv, int hd, int vd, int mixed) {
  if ((hd != 64 && hd != 128) || (vd != 64 && vd != 128) || nkv <= 0) return 0;
  const long bytes = 2L * AS_TK * (mixed ? nkv : 1) * hd * 2 + 2L * AS_TK * vd * 2;
  return bytes <= 200 * 1024 ? bytes : 0;
}

// q: without `mixed`, rows of q_stride elements with head h at h * hd; with it, Q' rows of q_stride elements with
// head h at h * nkv * hd (the kv heads' parts side by side).  gate (optional): token t, head h at
// gate[t * gate_stride + h]; temp (optional, ignored with `mixed`: it is inside Q'): float32 [nh].
// out [tokens, nh * vd].  k_cache [pages, nkv, page_size, hd], v_cache [pages, nkv, page_size, vd].
// cu_q, ctx_len, req_slot: the entries; row_blocks = sum over them of ceil(q_len * group / 128).
// sink_val (optional float32 [nh]), rel (optional float32 [nd, nh]), keep, cap (0: none), qt_coef / qt_every
// (0: none), gate_channels, out_scale: see the head of this file.
// mask 0 causal, 1 window, 2 chunks of mask_size.  nsplit > 1 (every entry brings one token): the keys of a
// row are cut into parts of `span` stages of 64 keys; part float32 [tokens, nh, nsplit, vd + 2].
extern "C" int ll_attn_shaped(void* out, long out_stride, const void* q, long q_stride, int mixed, const void* gate,
                              long gate_stride, const float* temp, const void* k_cache, const void* v_cache,
                              const int* block_table, int bt_stride, const int* cu_q, const int* ctx_len,
                              const int* req_slot, int n_entries, int row_blocks, int nh, int nkv, int hd, int vd,
                              int page_size, int num_pages, int mask, int mask_size, int sink, float scale, int nsplit,
                              int span, float* part, int* status, const float* sink_val, const float* rel, int nd,
                              int keep, float cap, float qt_coef, int qt_every, int gate_channels, float out_scale,
                              cudaStream_t stream) {
  if (row_blocks <= 0 || n_entries <= 0) return 0;
  const long smem = ll_attn_shaped_smem(nkv, hd, vd, mixed);
  if (smem == 0 || page_size % 16 != 0 || nh % nkv != 0 || nkv > 65535 || mask < 0 || mask > 2 ||
      (mask != 0 && mask_size <= 0) || nsplit < 1 || nsplit > 65535 || (nsplit > 1 && (part == nullptr || span < 1)))
    return (int)cudaErrorInvalidValue;
  if ((q_stride % 8) != 0 || (out_stride % 8) != 0 || (rel != nullptr && nd <= 0) || keep < 0 ||
      (mixed && (rel != nullptr || cap > 0.f || sink_val != nullptr)))
    return (int)cudaErrorInvalidValue;
  AttnShapedParams p;
  p.q = (const bf16*)q;
  p.q_stride = q_stride;
  p.gate = (const bf16*)gate;
  p.gate_stride = gate_stride;
  p.temp = temp;
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
  p.mask = mask;
  p.mask_size = mask_size;
  p.sink = sink;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.nsplit = nsplit;
  p.span = span;
  p.part = part;
  p.sink_val = sink ? sink_val : nullptr;
  p.rel = rel;
  p.nd = nd;
  p.keep = keep;
  p.cap_log2 = cap > 0.f ? cap * AS_LOG2E : 0.f;
  p.inv_cap_log2 = cap > 0.f ? 1.0f / (cap * AS_LOG2E) : 0.f;
  p.qt_coef = qt_coef;
  p.qt_every = qt_every;
  p.gate_channels = gate_channels;
  p.out_scale = out_scale;
  dim3 grid(row_blocks, nkv, nsplit);
#define AS_LAUNCH(HD_, VD_, MIX_)                                                                                  \
  do {                                                                                                             \
    cudaFuncSetAttribute(attn_shaped_kernel<HD_, VD_, MIX_>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                         (int)smem);                                                                               \
    ll_launch(attn_shaped_kernel<HD_, VD_, MIX_>, grid, dim3(AS_THREADS), (size_t)smem, stream, p);                \
  } while (0)
#define AS_PICK(MIX_)                                                                                              \
  do {                                                                                                             \
    if (hd == 64 && vd == 64) AS_LAUNCH(64, 64, MIX_);                                                             \
    else if (hd == 64) AS_LAUNCH(64, 128, MIX_);                                                                   \
    else if (vd == 64) AS_LAUNCH(128, 64, MIX_);                                                                   \
    else AS_LAUNCH(128, 128, MIX_);                                                                                \
  } while (0)
  if (mixed) AS_PICK(true);
  else AS_PICK(false);
#undef AS_PICK
#undef AS_LAUNCH
  int rc = LL_LAUNCH_RESULT();
  if (rc != 0 || nsplit == 1) return rc;
  // the rows of the single tokens: row_blocks counts ceil(group / 128) blocks an entry here
  dim3 jgrid(n_entries, nh);
  if (vd == 64) ll_launch(attn_shaped_join_kernel<64>, jgrid, dim3(64), 0, stream, p);
  else ll_launch(attn_shaped_join_kernel<128>, jgrid, dim3(128), 0, stream, p);
  return LL_LAUNCH_RESULT();
}
