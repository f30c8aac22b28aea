// Latent attention of single tokens and short portions on tensor cores (bfloat16, mma.sync m16n8k16).
//
// The same work as `latent_attention_kernel` (latent_attention.cu): per (token, group of heads, part of the keys) an
// online softmax over the request's cached rows [R latent | r rotated] with the latent-space queries, returning
// sum_j p_j c_j a head (or, with parts, the unnormalised sums with the maximum and the sum for `latent_merge`).
// All heads read the same rows, so the heads are the M side of the products: a CTA takes up to 16 heads,
//   S [16 heads x 32 keys]  = Q [16 x KD] K^T     each of the 4 warps one column tile of 8 keys, KD / 16 steps
//   O [16 heads x R]       += P [16 x 32] C        each warp R / 4 columns, P from shared memory
// with KD = R + r.  The tile's rows come by cp.async (16 bytes a copy, zero-filled where a position is not visible)
// into two buffers, a tile ahead; rows are 2 KD + 16 bytes apart, which makes the 4-byte fragment reads and the
// 8 x 16-byte ldmatrix reads meet different banks whenever KD is a multiple of 16.  The rows' maxima go through
// shared memory between the warps; the softmax weights enter the second product as two bfloat16 terms (hi + lo,
// sixteen bits of mantissa), accumulated in float32.  Tiles start at multiples of 32 positions, so the order of every
// sum depends on the position only.
// Taken for: bfloat16, KD a multiple of 16, R a multiple of 32 and at most 512.
#include "common.cuh"

#define LM_TK 32
#define LM_THREADS 128
#define LM_HEADS 16
#define LM_MAX_NT 16              // column tiles of 8 a warp: R / 32
#define LM_PPITCH 80              // bytes from one head's row of P to the next (32 bfloat16 + 16 bytes)
#define LM_LOG2E 1.4426950408889634f

__device__ __forceinline__ void lm_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float lm_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned lm_lds32(unsigned addr) {
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void lm_sts32(unsigned addr, unsigned v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void lm_ldmatrix_x2_trans(unsigned& r0, unsigned& r1, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x2(unsigned& r0, unsigned& r1, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void lm_cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ unsigned lm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// q: [tokens, H, KD]; cache: one plane [pages, 1, page_size, KD]; out: [tokens, H, R].  `first`: the launch's first
// token.  gridDim = (tokens, ceil(H / 16), parts).
__global__ void __launch_bounds__(LM_THREADS)
latent_attention_mma_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ cache,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
                            const int* __restrict__ req_slot, const int* __restrict__ positions, int first, int H, int R,
                            int r, int page_size, int num_pages, int window, float scale_log2, int* status,
                            int tiles_per_split, float* __restrict__ part_acc, float* __restrict__ part_ml,
                            const float* __restrict__ sink) {
  extern __shared__ __align__(16) unsigned char lm_smem[];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = first + blockIdx.x;
  const int h0 = blockIdx.y * LM_HEADS;
  const int hc = min(LM_HEADS, H - h0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int KD = R + r;
  const int pitch = 2 * KD + 16;                    // bytes from one row to the next (queries and tile alike)
  const int ntw = R / 32;                           // column tiles a warp
  const unsigned q_base = (unsigned)__cvta_generic_to_shared(lm_smem);
  const unsigned k_base = q_base + LM_HEADS * pitch;                 // two tiles of LM_TK rows
  const unsigned ph_base = k_base + 2 * LM_TK * pitch;               // P hi [16][LM_PPITCH]
  const unsigned pl_base = ph_base + LM_HEADS * LM_PPITCH;           // P lo
  float* wmax = reinterpret_cast<float*>(lm_smem + (size_t)LM_HEADS * pitch + 2 * (size_t)LM_TK * pitch +
                                         2 * LM_HEADS * LM_PPITCH);   // [4 warps][16 rows]
  float* wsum = wmax + 4 * LM_HEADS;                                  // [4 warps][16 rows]

  const int entry = token_req[t];
  const int slot = entry >= 0 ? req_slot[entry] : -1;
  const int p = positions[t];
  const int nsplit = gridDim.z, split = blockIdx.z;
  float* pa = part_acc ? part_acc + (((size_t)(t - first) * H + h0) * nsplit + split) * R : nullptr;
  float* pm = part_ml ? part_ml + (((size_t)(t - first) * H + h0) * nsplit + split) * 2 : nullptr;
  if (slot < 0 || p < 0) {     // a padding entry: defined output, nothing read
    if (nsplit == 1) {
      for (int i = tid; i < hc * R; i += LM_THREADS) out[((size_t)t * H + h0) * R + i] = __float2bfloat16_rn(0.f);
    } else if (tid < hc) {
      pm[(size_t)tid * nsplit * 2] = -INFINITY;
      pm[(size_t)tid * nsplit * 2 + 1] = 0.f;
    }
    return;
  }
  const int* bt = block_table + (size_t)slot * bt_stride;
  const int lo = (window > 0) ? max(0, p - window + 1) : 0;
  const int vpr = KD / 8;                           // 16-byte pieces of a row

  // ---- the queries of the CTA's heads (rows of heads that do not exist are zeros) ----
  for (int i = tid; i < LM_HEADS * vpr; i += LM_THREADS) {
    const int row = i / vpr, piece = i - row * vpr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < hc) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * H + h0 + row) * KD + 8 * piece);
    *reinterpret_cast<uint4*>(lm_smem + (size_t)row * pitch + 16 * piece) = v;
  }

  int tile_begin = (lo / LM_TK) * LM_TK, tile_end = p;      // first positions of the first and (at most) last tile
  if (nsplit > 1) {
    tile_begin += split * tiles_per_split * LM_TK;
    tile_end = min(p, tile_begin + (tiles_per_split - 1) * LM_TK);
  }
  // four threads a key: one look at the block table a thread and tile, then the row's pieces in turn
  const int lkey = tid >> 2, lsub = tid & 3;
  auto load_tile = [&](int buf, int tile0) {
    const int pos = tile0 + lkey;
    const bf16* src = cache;
    int bytes = 0;
    if (pos >= lo && pos <= p) {
      const int page = bt[pos / page_size];
      if (page < 0 || page >= num_pages) {
        set_status(status, LL_ERR_PAGE_RANGE);
      } else {
        src = cache + ((size_t)page * page_size + (pos % page_size)) * KD;
        bytes = 16;
      }
    }
    const unsigned dst = k_base + (buf * LM_TK + lkey) * pitch;
    for (int piece = lsub; piece < vpr; piece += 4)
      lm_cp_async16(dst + 16 * piece, bytes ? src + 8 * piece : src, bytes);
  };

  float o_acc[LM_MAX_NT][4];
#pragma unroll
  for (int nt = 0; nt < LM_MAX_NT; ++nt) o_acc[nt][0] = o_acc[nt][1] = o_acc[nt][2] = o_acc[nt][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8 (l: this thread's share)

  if (tile_begin <= tile_end) load_tile(0, tile_begin);
  lm_commit();
  int n = 0;
  for (int tile0 = tile_begin; tile0 <= tile_end; tile0 += LM_TK, ++n) {
    const int buf = n & 1;
    if (tile0 + LM_TK <= tile_end) load_tile(buf ^ 1, tile0 + LM_TK);
    lm_commit();
    lm_wait<1>();        // everything but the newest group has landed: this tile is complete
    __syncthreads();     // (also: the queries are in place before their first use)
    const unsigned kt = k_base + buf * LM_TK * pitch;
    // ---- S for the warp's 8 keys: two accumulation chains ----
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    {
      // fragments by ldmatrix: the queries' 16 x 16 piece as four 8 x 8 matrices (lane l names row l % 8 of matrix
      // l / 8: heads +8 for the odd ones, channels +8 for the last two), the keys' 8 x 16 piece as two
      const unsigned qa = q_base + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (lane >> 4) * 16;
      const unsigned kk = kt + (8 * warp + (lane & 7)) * pitch + ((lane >> 3) & 1) * 16;
      const int steps = KD / 16;
#pragma unroll 2
      for (int s = 0; s < steps; ++s) {
        unsigned a0, a1, a2, a3, b0, b1;
        lm_ldmatrix_x4(a0, a1, a2, a3, qa + 32 * s);
        lm_ldmatrix_x2(b0, b1, kk + 32 * s);
        if (s & 1) lm_mma(sb, a0, a1, a2, a3, b0, b1);
        else lm_mma(sa, a0, a1, a2, a3, b0, b1);
      }
    }
    float v[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int pos = tile0 + 8 * warp + 2 * c + (x & 1);
      v[x] = (pos >= lo && pos <= p) ? (sa[x] + sb[x]) * scale_log2 : -INFINITY;
    }
    // ---- the rows' maxima over the tile: a quad holds a row's 8 keys of this warp; the warps meet in shared memory
    float mx[2] = {fmaxf(v[0], v[1]), fmaxf(v[2], v[3])};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    if (c == 0) {
      wmax[warp * LM_HEADS + g] = mx[0];
      wmax[warp * LM_HEADS + g + 8] = mx[1];
    }
    __syncthreads();
    float alpha[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = g + 8 * i;
      const float mt = fmaxf(fmaxf(wmax[row], wmax[LM_HEADS + row]), fmaxf(wmax[2 * LM_HEADS + row], wmax[3 * LM_HEADS + row]));
      const float m_new = fmaxf(m_run[i], mt);
      msafe[i] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[i] = lm_exp2(m_run[i] - msafe[i]);
      m_run[i] = m_new;
    }
    float pw[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) pw[x] = lm_exp2(v[x] - msafe[x >> 1]);
    l_run[0] = l_run[0] * alpha[0] + (pw[0] + pw[1]);
    l_run[1] = l_run[1] * alpha[1] + (pw[2] + pw[3]);
    // P into shared memory in two bfloat16 terms: hi, and what hi lost
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat162 hi = __floats2bfloat162_rn(pw[2 * i], pw[2 * i + 1]);
      const unsigned off = (g + 8 * i) * LM_PPITCH + 2 * (8 * warp + 2 * c);
      lm_sts32(ph_base + off, *reinterpret_cast<const unsigned*>(&hi));
      lm_sts32(pl_base + off, lm_pack(pw[2 * i] - __low2float(hi), pw[2 * i + 1] - __high2float(hi)));
    }
    __syncthreads();
    // ---- O = O alpha + P C over the warp's columns ----
    if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
      for (int nt = 0; nt < LM_MAX_NT; ++nt) {
        o_acc[nt][0] *= alpha[0];
        o_acc[nt][1] *= alpha[0];
        o_acc[nt][2] *= alpha[1];
        o_acc[nt][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const unsigned pa0 = ((lane & 7) + ((lane >> 3) & 1) * 8) * LM_PPITCH + (lane >> 4) * 16 + 32 * ks;
      unsigned h0r, h1r, h2r, h3r, l0r, l1r, l2r, l3r;
      lm_ldmatrix_x4(h0r, h1r, h2r, h3r, ph_base + pa0);
      lm_ldmatrix_x4(l0r, l1r, l2r, l3r, pl_base + pa0);
      const unsigned vrow = kt + (16 * ks + (lane & 15)) * pitch + 2 * (8 * warp * ntw);
#pragma unroll
      for (int nt = 0; nt < LM_MAX_NT; ++nt) {
        if (nt < ntw) {
          unsigned b0, b1;
          lm_ldmatrix_x2_trans(b0, b1, vrow + 16 * nt);
          lm_mma(o_acc[nt], h0r, h1r, h2r, h3r, b0, b1);
          lm_mma(o_acc[nt], l0r, l1r, l2r, l3r, b0, b1);
        }
      }
    }
    __syncthreads();     // the tile, P and the maxima may be overwritten
  }
  lm_wait<0>();

  // ---- the rows' sums: over the quad, then over the warps ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  if (c == 0) {
    wsum[warp * LM_HEADS + g] = l_run[0];
    wsum[warp * LM_HEADS + g + 8] = l_run[1];
  }
  __syncthreads();
  float l_tot[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = g + 8 * i;
    l_tot[i] = (wsum[row] + wsum[LM_HEADS + row]) + (wsum[2 * LM_HEADS + row] + wsum[3 * LM_HEADS + row]);
  }
  if (nsplit == 1) {
    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = g + 8 * i;
      // the key without a value: one more term of the sum
      const float l = (sink && row < hc) ? l_tot[i] + lm_exp2(sink[h0 + row] * LM_LOG2E - m_run[i]) : l_tot[i];
      inv[i] = l > 0.f ? 1.0f / l : 0.f;
    }
#pragma unroll
    for (int nt = 0; nt < LM_MAX_NT; ++nt) {
      if (nt < ntw) {
        const int col = 8 * (warp * ntw + nt) + 2 * c;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int row = g + 8 * i;
          if (row < hc)
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * H + h0 + row) * R + col) =
                __floats2bfloat162_rn(o_acc[nt][2 * i] * inv[i], o_acc[nt][2 * i + 1] * inv[i]);
        }
      }
    }
    return;
  }
  // ---- this part of every row for the merge: sums as they are, the maximum (natural units) and the sum ----
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = g + 8 * i;
    if (row < hc) {
      float* dst = pa + (size_t)row * nsplit * R;
#pragma unroll
      for (int nt = 0; nt < LM_MAX_NT; ++nt) {
        if (nt < ntw) {
          const int col = 8 * (warp * ntw + nt) + 2 * c;
          *reinterpret_cast<float2*>(dst + col) = make_float2(o_acc[nt][2 * i], o_acc[nt][2 * i + 1]);
        }
      }
      if (warp == 0 && c == 0) {
        pm[(size_t)row * nsplit * 2] = m_run[i] == -INFINITY ? -INFINITY : m_run[i] * (1.0f / LM_LOG2E);
        pm[(size_t)row * nsplit * 2 + 1] = l_tot[i];
      }
    }
  }
}

// Whether the tensor-core kernel takes these sizes (bfloat16 only; the launcher checks the dtype and alignment).
extern "C" int ll_latent_attention_mma_ok(int R, int r) {
  const int KD = R + r;
  return (KD % 16) == 0 && (R % 32) == 0 && R > 0 && R <= 32 * LM_MAX_NT && r >= 0;
}

extern "C" int ll_latent_attention_mma(void* out, const void* q, const void* cache, const int* block_table, int bt_stride,
                                       const int* token_req, const int* req_slot, const int* positions, int first,
                                       int num_tokens, int H, int R, int r, int page_size, int num_pages, int window,
                                       float scale, int* status, int nsplit, int tiles_per_split, float* part_acc,
                                       float* part_ml, const float* sink, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (!ll_latent_attention_mma_ok(R, r) || H <= 0 || page_size <= 0 || nsplit < 1) return (int)cudaErrorInvalidValue;
  const int pitch = 2 * (R + r) + 16;
  const size_t smem = (size_t)LM_HEADS * pitch + 2 * (size_t)LM_TK * pitch + 2 * LM_HEADS * LM_PPITCH +
                      2 * 4 * LM_HEADS * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(num_tokens, (H + LM_HEADS - 1) / LM_HEADS, nsplit);
  ll_launch(latent_attention_mma_kernel, grid, dim3(LM_THREADS), smem, stream, (bf16*)out, (const bf16*)q,
            (const bf16*)cache, block_table, bt_stride, token_req, req_slot, positions, first, H, R, r, page_size,
            num_pages, window, scale * LM_LOG2E, status, tiles_per_split, part_acc, part_ml, sink);
  return LL_LAUNCH_RESULT();
}
