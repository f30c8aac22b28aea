// Latent attention: softmax attention whose keys and values are expansions of one latent vector per token.
//
// Per token the cache holds one row [R + r]: the normed latent c (R numbers) and a rotated key part k_r (r
// numbers) that all heads share.  With per-head expansions k_h = Uk_h c and v_h = Uv_h c the score of query
// head h against a token is (q_h . Uk_h c + q_r,h . k_r) * scale = ((Uk_h^T q_h) . c + q_r,h . k_r) * scale, and
// the head's output is Uv_h (sum_j p_j c_j).  So the kernel here works in the latent space: its queries are
// a_h = Uk_h^T q_h (R numbers, made by a batched product before it) and the rotated part, its keys are the
// cached rows, its values the first R numbers of the same rows, and what it returns is sum_j p_j c_j per head
// (expanded by a batched product after it).  Nothing per head is ever cached or re-expanded.
//
// Rotation (interleaved pairs): numbers 2i and 2i+1 of a rotated part, for 2i < rot_dims, turn by the angle
// position * freq[i]; (u, v) -> (u cos - v sin, v cos + u sin); the rest passes unchanged.  Angles, the
// latent's norm, scores and softmax are float32.
//
//   latent_prepare    per token: RMS norm of the latent, rotation of k_r and of every head's q_r, cache write
//   latent_attention  per (token, 8 heads): online softmax over the visible rows of the request, i.e.
//                     positions lo..p with lo = max(0, p - window + 1) (window <= 0: all)
//   latent_gather, latent_masked_softmax: the pieces between two library products for long prompt portions,
//                     where all (token, head) rows of a block of queries meet the same run of cached rows:
//                     the run is copied out of its pages, scores = Q K^T and sum = P C are products, and the
//                     masked softmax between them is the kernel here
// In latent_attention keys are walked in tiles of 32 positions that start at multiples of 32, so the order of
// every sum depends on the position only, not on how the tokens were cut into steps or batched.
#include "common.cuh"

// qsrc row t (row stride q_stride; the projection itself, or the output of a second product when the queries go
// through a latent of their own): q heads at q_off, head h's rotated part at q_off + h * (d + r) + d; proj row t:
// the latent at kv_off (R wide), then the rotated key part (r wide).  Both cos and sin are multiplied by
// `amplitude` (a scaled rotation's factor; 1 otherwise).
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, long proj_stride, int q_off, int kv_off, const float* __restrict__ norm_w,
                      float eps, const float* __restrict__ freq, int rot_dims, const int* __restrict__ positions,
                      const int* __restrict__ slot_map, T* __restrict__ cache, long num_slots,
                      T* __restrict__ q_full, int H, int d, int r, int R, int* status, float amplitude,
                      const T* __restrict__ qsrc, long q_stride) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x, tid = threadIdx.x;
  const T* row = proj + (size_t)t * proj_stride;
  const float p = (float)positions[t];
  // every head's rotated query part -> q_full [tokens, H, R + r] behind the R latent-space numbers
  const int half = rot_dims / 2;
  for (int i = tid; i < H * r; i += blockDim.x) {
    const int h = i / r, j = i % r;
    const T* src = qsrc + (size_t)t * q_stride + q_off + (size_t)h * (d + r) + d;
    float out;
    if (j < 2 * half) {
      float sn, cs;
      sincosf(p * freq[j >> 1], &sn, &cs);
      sn *= amplitude;
      cs *= amplitude;
      const float u = to_f32<T>(src[j & ~1]), v = to_f32<T>(src[j | 1]);
      out = (j & 1) ? v * cs + u * sn : u * cs - v * sn;
    } else {
      out = to_f32<T>(src[j]);
    }
    q_full[((size_t)t * H + h) * (R + r) + R + j] = from_f32<T>(out);
  }
  const long slot = slot_map ? slot_map[t] : -1;
  if (slot < 0) return;     // padding token, or a run-step that only reads this plane
  if (slot >= num_slots) {
    if (tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    return;
  }
  const T* lat = row + kv_off;
  float ss = 0.f;
  for (int i = tid; i < R; i += blockDim.x) {
    const float x = to_f32<T>(lat[i]);
    ss = fmaf(x, x, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)R + eps);
  T* dst = cache + (size_t)slot * (R + r);
  for (int i = tid; i < R; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(lat[i]) * inv * norm_w[i]);
  for (int j = tid; j < r; j += blockDim.x) {
    float out;
    if (j < 2 * half) {
      float sn, cs;
      sincosf(p * freq[j >> 1], &sn, &cs);
      sn *= amplitude;
      cs *= amplitude;
      const float u = to_f32<T>(lat[R + (j & ~1)]), v = to_f32<T>(lat[R + (j | 1)]);
      out = (j & 1) ? v * cs + u * sn : u * cs - v * sn;
    } else {
      out = to_f32<T>(lat[R + j]);
    }
    dst[R + j] = from_f32<T>(out);
  }
}

#define LA_TK 32
#define LA_THREADS 256
#define LA_WARPS 8
#define LA_HPW (LA_GH / LA_WARPS)     // heads a warp scores
#define LA_CPT (LA_MAX_R / LA_THREADS) // latent columns a thread sums
#define LA_GH 8
#define LA_MAX_R 512
#define LA_PIPE 9       // 16-byte pieces of a tile a thread may hold: rows of up to 576 bfloat16 numbers
// floats from one row of a tile in shared memory to the next
__host__ __device__ static inline int la_pitch(int KD) { return (KD & 3) == 0 ? ((KD + 27) / 32) * 32 + 4 : KD + 1; }

// q: [tokens, H, R + r] of T (latent-space queries, then the rotated part); cache: one plane
// [pages, 1, page_size, R + r]; out: [tokens, H, R] of T.  `first` is the first token of the launch.
template <typename T>
__global__ void __launch_bounds__(LA_THREADS)
latent_attention_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ cache,
                        const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
                        const int* __restrict__ req_slot, const int* __restrict__ positions, int first, int H, int R,
                        int r, int page_size, int num_pages, int window, float scale, int* status,
                        int tiles_per_split, float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const float* __restrict__ sink) {
  extern __shared__ __align__(16) float smem[];
  __shared__ long base_s[LA_TK];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = first + blockIdx.x;
  const int h0 = blockIdx.y * LA_GH;
  const int hc = min(LA_GH, H - h0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int KD = R + r;
  float* qs = smem;                         // [LA_GH][KD]
  // a row of the tile is KP floats apart.  Rows whose width is a multiple of 4 are read four numbers at a time:
  // KP = 4 mod 32 then, so that the 16-byte reads of a quarter warp (lane = key) meet 32 different banks
  const bool v4 = (KD & 3) == 0;
  const int KP = la_pitch(KD);
  float* ks = qs + LA_GH * KD;              // [LA_TK][KP]
  float* ps = ks + LA_TK * KP;              // [LA_TK][LA_GH]
  float* alpha_s = ps + LA_GH * LA_TK;      // [LA_GH]
  float* l_s = alpha_s + LA_GH;             // [LA_GH]

  const int entry = token_req[t];
  const int slot = entry >= 0 ? req_slot[entry] : -1;
  const int p = positions[t];
  T* o_row = out + ((size_t)t * H + h0) * R;
  // with gridDim.z > 1 the keys of a query are shared out: split z walks tiles_per_split tiles (counted from the
  // query's first tile) and leaves its running maximum, sum and unnormalised accumulator for the merge kernel
  const int nsplit = gridDim.z, split = blockIdx.z;
  float* pa = part_acc ? part_acc + (((size_t)(t - first) * H + h0) * nsplit + split) * R : nullptr;
  float* pm = part_ml ? part_ml + (((size_t)(t - first) * H + h0) * nsplit + split) * 2 : nullptr;
  if (slot < 0 || p < 0) {
    if (nsplit == 1) {
      for (int i = tid; i < hc * R; i += LA_THREADS) o_row[i] = from_f32<T>(0.f);
    } else if (tid < hc) {
      pm[(size_t)tid * nsplit * 2] = -INFINITY;
      pm[(size_t)tid * nsplit * 2 + 1] = 0.f;
    }
    return;
  }
  const int* bt = block_table + (size_t)slot * bt_stride;
  const int lo = (window > 0) ? max(0, p - window + 1) : 0;
  const T* q_row = q + ((size_t)t * H + h0) * KD;
  for (int i = tid; i < hc * KD; i += LA_THREADS) qs[i] = to_f32<T>(q_row[i]);
  for (int i = hc * KD + tid; i < LA_GH * KD; i += LA_THREADS) qs[i] = 0.f;
  float m_run[LA_GH / LA_WARPS], l_run[LA_GH / LA_WARPS];
#pragma unroll
  for (int i = 0; i < LA_GH / LA_WARPS; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
  }
  float acc[LA_GH][LA_MAX_R / LA_THREADS];
#pragma unroll
  for (int g = 0; g < LA_GH; ++g)
#pragma unroll
    for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) acc[g][c] = 0.f;
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec_ok = (KD % VEC) == 0 && ((uintptr_t)cache % 16) == 0;

  // The rows of a tile come through registers a tile ahead where the pieces fit (16-byte pieces, at most LA_PIPE a
  // thread): every thread asks for all its pieces of the next tile before it works on this one, so a CTA has a
  // whole tile in flight instead of four pieces a thread, and the wait lies under the arithmetic.
  const int vpr = KD / VEC;
  const bool piped = vec_ok && LA_TK * vpr <= LA_PIPE * LA_THREADS;
  uint4 raw[LA_PIPE];
  auto ask = [&](int tile0) {
#pragma unroll
    for (int u = 0; u < LA_PIPE; ++u) {
      const int i = tid + u * LA_THREADS;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (i < LA_TK * vpr) {
        const int row = i / vpr;
        const int pos = tile0 + row;
        if (pos >= lo && pos <= p) {
          const int page = bt[pos / page_size];
          if (page < 0 || page >= num_pages) set_status(status, LL_ERR_PAGE_RANGE);
          else raw[u] = *reinterpret_cast<const uint4*>(cache + ((long)page * page_size + (pos % page_size)) * KD +
                                                        (size_t)(i - row * vpr) * VEC);
        }
      }
    }
  };
  auto put = [&]() {
#pragma unroll
    for (int u = 0; u < LA_PIPE; ++u) {
      const int i = tid + u * LA_THREADS;
      if (i < LA_TK * vpr) {
        const T* e = reinterpret_cast<const T*>(&raw[u]);
        float* dst = ks + (i / vpr) * KP + (i % vpr) * VEC;
        if (v4) {       // (rows start at multiples of 16 bytes then)
#pragma unroll
          for (int x = 0; x < VEC; x += 4)
            *reinterpret_cast<float4*>(dst + x) =
                make_float4(to_f32<T>(e[x]), to_f32<T>(e[x + 1]), to_f32<T>(e[x + 2]), to_f32<T>(e[x + 3]));
        } else {
#pragma unroll
          for (int x = 0; x < VEC; ++x) dst[x] = to_f32<T>(e[x]);
        }
      }
    }
  };
  int tile_begin = (lo / LA_TK) * LA_TK, tile_end = p;      // first positions of the first and (at most) last tile
  if (nsplit > 1) {
    tile_begin += split * tiles_per_split * LA_TK;
    tile_end = min(p, tile_begin + (tiles_per_split - 1) * LA_TK);
  }
  if (piped && tile_begin <= tile_end) ask(tile_begin);
  for (int tile0 = tile_begin; tile0 <= tile_end; tile0 += LA_TK) {
    __syncthreads();
    if (piped) {
      put();
      __syncthreads();
      if (tile0 + LA_TK <= tile_end) ask(tile0 + LA_TK);
    } else {
    if (tid < LA_TK) {
      const int pos = tile0 + tid;
      long base = -1;
      if (pos >= lo && pos <= p) {
        const int page = bt[pos / page_size];
        if (page < 0 || page >= num_pages) set_status(status, LL_ERR_PAGE_RANGE);
        else base = ((long)page * page_size + (pos % page_size)) * KD;
      }
      base_s[tid] = base;
    }
    __syncthreads();
    // the tile's rows: every thread asks for four pieces before it uses the first
    if (vec_ok) {
      const int vpr = KD / VEC, total = LA_TK * vpr;
      for (int i0 = tid; i0 < total; i0 += LA_THREADS * 4) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * LA_THREADS;
          v[u] = make_uint4(0, 0, 0, 0);
          if (i < total) {
            const long base = base_s[i / vpr];
            if (base >= 0) v[u] = *reinterpret_cast<const uint4*>(cache + base + (size_t)(i % vpr) * VEC);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * LA_THREADS;
          if (i < total) {
            const T* e = reinterpret_cast<const T*>(&v[u]);
            float* dst = ks + (i / vpr) * KP + (i % vpr) * VEC;
#pragma unroll
            for (int x = 0; x < VEC; ++x) dst[x] = to_f32<T>(e[x]);
          }
        }
      }
    } else {
      const int total = LA_TK * KD;
      for (int i0 = tid; i0 < total; i0 += LA_THREADS * 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * LA_THREADS;
          v[u] = 0.f;
          if (i < total) {
            const long base = base_s[i / KD];
            if (base >= 0) v[u] = to_f32<T>(cache[base + i % KD]);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * LA_THREADS;
          if (i < total) ks[(i / KD) * KP + i % KD] = v[u];
        }
      }
    }
    __syncthreads();
    }
    {
      // scores and online softmax: warp w owns heads w, w + LA_WARPS, ...; lane = key
      const int pos = tile0 + lane;
      const bool valid = (pos >= lo && pos <= p);
      float sh[LA_HPW];
      const float* kj = ks + lane * KP;
      if (v4) {
        const float4* kv4 = reinterpret_cast<const float4*>(kj);
        float sa[LA_HPW], sb[LA_HPW], sc[LA_HPW], sd[LA_HPW];      // four sums side by side a head
#pragma unroll
        for (int i = 0; i < LA_HPW; ++i) sa[i] = sb[i] = sc[i] = sd[i] = 0.f;
#pragma unroll 4
        for (int c = 0; c < KD / 4; ++c) {
          const float4 kv = kv4[c];
#pragma unroll
          for (int i = 0; i < LA_HPW; ++i) {
            const float4 a = reinterpret_cast<const float4*>(qs + (warp + i * LA_WARPS) * KD)[c];
            sa[i] = fmaf(a.x, kv.x, sa[i]);
            sb[i] = fmaf(a.y, kv.y, sb[i]);
            sc[i] = fmaf(a.z, kv.z, sc[i]);
            sd[i] = fmaf(a.w, kv.w, sd[i]);
          }
        }
#pragma unroll
        for (int i = 0; i < LA_HPW; ++i) sh[i] = (sa[i] + sb[i]) + (sc[i] + sd[i]);
      } else {
#pragma unroll
        for (int i = 0; i < LA_HPW; ++i) sh[i] = 0.f;
        for (int c = 0; c < KD; ++c) {
          const float kv = kj[c];
#pragma unroll
          for (int i = 0; i < LA_HPW; ++i) sh[i] = fmaf(qs[(warp + i * LA_WARPS) * KD + c], kv, sh[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < LA_HPW; ++i) {
        const int g = warp + i * LA_WARPS;
        if (g < hc) {
          const float s = valid ? sh[i] * scale : -INFINITY;
          const float m_new = fmaxf(m_run[i], warp_max(s));
          const float pj = valid ? expf(s - m_new) : 0.f;
          const float alpha = expf(m_run[i] - m_new);
          l_run[i] = l_run[i] * alpha + warp_sum(pj);
          m_run[i] = m_new;
          ps[lane * LA_GH + g] = pj;
          if (lane == 0) alpha_s[g] = alpha;
        } else {
          ps[lane * LA_GH + g] = 0.f;
          if (lane == 0) alpha_s[g] = 1.f;
        }
      }
    }
    __syncthreads();
    // accumulate P C: a thread owns LA_CPT neighbouring latent columns (rows read that many numbers at a time) or
    // columns tid, tid + LA_THREADS, ...; a key's number is read once for all heads
    if (v4) {
      static_assert(LA_CPT == 2, "the vector path reads two columns a thread");
      if (LA_CPT * tid < R) {
#pragma unroll
        for (int g = 0; g < LA_GH; ++g)
#pragma unroll
          for (int c = 0; c < LA_CPT; ++c) acc[g][c] *= alpha_s[g];
#pragma unroll 4
        for (int j = 0; j < LA_TK; ++j) {
          const float2 kv = *reinterpret_cast<const float2*>(ks + j * KP + LA_CPT * tid);
          const float4 pa = *reinterpret_cast<const float4*>(ps + j * LA_GH);
          const float4 pb = *reinterpret_cast<const float4*>(ps + j * LA_GH + 4);
          const float pw[LA_GH] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
          for (int g = 0; g < LA_GH; ++g) {
            acc[g][0] = fmaf(pw[g], kv.x, acc[g][0]);
            acc[g][1] = fmaf(pw[g], kv.y, acc[g][1]);
          }
        }
      }
    } else
#pragma unroll
    for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) {
      const int dd = tid + c * LA_THREADS;
      if (dd < R) {
#pragma unroll
        for (int g = 0; g < LA_GH; ++g) acc[g][c] *= alpha_s[g];
#pragma unroll 4
        for (int j = 0; j < LA_TK; ++j) {
          const float kv = ks[j * KP + dd];
          const float4 pa = *reinterpret_cast<const float4*>(ps + j * LA_GH);
          const float4 pb = *reinterpret_cast<const float4*>(ps + j * LA_GH + 4);
          acc[0][c] = fmaf(pa.x, kv, acc[0][c]);
          acc[1][c] = fmaf(pa.y, kv, acc[1][c]);
          acc[2][c] = fmaf(pa.z, kv, acc[2][c]);
          acc[3][c] = fmaf(pa.w, kv, acc[3][c]);
          acc[4][c] = fmaf(pb.x, kv, acc[4][c]);
          acc[5][c] = fmaf(pb.y, kv, acc[5][c]);
          acc[6][c] = fmaf(pb.z, kv, acc[6][c]);
          acc[7][c] = fmaf(pb.w, kv, acc[7][c]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < LA_GH / LA_WARPS; ++i) {
    const int g = warp + i * LA_WARPS;
    if (g < hc && lane == 0) {
      // the key without a value: one more term of the sum (with splits the merge adds it)
      l_s[g] = (sink && nsplit == 1) ? l_run[i] + expf(sink[h0 + g] - m_run[i]) : l_run[i];
      if (nsplit > 1) {
        pm[(size_t)g * nsplit * 2] = m_run[i];
        pm[(size_t)g * nsplit * 2 + 1] = l_run[i];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < LA_MAX_R / LA_THREADS; ++c) {
    const int dd = v4 ? LA_CPT * tid + c : tid + c * LA_THREADS;
    if (dd < R) {
#pragma unroll
      for (int g = 0; g < LA_GH; ++g)
        if (g < hc) {
          if (nsplit == 1) o_row[(size_t)g * R + dd] = from_f32<T>(acc[g][c] / l_s[g]);
          else pa[(size_t)g * nsplit * R + dd] = acc[g][c];
        }
    }
  }
}

// The splits of a (token, head) put together, in the order of the splits: out = sum_s e^(m_s - M) acc_s /
// sum_s e^(m_s - M) l_s with M the largest m_s.  One block per (token, head); a thread owns latent numbers
// tid, tid + 128, ... and asks for all splits' values of a number before it adds them up.
#define LA_MAX_SPLIT 32
template <typename T>
__global__ void __launch_bounds__(128)
latent_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                    int pairs, int R, int nsplit, const float* __restrict__ sink, int H) {
  __shared__ float w_s[LA_MAX_SPLIT];
  __shared__ float inv_s;
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int pair = blockIdx.x;
  const int tid = threadIdx.x;
  const float* ml = part_ml + (size_t)pair * nsplit * 2;
  if (tid < 32) {
    float m = tid < nsplit ? ml[2 * tid] : -INFINITY;
    float M = warp_max(m);
    const float sk = sink ? sink[pair % H] : -INFINITY;
    M = fmaxf(M, sk);
    const float w = (tid < nsplit && m != -INFINITY) ? expf(m - M) : 0.f;
    w_s[tid] = w;
    float L = 0.f;
    for (int s = 0; s < nsplit; ++s) L = fmaf(__shfl_sync(0xffffffffu, w, s), ml[2 * s + 1], L);   // split order
    if (sink) L += expf(sk - M);
    if (tid == 0) inv_s = L > 0.f ? 1.0f / L : 0.f;
  }
  __syncthreads();
  T* o = out + (size_t)pair * R;      // (`out` points at the launch's first token)
  const float* pa = part_acc + (size_t)pair * nsplit * R;
  for (int d = tid; d < R; d += 128) {
    float a = 0.f;
#pragma unroll 8
    for (int s = 0; s < nsplit; ++s) a = fmaf(w_s[s], pa[(size_t)s * R + d], a);
    o[d] = from_f32<T>(a * inv_s);
  }
}

// Rows first .. last of a request's cached rows, copied out of their pages into dst [n, KD], row j being
// position lo + j; rows of positions outside first .. last are zeros (the run is padded to a width that
// library products like).
template <typename T>
__global__ void latent_gather_kernel(T* __restrict__ dst, const T* __restrict__ cache, const int* __restrict__ bt,
                                     int lo, int first, int last, int n, int KD, int page_size, int num_pages,
                                     int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  for (int j = blockIdx.x; j < n; j += gridDim.x) {
    const int pos = lo + j;
    if (pos < first || pos > last) {
      for (int c = threadIdx.x; c < KD; c += blockDim.x) dst[(size_t)j * KD + c] = from_f32<T>(0.f);
      continue;
    }
    const int page = bt[pos / page_size];
    const bool ok = page >= 0 && page < num_pages;
    if (!ok && threadIdx.x == 0) set_status(status, LL_ERR_PAGE_RANGE);
    const T* src = cache + ((size_t)(ok ? page : 0) * page_size + (pos % page_size)) * KD;
    for (int c = threadIdx.x; c < KD; c += blockDim.x) dst[(size_t)j * KD + c] = ok ? src[c] : from_f32<T>(0.f);
  }
}

// Row i = (query token i / H of the block, head i % H): scores S [rows, n_keys] float32, key column j is
// position lo + j; the query's position is p0 + i / H and it sees columns with
// max(lo, p - window + 1) <= lo + j <= p.  P = softmax(scale * S) over those, zero elsewhere, in T.
template <typename T>
__global__ void __launch_bounds__(256)
latent_masked_softmax_kernel(T* __restrict__ P, const float* __restrict__ S, int rows, int n_keys, int H, int p0, int lo,
                             int window, float scale, const float* __restrict__ sink) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int i = blockIdx.x;
  const int p = p0 + i / H;
  const int first = (window > 0 ? max(lo, p - window + 1) : lo) - lo, last = p - lo;   // visible columns, inclusive
  const float* s = S + (size_t)i * n_keys;
  T* out = P + (size_t)i * n_keys;
  float m = -INFINITY;
  for (int j = first + threadIdx.x; j <= last; j += blockDim.x) m = fmaxf(m, s[j] * scale);
  m = block_max(m, scratch);
  if (sink) m = fmaxf(m, sink[i % H]);        // the key without a value: in the denominator only
  float sum = 0.f;
  for (int j = first + threadIdx.x; j <= last; j += blockDim.x) sum += expf(s[j] * scale - m);
  sum = block_sum(sum, scratch);
  if (sink) sum += expf(sink[i % H] - m);
  const float inv = 1.0f / sum;
  for (int j = threadIdx.x; j < n_keys; j += blockDim.x)
    out[j] = from_f32<T>((j >= first && j <= last) ? expf(s[j] * scale - m) * inv : 0.f);
}

extern "C" int ll_latent_prepare(int dtype, const void* proj, long proj_stride, int q_off, int kv_off,
                                 const float* norm_w, float eps, const float* freq, int rot_dims, const int* positions,
                                 const int* slot_map, void* cache, long num_slots, void* q_full, int num_tokens, int H,
                                 int d, int r, int R, int* status, float amplitude, const void* qsrc, long q_stride,
                                 cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || d < 0 || r < 0 || R <= 0 || rot_dims < 0 || rot_dims > r) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, ll_launch(latent_prepare_kernel<T>, dim3(num_tokens), dim3(128), 0, stream, (const T*)proj,
                                     proj_stride, q_off, kv_off, norm_w, eps, freq, rot_dims, positions, slot_map,
                                     (T*)cache, num_slots, (T*)q_full, H, d, r, R, status, amplitude,
                                     (const T*)qsrc, q_stride));
  return LL_LAUNCH_RESULT();
}

// (latent_attention_mma.cu: the same work on tensor cores, for the sizes it takes)
extern "C" int ll_latent_attention_mma_ok(int R, int r);
extern "C" int ll_latent_attention_mma(void* out, const void* q, const void* cache, const int* block_table, int bt_stride,
                                       const int* token_req, const int* req_slot, const int* positions, int first,
                                       int num_tokens, int H, int R, int r, int page_size, int num_pages, int window,
                                       float scale, int* status, int nsplit, int tiles_per_split, float* part_acc,
                                       float* part_ml, const float* sink, cudaStream_t stream);
static bool la_mma_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("LITE_LANG_B200_LATENT_MMA");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
// Heads a CTA takes for these sizes: 16 on the tensor-core kernel, 8 on the other.
extern "C" int ll_latent_attention_heads(int dtype, int R, int r) {
  return (dtype == LL_DTYPE_BF16 && la_mma_enabled() && ll_latent_attention_mma_ok(R, r)) ? 16 : LA_GH;
}

extern "C" int ll_latent_attention(int dtype, void* out, const void* q, const void* cache, const int* block_table,
                                   int bt_stride, const int* token_req, const int* req_slot, const int* positions,
                                   int first, int num_tokens, int H, int R, int r, int page_size, int num_pages,
                                   int window, float scale, int* status, int nsplit, int tiles_per_split,
                                   float* part_acc, float* part_ml, const float* sink, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || R <= 0 || R > LA_MAX_R || r < 0 || page_size <= 0 || nsplit < 1) return (int)cudaErrorInvalidValue;
  if (nsplit > 32 || (nsplit > 1 && (tiles_per_split < 1 || part_acc == nullptr || part_ml == nullptr)))
    return (int)cudaErrorInvalidValue;
  const int KD = R + r;
  if (ll_latent_attention_heads(dtype, R, r) == 16 && ((uintptr_t)cache % 16) == 0 && ((uintptr_t)q % 16) == 0) {
    const int rc = ll_latent_attention_mma(out, q, cache, block_table, bt_stride, token_req, req_slot, positions, first,
                                           num_tokens, H, R, r, page_size, num_pages, window, scale, status, nsplit,
                                           tiles_per_split, part_acc, part_ml, sink, stream);
    if (rc != 0 || nsplit == 1) return rc;
    const int pairs = num_tokens * H;
    ll_launch(latent_merge_kernel<bf16>, dim3(pairs), dim3(128), 0, stream, (bf16*)out + (size_t)first * H * R,
              (const float*)part_acc, (const float*)part_ml, pairs, R, nsplit, sink, H);
    return LL_LAUNCH_RESULT();
  }
  const size_t smem = sizeof(float) * ((size_t)LA_GH * KD + (size_t)LA_TK * la_pitch(KD) + LA_GH * LA_TK + 2 * LA_GH);
  dim3 grid(num_tokens, (H + LA_GH - 1) / LA_GH, nsplit);
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(latent_attention_kernel<T>, grid, dim3(LA_THREADS), smem, stream, (T*)out, (const T*)q, (const T*)cache,
              block_table, bt_stride, token_req, req_slot, positions, first, H, R, r, page_size, num_pages, window,
              scale, status, tiles_per_split, part_acc, part_ml, sink);
    if (nsplit > 1) {
      const int pairs = num_tokens * H;
      ll_launch(latent_merge_kernel<T>, dim3(pairs), dim3(128), 0, stream, (T*)out + (size_t)first * H * R,
                (const float*)part_acc, (const float*)part_ml, pairs, R, nsplit, sink, H);
    }
  });
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_latent_gather(int dtype, void* dst, const void* cache, const int* bt_row, int lo, int first, int last,
                                int n, int KD, int page_size, int num_pages, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(latent_gather_kernel<T>, dim3(n < 1024 ? n : 1024), dim3(128), 0, stream, (T*)dst,
                                     (const T*)cache, bt_row, lo, first, last, n, KD, page_size, num_pages, status));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_latent_masked_softmax(int dtype, void* P, const float* S, int rows, int n_keys, int H, int p0, int lo,
                                        int window, float scale, const float* sink, cudaStream_t stream) {
  if (rows <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(latent_masked_softmax_kernel<T>, dim3(rows), dim3(256), 0, stream, (T*)P, S, rows,
                                     n_keys, H, p0, lo, window, scale, sink));
  return LL_LAUNCH_RESULT();
}
