// What stands between a q|k|v projection and an attention whose queries, keys and values are normalised:
// bias, norms, rotary position encoding with angles made in the kernel, and the write into the paged cache.
//
// Row t of `qkv` holds nh query heads and nkv key heads of hd values, then nkv value heads of vd values (columns
// behind those, a per-head gate say, are left alone).  In this order, all in float32:
//   * bias (optional) is added;
//   * norm_mode 2: q as one vector of nh * hd values becomes q / sqrt(mean(q^2) + eps) * qw, and k alike over
//     its nkv * hd values with kw (a norm over the whole projection, with weights, before the rotation);
//   * the first rot_dim values of every q and k head are rotated by angle = float(position) * freq[i]
//     (freq float32 [rot_dim / 2], any scaling of the frequencies already inside), pairs (2i, 2i+1) when
//     `interleaved`, (i, i + rot_dim/2) otherwise: (u, v) -> amp (u cos a - v sin a, v cos a + u sin a), with
//     the accurate cosf and sinf; `amp` is a constant on both (1: plain rotation);
//   * norm_mode 1: every q and k head becomes u / sqrt(mean(u^2) + eps) (per head, no weight, after the
//     rotation);
//   * value_norm: every value head becomes u / sqrt(mean(u^2) + eps).
// q is written back in place, rounded once; k and v go to the token's cache slot, so the cache holds them
// normalised.  One block a token, the row in shared memory.
//
// With `mix` (float32 [nh, nh]) the kernel also leaves, for an attention that mixes its heads' scores by that
// matrix, the queries such an attention can take in one product: s'_h = sum_a mix[h, a] t_a (q_a . k_kv(a)) is
// Q'_h . [k_0 | .. | k_(nkv-1)] with Q'_h[c * hd + d] = sum over the heads a of kv head c of mix[h, a] t_a q_a[d]
// (t: `mix_temp`, float32 [nh], optional).  qmix [tokens, nh, nkv * hd], made from the float32 row, rounded once.
//
// Without `mix`, `mix_temp` (float32 [nh], optional) is a factor a head on q itself, applied before the one
// rounding: an attention that takes its scores times a number a head can then run as a plain one.
//
// Two kernels.  The general one keeps the token's row in shared memory (any sizes, both pair layouts).  When the
// rotation pairs are neighbours (or there is no rotation) and the head sizes are multiples of 8 up to 256, a team
// of 8, 16 or 32 lanes takes a head and a lane eight neighbouring values (four pairs) in registers: 16 bytes of
// bfloat16 a load and a store, one pass, the head's sum of squares by shuffles within the team; only the mixed
// queries go through shared memory.
//
// Cache plane: K [num_pages, nkv, page_size, hd], V [num_pages, nkv, page_size, vd].
#include "common.cuh"

// eight neighbouring values (p on a 16-byte boundary for bfloat16, a 32-byte one for float32)
template <typename T> __device__ __forceinline__ void qn_load8(const T* p, float v[8]);
template <> __device__ __forceinline__ void qn_load8<float>(const float* p, float v[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <> __device__ __forceinline__ void qn_load8<bf16>(const bf16* p, float v[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    v[2 * k] = f.x, v[2 * k + 1] = f.y;
  }
}
template <typename T> __device__ __forceinline__ void qn_store8(T* p, const float v[8], float factor);
template <> __device__ __forceinline__ void qn_store8<float>(float* p, const float v[8], float f) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0] * f, v[1] * f, v[2] * f, v[3] * f);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4] * f, v[5] * f, v[6] * f, v[7] * f);
}
template <> __device__ __forceinline__ void qn_store8<bf16>(bf16* p, const float v[8], float f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k] * f, v[2 * k + 1] * f);
  *reinterpret_cast<uint4*>(p) = u;
}

// L lanes a head (8, 16 or 32: head sizes up to 8 L), 32 / L heads a warp at a time.
template <typename T, int L>
__global__ void __launch_bounds__(256)
qkv_norm_rotate_store_teams_kernel(T* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                                   const int* __restrict__ positions, const float* __restrict__ freq, int rot_dim,
                                   float amp, int nh, int nkv, int hd, int vd, int norm_mode,
                                   const float* __restrict__ qw, const float* __restrict__ kw, int value_norm, float eps,
                                   const int* __restrict__ slot_map, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                   int page_size, long num_slots, const float* __restrict__ mix,
                                   const float* __restrict__ mix_temp, T* __restrict__ qmix, int* status) {
  extern __shared__ __align__(16) float team_row[];   // with mix: q as float32 [nh * hd]; then cos and sin [rot_dim / 2] each
  float* row = team_row;
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int qn = nh * hd, kn = nkv * hd;
  const int half = rot_dim >> 1;
  const bool mixing = mix != nullptr && qmix != nullptr;
  float* cs = row + (mixing ? qn : 0);
  float* sn = cs + half;
  T* g = qkv + (size_t)t * qkv_stride;
  long slot = slot_map ? (long)slot_map[t] : -1;
  const float pos = (float)(positions ? positions[t] : 0);
  for (int i = tid; i < half; i += blockDim.x) {
    const float a = pos * freq[i];
    cs[i] = cosf(a) * amp;
    sn[i] = sinf(a) * amp;
  }
  float iq = 1.0f, ik = 1.0f;
  if (norm_mode == 2) {
    float sq = 0.f, sk = 0.f;
    for (int i = 8 * tid; i < qn + kn; i += 8 * blockDim.x) {       // (qn is a multiple of 8: no piece straddles)
      float v[8];
      qn_load8<T>(g + i, v);
      float s8 = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float x = v[k] + (bias ? bias[i + k] : 0.f);
        s8 += x * x;
      }
      if (i < qn) sq += s8; else sk += s8;
    }
    iq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)qn + eps);
    ik = 1.0f / sqrtf(block_sum(sk, scratch) / (float)kn + eps);
  }
  __syncthreads();
  if (slot >= num_slots) {
    if (tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  constexpr int PER = 32 / L;
  const int team = lane / L, e = 8 * (lane % L);
  const int heads = nh + 2 * nkv;
  for (int h0 = warp * PER; h0 < heads; h0 += nwarps * PER) {
    const int h = h0 + team;
    const int kind = h < nh ? 0 : h < nh + nkv ? 1 : 2;          // q, k, v
    const int hl = kind == 0 ? h : kind == 1 ? h - nh : h - nh - nkv;
    const int n = kind == 2 ? vd : hd;
    const int base = kind == 0 ? h * hd : kind == 1 ? qn + hl * hd : qn + kn + hl * vd;
    const bool on = h < heads && e < n;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.f;
    if (on) {
      qn_load8<T>(g + base + e, v);
      if (bias) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] += bias[base + e + k];
      }
      if (kind != 2) {
        if (norm_mode == 2) {
          const float* w = kind == 0 ? qw + (size_t)hl * hd : kw + (size_t)hl * hd;
          const float whole = kind == 0 ? iq : ik;
#pragma unroll
          for (int k = 0; k < 8; ++k) v[k] = v[k] * whole * w[e + k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int pi = (e >> 1) + k;
          if (pi < half) {
            const float c = cs[pi], sv = sn[pi], u = v[2 * k], y = v[2 * k + 1];
            v[2 * k] = u * c - y * sv;
            v[2 * k + 1] = y * c + u * sv;
          }
        }
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
#pragma unroll
    for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!on) continue;
    if (kind == 2 ? value_norm != 0 : norm_mode == 1) {
      const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= inv;
    }
    if (kind == 0) {
      if (mixing) {
#pragma unroll
        for (int k = 0; k < 8; ++k) row[base + e + k] = v[k];
      }
      qn_store8<T>(g + base + e, v, (!mixing && mix_temp) ? mix_temp[h] : 1.0f);
    } else if (slot >= 0) {
      T* dst = (kind == 1 ? k_cache : v_cache) + (((size_t)page * nkv + hl) * page_size + off) * n;
      qn_store8<T>(dst + e, v, 1.0f);
    }
  }
  if (mixing) {
    __syncthreads();
    const int group = nh / nkv, wide = nkv * hd;
    T* dst = qmix + (size_t)t * nh * wide;
    for (int i0 = warp * PER; i0 < nh * nkv; i0 += nwarps * PER) {   // a team a (head, kv head): hd values of the wide query
      const int idx = i0 + team;
      if (idx >= nh * nkv || e >= hd) continue;
      const int h = idx / nkv, c = idx - h * nkv;
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      for (int a = c * group; a < (c + 1) * group; ++a) {
        const float coef = mix[h * nh + a] * (mix_temp ? mix_temp[a] : 1.0f);
        const float4 s0 = *reinterpret_cast<const float4*>(row + (size_t)a * hd + e);
        const float4 s1 = *reinterpret_cast<const float4*>(row + (size_t)a * hd + e + 4);
        acc[0] = fmaf(coef, s0.x, acc[0]), acc[1] = fmaf(coef, s0.y, acc[1]);
        acc[2] = fmaf(coef, s0.z, acc[2]), acc[3] = fmaf(coef, s0.w, acc[3]);
        acc[4] = fmaf(coef, s1.x, acc[4]), acc[5] = fmaf(coef, s1.y, acc[5]);
        acc[6] = fmaf(coef, s1.z, acc[6]), acc[7] = fmaf(coef, s1.w, acc[7]);
      }
      qn_store8<T>(dst + (size_t)h * wide + (size_t)c * hd + e, acc, 1.0f);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
qkv_norm_rotate_store_kernel(T* __restrict__ qkv, long qkv_stride, const float* __restrict__ bias,
                             const int* __restrict__ positions, const float* __restrict__ freq, int rot_dim, float amp,
                             int interleaved, int nh, int nkv, int hd, int vd, int norm_mode,
                             const float* __restrict__ qw, const float* __restrict__ kw, int value_norm, float eps,
                             const int* __restrict__ slot_map, T* __restrict__ k_cache, T* __restrict__ v_cache,
                             int page_size, long num_slots, const float* __restrict__ mix,
                             const float* __restrict__ mix_temp, T* __restrict__ qmix, int* status) {
  extern __shared__ float row[];          // [(nh + nkv) * hd + nkv * vd], then cos and sin [rot_dim / 2] each
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int qn = nh * hd, kn = nkv * hd, vn = nkv * vd, width = qn + kn + vn;
  const int half = rot_dim >> 1;
  float* cs = row + width;
  float* sn = cs + half;
  T* g = qkv + (size_t)t * qkv_stride;
  const float pos = (float)(positions ? positions[t] : 0);
  for (int i = tid; i < half; i += blockDim.x) {
    const float a = pos * freq[i];
    cs[i] = cosf(a) * amp;
    sn[i] = sinf(a) * amp;
  }
  for (int i = tid; i < width; i += blockDim.x) row[i] = to_f32<T>(g[i]) + (bias ? bias[i] : 0.f);
  __syncthreads();
  if (norm_mode == 2) {
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < qn; i += blockDim.x) sq += row[i] * row[i];
    for (int i = tid; i < kn; i += blockDim.x) sk += row[qn + i] * row[qn + i];
    const float iq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)qn + eps);
    const float ik = 1.0f / sqrtf(block_sum(sk, scratch) / (float)kn + eps);
    for (int i = tid; i < qn; i += blockDim.x) row[i] = row[i] * iq * qw[i];
    for (int i = tid; i < kn; i += blockDim.x) row[qn + i] = row[qn + i] * ik * kw[i];
    __syncthreads();
  }
  for (int w = tid; w < (nh + nkv) * half; w += blockDim.x) {
    const int h = w / half, i = w - h * half;
    float* head = row + (size_t)h * hd;
    const int j0 = interleaved ? 2 * i : i;
    const int j1 = interleaved ? 2 * i + 1 : i + half;
    const float u = head[j0], v = head[j1];
    head[j0] = u * cs[i] - v * sn[i];
    head[j1] = v * cs[i] + u * sn[i];
  }
  __syncthreads();
  // unit norms a head: a warp a head (the q and k heads, then the value heads)
  const int unit_qk = norm_mode == 1 ? nh + nkv : 0;
  const int unit_v = value_norm ? nkv : 0;
  for (int h = warp; h < unit_qk + unit_v; h += nwarps) {
    float* head = h < unit_qk ? row + (size_t)h * hd : row + qn + kn + (size_t)(h - unit_qk) * vd;
    const int n = h < unit_qk ? hd : vd;
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s += head[i] * head[i];
    const float inv = 1.0f / sqrtf(warp_sum(s) / (float)n + eps);
    for (int i = lane; i < n; i += 32) head[i] *= inv;
  }
  __syncthreads();
  long slot = slot_map ? (long)slot_map[t] : -1;
  if (slot >= num_slots) {
    if (tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    slot = -1;
  }
  const long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const bool q_scaled = !(mix != nullptr && qmix != nullptr) && mix_temp != nullptr;
  for (int i = tid; i < qn; i += blockDim.x) g[i] = from_f32<T>(q_scaled ? row[i] * mix_temp[i / hd] : row[i]);
  if (mix != nullptr && qmix != nullptr) {
    const int group = nh / nkv, wide = nkv * hd;
    T* dst = qmix + (size_t)t * nh * wide;
    for (int i = tid; i < nh * wide; i += blockDim.x) {
      const int h = i / wide, rem = i - h * wide;
      const int kl = rem / hd, d = rem - kl * hd;
      float s = 0.f;
      for (int a = kl * group; a < (kl + 1) * group; ++a)
        s = fmaf(mix[h * nh + a] * (mix_temp ? mix_temp[a] : 1.0f), row[(size_t)a * hd + d], s);
      dst[i] = from_f32<T>(s);
    }
  }
  if (slot >= 0) {
    for (int i = tid; i < kn; i += blockDim.x) {
      const int h = i / hd, j = i - h * hd;
      k_cache[(((size_t)page * nkv + h) * page_size + off) * hd + j] = from_f32<T>(row[qn + i]);
    }
    for (int i = tid; i < vn; i += blockDim.x) {
      const int h = i / vd, j = i - h * vd;
      v_cache[(((size_t)page * nkv + h) * page_size + off) * vd + j] = from_f32<T>(row[qn + kn + i]);
    }
  }
}

extern "C" int ll_qkv_norm_rotate_store(int dtype, void* qkv, long qkv_stride, const float* bias, const int* positions,
                                        const float* freq, int rot_dim, float amp, int interleaved, int nh, int nkv,
                                        int hd, int vd, int norm_mode, const float* qw, const float* kw, int value_norm,
                                        float eps, const int* slot_map, void* k_cache, void* v_cache, int page_size,
                                        long num_slots, int num_tokens, const float* mix, const float* mix_temp,
                                        void* qmix, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1) || hd <= 0 || vd <= 0 || norm_mode < 0 || norm_mode > 2 ||
      (norm_mode == 2 && (qw == nullptr || kw == nullptr)) || (rot_dim > 0 && freq == nullptr))
    return (int)cudaErrorInvalidValue;
  const size_t piece = dtype == LL_DTYPE_BF16 ? 16 : 32;     // bytes of eight values
  const bool teams = (interleaved || rot_dim == 0) && hd % 8 == 0 && vd % 8 == 0 && hd <= 256 && vd <= 256 &&
                     qkv_stride % 8 == 0 && (uintptr_t)qkv % piece == 0 &&
                     (qmix == nullptr || (uintptr_t)qmix % piece == 0) &&
                     (slot_map == nullptr || ((uintptr_t)k_cache % piece == 0 && (uintptr_t)v_cache % piece == 0));
  if (teams) {
    const size_t smem = sizeof(float) * ((mix != nullptr && qmix != nullptr ? (size_t)nh * hd : 0) + rot_dim);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int most = hd > vd ? hd : vd;
    const int lanes = most <= 64 ? 8 : most <= 128 ? 16 : 32;
    const int warps = ((nh + 2 * nkv) * lanes + 31) / 32;
    const int threads = warps >= 8 ? 256 : warps >= 4 ? 128 : 64;
#define QN_LAUNCH(LANES)                                                                                              \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(qkv_norm_rotate_store_teams_kernel<T, LANES>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                                \
    ll_launch(qkv_norm_rotate_store_teams_kernel<T, LANES>, dim3(num_tokens), dim3(threads), smem, stream, (T*)qkv,   \
              qkv_stride, bias, positions, freq, rot_dim, amp, nh, nkv, hd, vd, norm_mode, qw, kw, value_norm, eps,   \
              slot_map, (T*)k_cache, (T*)v_cache, page_size, num_slots, mix, mix_temp, (T*)qmix, status);             \
  } while (0)
    LL_DISPATCH_DTYPE(dtype, {
      if (lanes == 8) QN_LAUNCH(8);
      else if (lanes == 16) QN_LAUNCH(16);
      else QN_LAUNCH(32);
    });
#undef QN_LAUNCH
    return LL_LAUNCH_RESULT();
  }
  const size_t smem = sizeof(float) * ((size_t)(nh + nkv) * hd + (size_t)nkv * vd + rot_dim);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(qkv_norm_rotate_store_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(qkv_norm_rotate_store_kernel<T>, dim3(num_tokens), dim3(256), smem, stream, (T*)qkv, qkv_stride, bias,
              positions, freq, rot_dim, amp, interleaved, nh, nkv, hd, vd, norm_mode, qw, kw, value_norm, eps, slot_map,
              (T*)k_cache, (T*)v_cache, page_size, num_slots, mix, mix_temp, (T*)qmix, status);
  });
  return LL_LAUNCH_RESULT();
}
