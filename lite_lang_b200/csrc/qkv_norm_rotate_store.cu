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
// Cache plane: K [num_pages, nkv, page_size, hd], V [num_pages, nkv, page_size, vd].
#include "common.cuh"

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
  for (int i = tid; i < qn; i += blockDim.x) g[i] = from_f32<T>(row[i]);
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
