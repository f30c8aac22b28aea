// State-space layer with a scalar decay a head and token (the "state-space duality" form of a selective scan):
// the pieces around the scan.  One product gives, a token, [z | x | B | C | dt]: the gate's input (inner = heads x
// P numbers), the values x (inner), the write and read vectors B and C of `groups` groups (N numbers each) and a
// step size a head.  Then
//   [x | B | C] <- silu(conv(x | B | C))      a causal convolution a channel over the last `taps` inputs (weights
//                                             [channels, taps], the last for the token itself, and a bias); the
//                                             inputs before a request's first token are zeros
//   dt_h = softplus(dt_h + dt_bias_h),  a_h = exp(-exp(A_log_h) dt_h)
//   S_h <- a_h S_h + dt_h B_g x_h^T,    y_h = S_h^T C_g + D_h x_h            (the scan: `decay_scan`)
//   y <- y silu(z);  every one of `norm_groups` equal parts of y divided by its root mean square, times a weight
// A request's record (float32) holds S [heads][P][N] and, behind it, the convolution's last taps - 1 inputs
// [taps - 1][channels], oldest first.
//
//   ssd_prepare      per token: convolution + SiLU into float32 [tokens, channels]; dt and a into [tokens, heads]
//   ssd_conv_update  per entry: the record's last taps - 1 inputs after the step's portion
//   ssd_gated_norm   per (token, part): gate, norm, weight -> storage type
// All three read the step's device arrays only, so a step of single tokens can be captured and replayed.  The
// convolution adds its taps from the oldest to the newest whatever the token's place in a portion, so a
// position's numbers do not depend on how the tokens were cut into steps.
#include "common.cuh"

__device__ __forceinline__ float ssd_silu(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float ssd_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// proj row t: the convolution's channels at x_off (C wide), the step sizes' inputs at dt_off (H wide).
// conv_w float32 [C, taps], conv_b float32 [C] (or null).  state: float32 records, the tail at tail_off.
template <typename T>
__global__ void __launch_bounds__(256)
ssd_prepare_kernel(const T* __restrict__ proj, long proj_stride, int x_off, int dt_off,
                   const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                   const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                   const float* __restrict__ state, long state_stride, long tail_off, int num_slots,
                   const int* __restrict__ token_req, const int* __restrict__ cu_q, const int* __restrict__ req_slot,
                   float* __restrict__ xbc, float* __restrict__ dt_out, float* __restrict__ decay_out, int C, int H,
                   int taps, int* status) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const int e = token_req[t];
  const int slot = e >= 0 ? req_slot[e] : -1;
  if (slot < 0) return;   // padding entry: the scan writes its (zero) output
  if (slot >= num_slots) {
    if (threadIdx.x == 0) set_status(status, LL_ERR_SLOT_RANGE);
    return;
  }
  const int i = t - cu_q[e];                     // the token's place in its entry's portion
  const float* tail = state + (size_t)slot * state_stride + tail_off;
  // (the channels are shared out over gridDim.y blocks a token: with few tokens a block a token would leave the
  // device to a handful of blocks, each a chain of its channels' loads)
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;             // tap j weighs the input `back` positions before the token
      float x;
      if (back <= i) x = to_f32<T>(proj[(size_t)(t - back) * proj_stride + x_off + c]);
      else x = tail[(size_t)(taps - 1 + i - back) * C + c];
      acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
    }
    xbc[(size_t)t * C + c] = ssd_silu(acc);
  }
  if (blockIdx.y != 0) return;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = ssd_softplus(to_f32<T>(proj[(size_t)t * proj_stride + dt_off + h]) + dt_bias[h]);
    dt_out[(size_t)t * H + h] = dt;
    decay_out[(size_t)t * H + h] = expf(-expf(A_log[h]) * dt);
  }
}

// After a step the record's places 0 .. taps-2 hold the inputs of the last taps - 1 positions, oldest first: the
// step's own rows where the portion reaches back that far, else what the record held, moved up.  A thread owns a
// channel and goes from the oldest place to the newest, reading only places above the one it writes.
template <typename T>
__global__ void ssd_conv_update_kernel(const T* __restrict__ proj, long proj_stride, int x_off,
                                       float* __restrict__ state, long state_stride, long tail_off, int num_slots,
                                       const int* __restrict__ cu_q, const int* __restrict__ req_slot, int C,
                                       int taps) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int e = blockIdx.x;
  const int slot = req_slot[e];
  if (slot < 0 || slot >= num_slots) return;
  const int first = cu_q[e], L = cu_q[e + 1] - first;
  if (L <= 0) return;
  float* tail = state + (size_t)slot * state_stride + tail_off;
  const int K1 = taps - 1;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
    for (int i = 0; i < K1; ++i) {
      const int src = i + L;                     // place among (old tail, then the portion's rows) that moves to i
      float x;
      if (src >= K1) x = to_f32<T>(proj[(size_t)(first + src - K1) * proj_stride + x_off + c]);
      else x = tail[(size_t)src * C + c];
      tail[(size_t)i * C + c] = x;
    }
  }
}

// out[t, part] = u / sqrt(mean(u^2) + eps) * weight with u = y[t, part] * silu(z[t, part]); one block per
// (token, part), the part's numbers held in registers between the two passes where they fit.
#define SSD_NORM_PIECES 8
template <typename T>
__global__ void __launch_bounds__(128)
ssd_gated_norm_kernel(T* __restrict__ out, long out_stride, const float* __restrict__ y, const T* __restrict__ z,
                      long z_stride, const float* __restrict__ weight, float eps, int width, int parts) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x, part = blockIdx.y;
  const int w = width / parts, c0 = part * w;
  const float* yr = y + (size_t)t * width + c0;
  const T* zr = z + (size_t)t * z_stride + c0;
  const bool resident = w <= 128 * SSD_NORM_PIECES;
  float u[SSD_NORM_PIECES];
  float ss = 0.f;
  if (resident) {
#pragma unroll
    for (int p = 0; p < SSD_NORM_PIECES; ++p) {
      const int c = threadIdx.x + p * 128;
      u[p] = c < w ? yr[c] * ssd_silu(to_f32<T>(zr[c])) : 0.f;
      ss = fmaf(u[p], u[p], ss);
    }
  } else {
    for (int c = threadIdx.x; c < w; c += 128) {
      const float v = yr[c] * ssd_silu(to_f32<T>(zr[c]));
      ss = fmaf(v, v, ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)w + eps);
  T* o = out + (size_t)t * out_stride + c0;
  if (resident) {
#pragma unroll
    for (int p = 0; p < SSD_NORM_PIECES; ++p) {
      const int c = threadIdx.x + p * 128;
      if (c < w) o[c] = from_f32<T>(u[p] * inv * weight[c0 + c]);
    }
  } else {
    for (int c = threadIdx.x; c < w; c += 128)
      o[c] = from_f32<T>(yr[c] * ssd_silu(to_f32<T>(zr[c])) * inv * weight[c0 + c]);
  }
}

// state: float32 [num_slots, state_stride]; xbc float32 [tokens, C]; dt_out, decay_out float32 [tokens, H].
// Two launches: the convolution of every token, then (taps > 1 and write_state) the records' new tails.
extern "C" int ll_ssd_prepare(int dtype, const void* proj, long proj_stride, int x_off, int dt_off,
                              const float* conv_w, const float* conv_b, const float* A_log, const float* dt_bias,
                              float* state, long state_stride, long tail_off, int num_slots, const int* token_req,
                              const int* cu_q, const int* req_slot, float* xbc, float* dt_out, float* decay_out,
                              int num_tokens, int num_entries, int C, int H, int taps, int write_state, int* status,
                              cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (C <= 0 || H <= 0 || taps < 1) return (int)cudaErrorInvalidValue;
  // blocks a token: as many as give a few hundred blocks in all, at most one a 256 channels
  int by = (C + 255) / 256;
  const int want = (296 + num_tokens - 1) / num_tokens;
  by = by < want ? by : want;
  LL_DISPATCH_DTYPE(dtype, {
    ll_launch(ssd_prepare_kernel<T>, dim3(num_tokens, by), dim3(256), 0, stream, (const T*)proj, proj_stride, x_off, dt_off,
              conv_w, conv_b, A_log, dt_bias, (const float*)state, state_stride, tail_off, num_slots, token_req, cu_q,
              req_slot, xbc, dt_out, decay_out, C, H, taps, status);
    if (taps > 1 && write_state) {
      const int bu = (C + 255) / 256;
      ll_launch(ssd_conv_update_kernel<T>, dim3(num_entries, bu < 8 ? bu : 8), dim3(256), 0, stream, (const T*)proj,
                proj_stride, x_off, state, state_stride, tail_off, num_slots, cu_q, req_slot, C, taps);
    }
  });
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_ssd_gated_norm(int dtype, void* out, long out_stride, const float* y, const void* z, long z_stride,
                                 const float* weight, float eps, int num_tokens, int width, int parts,
                                 cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (width <= 0 || parts <= 0 || width % parts != 0) return (int)cudaErrorInvalidValue;
  LL_DISPATCH_DTYPE(dtype, ll_launch(ssd_gated_norm_kernel<T>, dim3(num_tokens, parts), dim3(128), 0, stream, (T*)out,
                                     out_stride, y, (const T*)z, z_stride, weight, eps, width, parts));
  return LL_LAUNCH_RESULT();
}
