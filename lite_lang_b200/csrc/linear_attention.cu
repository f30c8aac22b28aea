// Linear attention with a decay per head ("lightning attention"): a matrix state per head and request,
//     S_t = d_h * S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,
// with q, k (heads x dk) and v (heads x dv) = SiLU of the projections (`silu_rows`, once a step, in place: every
// block of the scan reads a head's q and k again, so the activation is not left to it).  The state is float32 and lives in
// the request's record [heads][dv][dk] (a value column's key channels side by side); everything here but the
// projections' storage is float32.
//
// `decay_scan`: one block per (entry, head, 8 value columns).  Every value column of S evolves on its own, so
// the scan is spread over them; a column's dk channels are held in registers by 16 lanes (lane l holds the
// channels 64 j + 4 l + i, i < 4: a float4 of shared memory a step).  The entry's tokens are walked in order, 16
// at a time: the next 16 tokens' rows are asked for (16-byte loads, all in flight at once) before the current 16
// are worked on, and go into shared memory as float32 afterwards.  The only chain from token to token is one
// multiply-add a channel; the read-outs' sums over the lanes are taken for 16 tokens together (a halving
// exchange: 15 shuffles instead of 64).  A token's arithmetic does not depend on where a step's portion began
// (the exchange adds the same pairs whatever the token's place among the 16), so a position's result is the
// same bits however the tokens were cut into steps.
//
// The same scan serves a state-space layer whose decay and step size differ from token to token
// (S_t = a_t,h S_(t-1) + dt_t,h k_t v_t^T, o_t = S_t^T q_t + D_h v_t, q and k shared by the `hpg` heads of a
// group): `tok_decay` and `tok_scale` [tokens, H] replace the constant decay and scale the written values,
// `skip` [H] adds the token's own value to its read-out.
//
// `linear_attn_out`: y = o / rms(o over all heads) * weight * sigmoid(gate), in the engine's dtype.
#include "common.cuh"

#define LA_COLS 8
#define LA_LANES 16
#define LA_THREADS (LA_COLS * LA_LANES)
#define LA_CHUNK 16

__device__ __forceinline__ float la_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T> struct LaVec;
template <> struct LaVec<float> {
  static constexpr int N = 4;
  __device__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
};
template <> struct LaVec<bf16> {
  static constexpr int N = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
};

// proj: T [tokens, stride]: q heads at q_off, k heads at k_off (dk each), v heads at v_off (dv each), activated.
// state: float32 [slots][H][dv][dk]; o: float32 [tokens, H * dv].  R = channels a lane: 4, 8 or 16 (dk <= 16 R).
// VEC: rows are read in 16-byte pieces (the launcher checked sizes and alignment).
template <typename T, int R, bool VEC>
__global__ void __launch_bounds__(LA_THREADS)
decay_scan_kernel(const T* __restrict__ proj, long stride, int q_off, int k_off, int v_off,
                  const float* __restrict__ decay, float* __restrict__ state, long slot_stride, int num_slots,
                  const int* __restrict__ cu_q, const int* __restrict__ req_slot, float* __restrict__ o, int H, int dk,
                  int dv, int write_state, int* status, int hpg, const float* __restrict__ tok_decay,
                  const float* __restrict__ tok_scale, const float* __restrict__ skip) {
  constexpr int DKP = R * LA_LANES;
  constexpr int VN = LaVec<T>::N;
  constexpr int ROWV = DKP / VN;                                      // 16-byte pieces of a (padded) q or k row
  constexpr int NV = (2 * LA_CHUNK * ROWV + LA_THREADS - 1) / LA_THREADS;   // pieces a thread brings a chunk
  __shared__ __align__(16) float qs[LA_CHUNK * DKP];
  __shared__ __align__(16) float ks[LA_CHUNK * DKP];
  __shared__ float vs[LA_CHUNK * LA_COLS];
  __shared__ float ds[LA_CHUNK], ws[LA_CHUNK];     // a token's decay and the factor on what it writes
  LL_PDL_TRIGGER();
  const int cg = blockIdx.x, h = blockIdx.y, e = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & (LA_LANES - 1), cl = tid / LA_LANES;
  const int col = cg * LA_COLS + cl;
  const float d_head = decay ? decay[h] : 1.f;
  const float skip_h = skip ? skip[h] : 0.f;
  const int hq = h / hpg;                        // the head whose q and k this head reads
  LL_PDL_WAIT();
  const int t0 = cu_q[e], t1 = cu_q[e + 1];
  const int slot = req_slot[e];
  if (slot < 0 || slot >= num_slots) {       // a padding entry: defined output, nothing read
    if (slot >= num_slots && tid == 0) set_status(status, LL_ERR_SLOT_RANGE);
    if (lane == 0 && col < dv)
      for (int t = t0; t < t1; ++t) o[(size_t)t * H * dv + (size_t)h * dv + col] = 0.f;
    return;
  }
  float* srow = state + (size_t)slot * slot_stride + ((size_t)h * dv + (col < dv ? col : 0)) * dk;
  const bool svec = (dk & 3) == 0 && (slot_stride & 3) == 0;
  float S[R];
#pragma unroll
  for (int j = 0; j < R / 4; ++j) {
    const int c = 64 * j + 4 * lane;
    if (svec && col < dv && c < dk) {
      const float4 v4 = *reinterpret_cast<const float4*>(srow + c);
      S[4 * j] = v4.x; S[4 * j + 1] = v4.y; S[4 * j + 2] = v4.z; S[4 * j + 3] = v4.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) S[4 * j + i] = (col < dv && c + i < dk) ? srow[c + i] : 0.f;
    }
  }

  // ---- staging: ask for a chunk's rows (registers), later put them into shared memory as float32 ----
  uint4 raw[VEC ? NV : 1];
  float vraw = 0.f, draw = 1.f, wraw = 1.f;
  auto ask = [&](int base) {
    const int n = min(LA_CHUNK, t1 - base);
    if (VEC) {
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        const int p = tid + u * LA_THREADS;              // piece: (q or k, token, piece of the row)
        const int which = p / (LA_CHUNK * ROWV), rem = p - which * (LA_CHUNK * ROWV);
        const int t = rem / ROWV, c = (rem - t * ROWV) * VN;
        raw[u] = make_uint4(0, 0, 0, 0);
        if (which < 2 && t < n && c < dk)
          raw[u] = *reinterpret_cast<const uint4*>(proj + (size_t)(base + t) * stride + (which ? k_off : q_off) + hq * dk + c);
      }
    }
    const int t = tid / LA_COLS, c = cg * LA_COLS + (tid - t * LA_COLS);
    vraw = (t < n && c < dv) ? to_f32<T>(proj[(size_t)(base + t) * stride + v_off + h * dv + c]) : 0.f;
    if (tid < LA_CHUNK) {
      draw = (tok_decay && tid < n) ? tok_decay[(size_t)(base + tid) * H + h] : d_head;
      wraw = (tok_scale && tid < n) ? tok_scale[(size_t)(base + tid) * H + h] : 1.f;
    }
  };
  auto put = [&](int base) {
    const int n = min(LA_CHUNK, t1 - base);
    if (VEC) {
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        const int p = tid + u * LA_THREADS;
        const int which = p / (LA_CHUNK * ROWV), rem = p - which * (LA_CHUNK * ROWV);
        if (which < 2) {
          float f[VN];
          LaVec<T>::unpack(raw[u], f);
          const int t = rem / ROWV, c = (rem - t * ROWV) * VN;
          float* dst = (which ? ks : qs) + rem * VN;
#pragma unroll
          for (int i = 0; i < VN; ++i) f[i] = (t < n && c + i < dk) ? f[i] : 0.f;
#pragma unroll
          for (int i = 0; i < VN; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        }
      }
    } else {
      for (int i = tid; i < LA_CHUNK * DKP; i += LA_THREADS) {
        const int t = i / DKP, c = i - t * DKP;
        const bool in = t < n && c < dk;
        const T* row = proj + (size_t)(base + (in ? t : 0)) * stride;
        qs[i] = in ? to_f32<T>(row[q_off + hq * dk + c]) : 0.f;
        ks[i] = in ? to_f32<T>(row[k_off + hq * dk + c]) : 0.f;
      }
    }
    vs[tid] = vraw;
    if (tid < LA_CHUNK) {
      ds[tid] = draw;
      ws[tid] = wraw;
    }
  };

  if (t0 < t1) ask(t0);
  for (int base = t0; base < t1; base += LA_CHUNK) {
    const int n = min(LA_CHUNK, t1 - base);
    __syncthreads();                      // the chunk before has been read
    put(base);
    __syncthreads();
    if (base + LA_CHUNK < t1) ask(base + LA_CHUNK);      // in flight while this chunk is worked on
    float part[LA_CHUNK];
#pragma unroll
    for (int t = 0; t < LA_CHUNK; ++t) {
      part[t] = 0.f;
      if (t < n) {
        const float v0 = vs[t * LA_COLS + cl];
        const float v = v0 * ws[t];
        const float d = ds[t];
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int j = 0; j < R / 4; ++j) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + t * DKP + 64 * j + 4 * lane);
          const float4 k4 = *reinterpret_cast<const float4*>(ks + t * DKP + 64 * j + 4 * lane);
          S[4 * j] = fmaf(d, S[4 * j], k4.x * v);
          S[4 * j + 1] = fmaf(d, S[4 * j + 1], k4.y * v);
          S[4 * j + 2] = fmaf(d, S[4 * j + 2], k4.z * v);
          S[4 * j + 3] = fmaf(d, S[4 * j + 3], k4.w * v);
          a0 = fmaf(S[4 * j], q4.x, a0);
          a1 = fmaf(S[4 * j + 1], q4.y, a1);
          a2 = fmaf(S[4 * j + 2], q4.z, a2);
          a3 = fmaf(S[4 * j + 3], q4.w, a3);
        }
        part[t] = (a0 + a1) + (a2 + a3);
        if (lane == 0) part[t] = fmaf(skip_h, v0, part[t]);      // (one lane of the column: the exchange sums the lanes)
      }
    }
    // sums over the 16 lanes of a column for the 16 tokens at once: after the exchange lane l holds token l's
#pragma unroll
    for (int w = LA_CHUNK / 2; w >= 1; w >>= 1) {
      const bool upper = (lane & w) != 0;
#pragma unroll
      for (int i = 0; i < w; ++i) {
        const float give = upper ? part[i] : part[i + w];
        const float keep = upper ? part[i + w] : part[i];
        part[i] = keep + __shfl_xor_sync(0xffffffffu, give, w);
      }
    }
    if (lane < n && col < dv) o[(size_t)(base + lane) * H * dv + (size_t)h * dv + col] = part[0];
  }
  if (write_state && col < dv) {
#pragma unroll
    for (int j = 0; j < R / 4; ++j) {
      const int c = 64 * j + 4 * lane;
      if (svec && c < dk) {
        *reinterpret_cast<float4*>(srow + c) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (c + i < dk) srow[c + i] = S[4 * j + i];
      }
    }
  }
}

// x[t, 0:width] <- silu(x[t, 0:width]) in place (float32 arithmetic, one rounding); VEC numbers a thread.
template <typename T, int VEC>
__global__ void silu_rows_kernel(T* __restrict__ x, long stride, long total_vec, int width) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int per_row = width / VEC;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec; idx += step) {
    const long t = idx / per_row;
    T* p = x + t * stride + (idx - t * per_row) * VEC;
    T v[VEC];
    if (VEC > 1) *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(p);
    else v[0] = p[0];
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = from_f32<T>(la_silu(to_f32<T>(v[k])));
    if (VEC > 1) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(v);
    else p[0] = v[0];
  }
}

extern "C" int ll_silu_rows(int dtype, void* x, long stride, int num_tokens, int width, int sms, cudaStream_t stream) {
  if (num_tokens <= 0 || width <= 0) return 0;
  const long most = (long)(sms > 0 ? sms : 148) * 16;
  LL_DISPATCH_DTYPE(dtype, {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = (width % VEC) == 0 && (stride % VEC) == 0 && ((uintptr_t)x % 16) == 0;
    const long total = (long)num_tokens * (wide ? width / VEC : width);
    const long want = (total + 255) / 256;
    const int blocks = (int)(want < most ? want : most);
    if (wide) ll_launch(silu_rows_kernel<T, VEC>, dim3(blocks), dim3(256), 0, stream, (T*)x, stride, total, width);
    else ll_launch(silu_rows_kernel<T, 1>, dim3(blocks), dim3(256), 0, stream, (T*)x, stride, total, width);
  });
  return LL_LAUNCH_RESULT();
}

// y[t, :] = o[t, :] / sqrt(mean(o[t, :]^2) + eps) * weight * sigmoid(gate[t, :]); one block per token.
// VEC = 4: four numbers an access, and rows of up to 256 x 4 x LO_PIECES numbers stay in registers between the sum
// of squares and the output (longer rows are read again).
#define LO_PIECES 4
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
linear_attn_out_kernel(T* __restrict__ y, const float* __restrict__ o, const float* __restrict__ weight,
                       const T* __restrict__ gate, long gate_stride, float eps, int width) {
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * width;
  const T* g = gate + (size_t)t * gate_stride;
  const bool resident = width <= 256 * VEC * LO_PIECES;
  float x[LO_PIECES][VEC];
  float ss = 0.f;
  auto load = [&](int c, float* v) {
    if (VEC == 4) {
      const float4 q = *reinterpret_cast<const float4*>(orow + c);
      v[0] = q.x; v[1 % VEC] = q.y; v[2 % VEC] = q.z; v[3 % VEC] = q.w;
    } else {
      v[0] = orow[c];
    }
  };
  auto store = [&](int c, const float* v, float inv) {
    T gv[VEC], out[VEC];
    float w[VEC];
    if (VEC == 4) {
      if (sizeof(T) == 2) *reinterpret_cast<uint2*>(gv) = *reinterpret_cast<const uint2*>(g + c);
      else *reinterpret_cast<uint4*>(gv) = *reinterpret_cast<const uint4*>(g + c);
      const float4 q = *reinterpret_cast<const float4*>(weight + c);
      w[0] = q.x; w[1 % VEC] = q.y; w[2 % VEC] = q.z; w[3 % VEC] = q.w;
    } else {
      gv[0] = g[c];
      w[0] = weight[c];
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) out[k] = from_f32<T>(v[k] * inv * w[k] / (1.0f + expf(-to_f32<T>(gv[k]))));
    if (VEC == 4 && sizeof(T) == 2) *reinterpret_cast<uint2*>(y + (size_t)t * width + c) = *reinterpret_cast<const uint2*>(out);
    else if (VEC == 4) *reinterpret_cast<uint4*>(y + (size_t)t * width + c) = *reinterpret_cast<const uint4*>(out);
    else y[(size_t)t * width + c] = out[0];
  };
  if (resident) {
#pragma unroll
    for (int p = 0; p < LO_PIECES; ++p) {
      const int c = (threadIdx.x + p * 256) * VEC;
      if (c < width) {
        load(c, x[p]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss = fmaf(x[p][k], x[p][k], ss);
      }
    }
  } else {
    for (int c = threadIdx.x * VEC; c < width; c += 256 * VEC) {
      load(c, x[0]);
#pragma unroll
      for (int k = 0; k < VEC; ++k) ss = fmaf(x[0][k], x[0][k], ss);
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  if (resident) {
#pragma unroll
    for (int p = 0; p < LO_PIECES; ++p) {
      const int c = (threadIdx.x + p * 256) * VEC;
      if (c < width) store(c, x[p], inv);
    }
  } else {
    for (int c = threadIdx.x * VEC; c < width; c += 256 * VEC) {
      load(c, x[0]);
      store(c, x[0], inv);
    }
  }
}

extern "C" int ll_decay_scan(int dtype, const void* proj, long stride, int q_off, int k_off, int v_off,
                             const float* decay, float* state, long slot_stride, int num_slots, const int* cu_q,
                             const int* req_slot, float* o, int num_entries, int H, int dk, int dv, int write_state,
                             int* status, int hpg, const float* tok_decay, const float* tok_scale, const float* skip,
                             cudaStream_t stream) {
  if (num_entries <= 0) return 0;
  if (H <= 0 || dk <= 0 || dk > 256 || dv <= 0 || hpg <= 0 || H % hpg != 0 || (decay == nullptr && tok_decay == nullptr))
    return (int)cudaErrorInvalidValue;
  const int need = (dk + LA_LANES - 1) / LA_LANES;
  const int R = need <= 4 ? 4 : need <= 8 ? 8 : 16;
  dim3 grid((dv + LA_COLS - 1) / LA_COLS, H, num_entries);
  const int esz = dtype == LL_DTYPE_F32 ? 4 : 2, ve = 16 / esz;
  const bool vec = ((uintptr_t)proj % 16) == 0 && (stride % ve) == 0 && (q_off % ve) == 0 && (k_off % ve) == 0 &&
                   (dk % ve) == 0;
#define LA_LAUNCH(RR, VV)                                                                                          \
  ll_launch(decay_scan_kernel<T, RR, VV>, grid, dim3(LA_THREADS), 0, stream, (const T*)proj, stride, q_off, k_off, \
            v_off, decay, state, slot_stride, num_slots, cu_q, req_slot, o, H, dk, dv, write_state, status, hpg,   \
            tok_decay, tok_scale, skip)
  LL_DISPATCH_DTYPE(dtype, {
    if (vec) {
      if (R == 4) LA_LAUNCH(4, true);
      else if (R == 8) LA_LAUNCH(8, true);
      else LA_LAUNCH(16, true);
    } else {
      if (R == 4) LA_LAUNCH(4, false);
      else if (R == 8) LA_LAUNCH(8, false);
      else LA_LAUNCH(16, false);
    }
  });
#undef LA_LAUNCH
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_linear_attn_out(int dtype, void* y, const float* o, const float* weight, const void* gate,
                                  long gate_stride, float eps, int num_tokens, int width, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const bool wide = (width % 4) == 0 && (gate_stride % 4) == 0 && ((uintptr_t)o % 16) == 0 &&
                    ((uintptr_t)weight % 16) == 0 && ((uintptr_t)gate % 16) == 0 && ((uintptr_t)y % 16) == 0;
  LL_DISPATCH_DTYPE(dtype, {
    if (wide)
      ll_launch(linear_attn_out_kernel<T, 4>, dim3(num_tokens), dim3(256), 0, stream, (T*)y, o, weight, (const T*)gate,
                gate_stride, eps, width);
    else
      ll_launch(linear_attn_out_kernel<T, 1>, dim3(num_tokens), dim3(256), 0, stream, (T*)y, o, weight, (const T*)gate,
                gate_stride, eps, width);
  });
  return LL_LAUNCH_RESULT();
}
