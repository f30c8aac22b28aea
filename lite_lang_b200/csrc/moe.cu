// Routed feed-forward (mixture of experts): the router and the activation between the two products.
//
// Router, per token, all in float32: logits z = Wr x over the experts, scores by softmax (or sigmoid) over
// all experts, the `top` experts with the largest scores (ties: the lower index), their weights the scores
// themselves or the scores divided by their sum.  The result is a dense row of weights per token, zero for
// experts that were not chosen, plus the chosen indices and weights.
//
// The experts' first products run as one product over all experts' rows (an always-on expert's rows first);
// `moe_act` then applies the activation and multiplies every hidden unit by the weight of its expert for that
// token (1 for the always-on rows, 0 for experts not chosen), so that one second product over all hidden units
// gives the weighted sum of the chosen experts' outputs plus the always-on expert's.
#include "common.cuh"

#define MOE_MAX_E 256

// Wr: float32 [E, hidden]; x: T [tokens, hidden]; gates: float32 [tokens, E]; top_idx int32 / top_w float32
// [tokens, top].  score_fn: 0 softmax over all experts, 1 sigmoid, 2 the `top` largest logits are chosen and
// their weights are a softmax taken over just those logits.  `bias` (float32 [E], optional) is added to the
// logits.  With `shared_w` (float32 [tokens]) the router matrix has one more row, the gate of an expert that
// every token uses: shared_w[t] = sigmoid(Wr[E] . x).  One block per token: its eight warps share out the experts
// (the token's row waits in shared memory as float32), then the first warp scores and picks.
#define MOE_ROUTER_THREADS 256
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTER_THREADS)
moe_router_kernel(const T* __restrict__ x, long x_stride, const float* __restrict__ Wr, const float* __restrict__ bias,
                  float* __restrict__ gates, int* __restrict__ top_idx, float* __restrict__ top_w,
                  float* __restrict__ shared_w, int num_tokens, int hidden, int E, int top, int score_fn,
                  int renormalize) {
  __shared__ float z[MOE_MAX_E + 2];
  extern __shared__ __align__(16) float xrow[];          // the token's row as float32 [hidden]
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * x_stride;
  for (int i = threadIdx.x; i < hidden; i += MOE_ROUTER_THREADS) xrow[i] = to_f32<T>(xr[i]);
  __syncthreads();
  const int n_rows = E + (shared_w ? 1 : 0);
  // a warp a row: a lane sums its pieces of four numbers (four sums side by side), then the lanes are added up:
  // an order that depends on the sizes only
  const bool vec = (hidden & 3) == 0;
  for (int e = warp; e < n_rows; e += MOE_ROUTER_THREADS / 32) {
    const float* wrow = Wr + (size_t)e * hidden;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (vec) {
#pragma unroll 4
      for (int i = 4 * lane; i < hidden; i += 128) {
        const float4 w4 = *reinterpret_cast<const float4*>(wrow + i);
        const float4 x4 = *reinterpret_cast<const float4*>(xrow + i);
        a0 = fmaf(w4.x, x4.x, a0);
        a1 = fmaf(w4.y, x4.y, a1);
        a2 = fmaf(w4.z, x4.z, a2);
        a3 = fmaf(w4.w, x4.w, a3);
      }
    } else {
#pragma unroll 4
      for (int i = lane; i < hidden; i += 32) a0 = fmaf(wrow[i], xrow[i], a0);
    }
    const float a = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) z[e] = a + ((bias && e < E) ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  if (shared_w && lane == 0) shared_w[t] = 1.0f / (1.0f + expf(-z[E]));
  if (score_fn == 2) {
    // the logits themselves are compared; the weights are made from the chosen ones below
  } else if (score_fn == 0) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - m) / sum;
  } else {
    for (int e = lane; e < E; e += 32) z[e] = 1.0f / (1.0f + expf(-z[e]));
  }
  __syncwarp();
  float* gr = gates + (size_t)t * E;
  for (int e = lane; e < E; e += 32) gr[e] = 0.f;
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int arg = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) {   // (a lane walks upwards, so it keeps its lowest index among equals)
        best = v;
        arg = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    if (arg >= E) break;
    if (lane == 0) {
      top_idx[(size_t)t * top + k] = arg;
      top_w[(size_t)t * top + k] = best;
      gr[arg] = best;
      z[arg] = -INFINITY;
    }
    total += best;
    __syncwarp();
  }
  if (score_fn == 2) {
    // softmax over the chosen logits (the first chosen is the largest), summed in the order they were chosen
    __syncwarp();
    const float m = top_w[(size_t)t * top];
    float sum = 0.f;
    for (int k = 0; k < top; ++k) sum += expf(top_w[(size_t)t * top + k] - m);
    __syncwarp();
    for (int k = lane; k < top; k += 32) {
      const float w = expf(top_w[(size_t)t * top + k] - m) / sum;
      top_w[(size_t)t * top + k] = w;
      gr[top_idx[(size_t)t * top + k]] = w;
    }
    return;
  }
  if (renormalize && total > 0.f) {
    __syncwarp();
    for (int e = lane; e < E; e += 32) gr[e] = gr[e] / total;
    for (int k = lane; k < top; k += 32) top_w[(size_t)t * top + k] /= total;
  }
}

// act: 0 relu(z)^2, 1 silu(z), 2 gelu_tanh(z), 3 gelu(z) (the erf form).
__device__ __forceinline__ float moe_activation(float z, int act) {
  if (act == 0) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  if (act == 1) return z / (1.0f + expf(-z));
  if (act == 3) return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
// The expert's weight w for the token goes onto the activation's output, act(z) w, or (MOE_ACT_WEIGHT_IN set in
// `act`) onto its input, act(w z): the expert then works on w times the token's row, since U (w x) = w (U x).
#define MOE_ACT_WEIGHT_IN 16
__device__ __forceinline__ float moe_weighted_activation(float z, float w, int act) {
  return (act & MOE_ACT_WEIGHT_IN) ? moe_activation(z * w, act & 15) : moe_activation(z, act) * w;
}

// h: T [tokens, shared_ff + E * ff] in place: h = act(h) * weight, weight 1 for the first shared_ff columns,
// gates[t, (col - shared_ff) / ff] for the rest.  A thread takes VEC neighbouring columns of a row (one 16-byte
// access where the row's width allows it).
template <typename T, int VEC>
__global__ void moe_act_kernel(T* __restrict__ h, const float* __restrict__ gates, int num_tokens, int width,
                               int shared_ff, int ff, int E, int act) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int per_row = (width + VEC - 1) / VEC;
  const long total = (long)num_tokens * per_row;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const int t = (int)(idx / per_row);
    const int c0 = (int)(idx - (long)t * per_row) * VEC;
    T* p = h + (size_t)t * width + c0;
    T v[VEC];
    if (VEC > 1) {
      // the piece lies inside one expert (the launcher checked the widths): if that expert was not chosen for
      // the token, zeros are written and nothing is read
      if (c0 >= shared_ff && gates[(size_t)t * E + (c0 - shared_ff) / ff] == 0.f) {
        *reinterpret_cast<uint4*>(p) = make_uint4(0, 0, 0, 0);
        continue;
      }
      *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(p);
    } else {
      v[0] = p[0];
    }
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      const int c = c0 + u;
      const float w = c < shared_ff ? 1.f : gates[(size_t)t * E + (c - shared_ff) / ff];
      // an expert that was not chosen contributes an exact zero whatever its first product gave
      v[u] = from_f32<T>(w == 0.f ? 0.f : moe_weighted_activation(to_f32<T>(v[u]), w, act));
    }
    if (VEC > 1) {
      *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(v);
    } else {
      p[0] = v[0];
    }
  }
}

extern "C" int ll_moe_router(int dtype, const void* x, long x_stride, const float* Wr, const float* bias, float* gates,
                             int* top_idx, float* top_w, float* shared_w, int num_tokens, int hidden, int E, int top,
                             int score_fn, int renormalize, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_E || top <= 0 || top > E || hidden <= 0) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (size_t)((hidden + 3) / 4 * 4);
  if (smem > 40 * 1024) return (int)cudaErrorInvalidValue;      // (rows of up to 10,240 numbers)
  LL_DISPATCH_DTYPE(dtype, ll_launch(moe_router_kernel<T>, dim3(num_tokens), dim3(MOE_ROUTER_THREADS), smem, stream,
                                     (const T*)x, x_stride, Wr, bias, gates, top_idx, top_w, shared_w, num_tokens,
                                     hidden, E, top, score_fn, renormalize));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_moe_act(int dtype, void* h, const float* gates, int num_tokens, int shared_ff, int ff, int E, int act,
                          int sms, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int width = shared_ff + E * ff;
  if (width <= 0 || (E > 0 && ff <= 0)) return (int)cudaErrorInvalidValue;
  const long most = (long)(sms > 0 ? sms : 148) * 16;
  LL_DISPATCH_DTYPE(dtype, {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = (width % VEC) == 0 && (shared_ff % VEC) == 0 && (ff % VEC) == 0 && ((uintptr_t)h % 16) == 0;
    const long total = (long)num_tokens * (wide ? width / VEC : width);
    const long want = (total + 255) / 256;
    const int blocks = (int)(want < most ? want : most);
    if (wide)
      ll_launch(moe_act_kernel<T, VEC>, dim3(blocks), dim3(256), 0, stream, (T*)h, gates, num_tokens, width, shared_ff,
                ff, E, act);
    else
      ll_launch(moe_act_kernel<T, 1>, dim3(blocks), dim3(256), 0, stream, (T*)h, gates, num_tokens, width, shared_ff,
                ff, E, act);
  });
  return LL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------
// Grouped path (many tokens): the (token, chosen expert) pairs are put in the order of the experts, the rows
// of the chosen tokens are gathered, and two grouped products (one group an expert, the groups' ends known on
// the device only) run over them; only the chosen experts' arithmetic is done.
// ---------------------------------------------------------------------------------------------------------

// One block.  ends [E]: the end of every expert's run of rows; row_token, row_w [pairs + E]: token and routing
// weight of every row; pair_row [pairs]: the row of pair (t, k).  Every expert's run starts with one row that no
// pair points at (token 0, weight 0), so that no run is empty: a grouped product does not have to cope with an
// expert that nobody chose.  Which row inside an expert's run a pair gets is decided by atomics; a row's result
// does not depend on its place.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ top_idx, const float* __restrict__ top_w, int pairs, int top, int E,
                int* __restrict__ ends, int* __restrict__ row_token, float* __restrict__ row_w,
                int* __restrict__ pair_row) {
  __shared__ int count[MOE_MAX_E];
  __shared__ int start[MOE_MAX_E];
  LL_PDL_WAIT();      // (no early release: what runs next may be a library kernel that does not wait itself)
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = top_idx[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      row_token[at] = 0;
      row_w[at] = 0.f;
      start[e] = at + 1;
      at += count[e];
      ends[e] = at;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = top_idx[p];
    if (e >= 0 && e < E) {
      const int row = atomicAdd(&start[e], 1);
      row_token[row] = p / top;
      row_w[row] = top_w[p];
      pair_row[p] = row;
    } else {
      pair_row[p] = -1;
    }
  }
}

// dst[row, :] = x[row_token[row], :]
template <typename T>
__global__ void moe_gather_rows_kernel(T* __restrict__ dst, const T* __restrict__ x, long x_stride,
                                       const int* __restrict__ row_token, int hidden) {
  LL_PDL_WAIT();      // (no early release: what runs next may be a library kernel that does not wait itself)
  const int row = blockIdx.x;
  const T* src = x + (size_t)row_token[row] * x_stride;
  T* d = dst + (size_t)row * hidden;
  constexpr int VEC = 16 / (int)sizeof(T);
  if ((hidden % VEC) == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)d % 16) == 0) {
    for (int i = threadIdx.x; i < hidden / VEC; i += blockDim.x)
      reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) d[i] = src[i];
  }
}

// h[row, :] = act(h[row, :]) * row_w[row], in place; VEC neighbouring numbers of a row a thread
template <typename T, int VEC>
__global__ void moe_row_act_kernel(T* __restrict__ h, const float* __restrict__ row_w, long total_vec, int ff, int act) {
  LL_PDL_WAIT();      // (no early release: what runs next may be a library kernel that does not wait itself)
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec; idx += step) {
    const float w = row_w[(idx * VEC) / ff];
    T v[VEC];
    if (VEC > 1) *reinterpret_cast<uint4*>(v) = reinterpret_cast<const uint4*>(h)[idx];
    else v[0] = h[idx];
#pragma unroll
    for (int u = 0; u < VEC; ++u) v[u] = from_f32<T>(moe_weighted_activation(to_f32<T>(v[u]), w, act));
    if (VEC > 1) reinterpret_cast<uint4*>(h)[idx] = *reinterpret_cast<const uint4*>(v);
    else h[idx] = v[0];
  }
}

// out[t, :] = base[t, :] + sum over k (in the order of k) of y[pair_row[t, k], :]; float32 sums, one rounding.
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const T* __restrict__ base, const T* __restrict__ y,
                                   const int* __restrict__ pair_row, int top, int hidden) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = pair_row[(size_t)t * top + k];
      if (row >= 0) a += to_f32<T>(y[(size_t)row * hidden + c]);
    }
    if (base) a += to_f32<T>(base[(size_t)t * hidden + c]);
    out[(size_t)t * hidden + c] = from_f32<T>(a);
  }
}

extern "C" int ll_moe_sort(const int* top_idx, const float* top_w, int num_tokens, int top, int E, int* ends,
                           int* row_token, float* row_w, int* pair_row, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_E || top <= 0) return (int)cudaErrorInvalidValue;
  ll_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, top_idx, top_w, num_tokens * top, top, E, ends, row_token,
            row_w, pair_row);
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_moe_gather_rows(int dtype, void* dst, const void* x, long x_stride, const int* row_token, int rows,
                                  int hidden, cudaStream_t stream) {
  if (rows <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(moe_gather_rows_kernel<T>, dim3(rows), dim3(128), 0, stream, (T*)dst, (const T*)x,
                                     x_stride, row_token, hidden));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_moe_row_act(int dtype, void* h, const float* row_w, int rows, int ff, int act, int sms,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  const long most = (long)(sms > 0 ? sms : 148) * 16;
  LL_DISPATCH_DTYPE(dtype, {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = (ff % VEC) == 0 && ((uintptr_t)h % 16) == 0;
    const long total = (long)rows * ff / (wide ? VEC : 1);
    const long want = (total + 255) / 256;
    const int blocks = (int)(want < most ? want : most);
    if (wide) ll_launch(moe_row_act_kernel<T, VEC>, dim3(blocks), dim3(256), 0, stream, (T*)h, row_w, total, ff, act);
    else ll_launch(moe_row_act_kernel<T, 1>, dim3(blocks), dim3(256), 0, stream, (T*)h, row_w, total, ff, act);
  });
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_moe_combine(int dtype, void* out, const void* base, const void* y, const int* pair_row,
                              int num_tokens, int top, int hidden, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  LL_DISPATCH_DTYPE(dtype, ll_launch(moe_combine_kernel<T>, dim3(num_tokens), dim3(256), 0, stream, (T*)out,
                                     (const T*)base, (const T*)y, pair_row, top, hidden));
  return LL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------
// Experts with a gate: an expert is down(a * sigmoid(alpha a) * (c + 1)) with a = min(gate x, limit) and
// c = clamp(up x, -limit, limit).  The first product's rows are, expert by expert, the gate rows then the up
// rows (an always-on expert's first).
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float clamped_swish_gate(float g, float u, float limit, float alpha) {
  const float a = fminf(g, limit);
  const float c = fminf(fmaxf(u, -limit), limit);
  return a / (1.0f + expf(-alpha * a)) * (c + 1.0f);
}

// in: T [tokens, 2 * (shared_ff + E * ff)]; out: T [tokens, shared_ff + E * ff] = activation times the
// expert's weight for the token: gates[t, e] for expert e (zero: not chosen, zeros are written and nothing is
// read), shared_w[t] (null: 1) for the always-on expert, which has a limit of its own.
template <typename T>
__global__ void moe_gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, const float* __restrict__ gates,
                                     const float* __restrict__ shared_w, int num_tokens, int shared_ff, int ff, int E,
                                     float limit, float shared_limit, float alpha) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int width = shared_ff + E * ff;
  const long total = (long)num_tokens * width;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const int t = (int)(idx / width);
    const int c = (int)(idx - (long)t * width);
    const T* row = in + (size_t)t * 2 * width;
    float w, g, u, lim;
    if (c < shared_ff) {
      w = shared_w ? shared_w[t] : 1.f;
      g = to_f32<T>(row[c]);
      u = to_f32<T>(row[shared_ff + c]);
      lim = shared_limit;
    } else {
      const int e = (c - shared_ff) / ff;
      const int j = (c - shared_ff) - e * ff;
      w = gates[(size_t)t * E + e];
      if (w == 0.f) {      // an expert that was not chosen contributes an exact zero whatever its first product gave
        out[idx] = from_f32<T>(0.f);
        continue;
      }
      const T* p = row + 2 * shared_ff + (size_t)e * 2 * ff;
      g = to_f32<T>(p[j]);
      u = to_f32<T>(p[ff + j]);
      lim = limit;
    }
    out[idx] = from_f32<T>(clamped_swish_gate(g, u, lim, alpha) * w);
  }
}

// in: T [rows, 2 * ff] (gate columns, then up columns); out: T [rows, ff] = activation times row_w[row].
// A thread takes VEC neighbouring units of a row (16-byte accesses where the width allows it).
template <typename T, int VEC>
__global__ void moe_row_gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, const float* __restrict__ row_w,
                                         long total_vec, int ff, float limit, float alpha) {
  LL_PDL_WAIT();      // (no early release: what runs next may be a library kernel that does not wait itself)
  const long step = (long)gridDim.x * blockDim.x;
  const int per_row = ff / VEC;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vec; idx += step) {
    const long r = idx / per_row;
    const int j = (int)(idx - r * per_row) * VEC;
    const float w = row_w ? row_w[r] : 1.f;
    const T* p = in + (size_t)r * 2 * ff + j;
    T g[VEC], u[VEC], y[VEC];
    if (VEC > 1) {
      *reinterpret_cast<uint4*>(g) = *reinterpret_cast<const uint4*>(p);
      *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(p + ff);
    } else {
      g[0] = p[0];
      u[0] = p[ff];
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      y[k] = from_f32<T>(clamped_swish_gate(to_f32<T>(g[k]), to_f32<T>(u[k]), limit, alpha) * w);
    if (VEC > 1) *reinterpret_cast<uint4*>(out + (size_t)r * ff + j) = *reinterpret_cast<const uint4*>(y);
    else out[(size_t)r * ff + j] = y[0];
  }
}

extern "C" int ll_moe_gated_act(int dtype, void* out, const void* in, const float* gates, const float* shared_w,
                                int num_tokens, int shared_ff, int ff, int E, float limit, float shared_limit,
                                float alpha, int sms, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long total = (long)num_tokens * (shared_ff + (long)E * ff);
  if (total <= 0) return (int)cudaErrorInvalidValue;
  const long most = (long)(sms > 0 ? sms : 148) * 16, want = (total + 255) / 256;
  LL_DISPATCH_DTYPE(dtype, ll_launch(moe_gated_act_kernel<T>, dim3((int)(want < most ? want : most)), dim3(256), 0,
                                     stream, (T*)out, (const T*)in, gates, shared_w, num_tokens, shared_ff, ff, E,
                                     limit, shared_limit, alpha));
  return LL_LAUNCH_RESULT();
}

extern "C" int ll_moe_row_gated_act(int dtype, void* out, const void* in, const float* row_w, int rows, int ff,
                                    float limit, float alpha, int sms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const long most = (long)(sms > 0 ? sms : 148) * 16;
  LL_DISPATCH_DTYPE(dtype, {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool wide = (ff % VEC) == 0 && ((uintptr_t)in % 16) == 0 && ((uintptr_t)out % 16) == 0;
    const long total = (long)rows * ff / (wide ? VEC : 1);
    const long want = (total + 255) / 256;
    const int blocks = (int)(want < most ? want : most);
    if (wide)
      ll_launch(moe_row_gated_act_kernel<T, VEC>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)in, row_w,
                total, ff, limit, alpha);
    else
      ll_launch(moe_row_gated_act_kernel<T, 1>, dim3(blocks), dim3(256), 0, stream, (T*)out, (const T*)in, row_w, total,
                ff, limit, alpha);
  });
  return LL_LAUNCH_RESULT();
}
