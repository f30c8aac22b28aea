// SiLU-gated product of the feed-forward: out[t, i] = silu(gu[t, i]) * gu[t, I + i].
//
// gate is the first I columns of the fused projection, up the last I.  The
// whole expression is evaluated in float32 and rounded once.
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, long total, int inter) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long idx0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = idx0; idx < total; idx += step) {
    const long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32<T>(gu[t * 2 * inter + i]);
    const float u = to_f32<T>(gu[t * 2 * inter + inter + i]);
    out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// 8 bf16 values a thread; needs inter % 8 == 0.
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gu, long total8, int inter8) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long idx0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = idx0; idx < total8; idx += step) {
    const long t = idx / inter8;
    const int i = (int)(idx - t * inter8);
    const uint4 gv = reinterpret_cast<const uint4*>(gu)[t * 2 * inter8 + i];
    const uint4 uv = reinterpret_cast<const uint4*>(gu)[t * 2 * inter8 + inter8 + i];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]);
      const float2 u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    reinterpret_cast<uint4*>(out)[idx] = ov;
  }
}

// SMs of the current device (asked once per device): the grid-stride kernels launch 16 blocks an SM at most
static int silu_device_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int ll_silu_mul(int dtype, void* out, const void* gate_up, int num_tokens, int inter, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long total = (long)num_tokens * inter;
  const long most = (long)silu_device_sms() * 16;
  if (dtype == LL_DTYPE_BF16 && (inter % 8) == 0) {
    const long total8 = total / 8;
    const int blocks = (int)min((total8 + 255) / 256, most);
    ll_launch(silu_mul_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (bf16*)out, (const bf16*)gate_up, total8,
              inter / 8);
    return LL_LAUNCH_RESULT();
  }
  const int blocks = (int)min((total + 255) / 256, most);
  LL_DISPATCH_DTYPE(dtype, ll_launch(silu_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out,
                                     (const T*)gate_up, total, inter));
  return LL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------
// The gated product with another activation: out[t, i] = act(gu[t, i]) * gu[t, I + i], act 0 SiLU, 1 ReLU.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float gate_activation(float g, int act) {
  return act == 1 ? fmaxf(g, 0.f) : g / (1.0f + expf(-g));
}

template <typename T>
__global__ void act_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, long total, int inter, int act) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long idx0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = idx0; idx < total; idx += step) {
    const long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_f32<T>(gu[t * 2 * inter + i]);
    const float u = to_f32<T>(gu[t * 2 * inter + inter + i]);
    out[idx] = from_f32<T>(gate_activation(g, act) * u);
  }
}

extern "C" int ll_act_mul(int dtype, void* out, const void* gate_up, int num_tokens, int inter, int act,
                          cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (act < 0 || act > 1) return (int)cudaErrorInvalidValue;
  const long total = (long)num_tokens * inter;
  const int blocks = (int)min((total + 255) / 256, (long)silu_device_sms() * 16);
  LL_DISPATCH_DTYPE(dtype, ll_launch(act_mul_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)out,
                                     (const T*)gate_up, total, inter, act));
  return LL_LAUNCH_RESULT();
}

// x[t, i] += bias[i] (float32 sum, rounded once), in place.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, long stride, const float* __restrict__ bias, long total, int width) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
    const long t = idx / width;
    const int i = (int)(idx - t * width);
    T* p = x + t * stride + i;
    *p = from_f32<T>(to_f32<T>(*p) + bias[i]);
  }
}

extern "C" int ll_add_bias(int dtype, void* x, long stride, const float* bias, int num_tokens, int width,
                           cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const long total = (long)num_tokens * width;
  const int blocks = (int)min((total + 255) / 256, (long)silu_device_sms() * 16);
  LL_DISPATCH_DTYPE(dtype, ll_launch(add_bias_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)x, stride, bias, total,
                                     width));
  return LL_LAUNCH_RESULT();
}

// z <- cap * tanh(z / cap) on float32 logits, in place.
__global__ void softcap_kernel(float* __restrict__ z, long total, float cap) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step)
    z[idx] = cap * tanhf(z[idx] / cap);
}

extern "C" int ll_softcap(float* z, long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
  const int blocks = (int)min((total + 255) / 256, (long)silu_device_sms() * 16);
  ll_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, z, total, cap);
  return LL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------
// Activation of a plain (ungated) feed-forward, in place: x <- act(x), float32, rounded once.
// act 0: gelu in its tanh form, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); 1: ReLU; 2: SiLU; 3: ReLU squared.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float row_activation(float z, int act) {
  if (act == 1) return fmaxf(z, 0.f);
  if (act == 2) return z / (1.0f + expf(-z));
  if (act == 3) return fmaxf(z, 0.f) * fmaxf(z, 0.f);
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ x, long total, int act) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step)
    x[i] = from_f32<T>(row_activation(to_f32<T>(x[i]), act));
}

// 8 bf16 values a thread (total % 8 == 0, 16-byte aligned)
__global__ void act_rows_bf16x8_kernel(bf16* __restrict__ x, long total8, int act) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += step) {
    uint4 v = reinterpret_cast<uint4*>(x)[i];
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      p[k] = __floats2bfloat162_rn(row_activation(f.x, act), row_activation(f.y, act));
    }
    reinterpret_cast<uint4*>(x)[i] = v;
  }
}

extern "C" int ll_act_rows(int dtype, void* x, long total, int act, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (act < 0 || act > 3) return (int)cudaErrorInvalidValue;
  const long most = (long)silu_device_sms() * 16;
  if (dtype == LL_DTYPE_BF16 && (total % 8) == 0 && ((uintptr_t)x % 16) == 0) {
    const int blocks = (int)min((total / 8 + 255) / 256, most);
    ll_launch(act_rows_bf16x8_kernel, dim3(blocks), dim3(256), 0, stream, (bf16*)x, total / 8, act);
    return LL_LAUNCH_RESULT();
  }
  const int blocks = (int)min((total + 255) / 256, most);
  LL_DISPATCH_DTYPE(dtype, ll_launch(act_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)x, total, act));
  return LL_LAUNCH_RESULT();
}

// z <- z * factor on float32 logits, in place.
__global__ void scale_f32_kernel(float* __restrict__ z, long total, float factor) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) z[idx] *= factor;
}

extern "C" int ll_scale_f32(float* z, long total, float factor, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)min((total + 255) / 256, (long)silu_device_sms() * 16);
  ll_launch(scale_f32_kernel, dim3(blocks), dim3(256), 0, stream, z, total, factor);
  return LL_LAUNCH_RESULT();
}
