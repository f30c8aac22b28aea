// Layer norm with a weight and no bias over a float32 residual stream, fused with the residual sum.
//
//   r = residual + (d1 + d2)                  (float32; d1, d2 optional, stored as T; d2 may instead come as
//                                              float32 partial sums of a product split over its inner
//                                              dimension, which are added up and rounded to T first, as the
//                                              unsplit product's result would have been)
//   y = (r - mean(r)) / sqrt(var(r) + eps) * w       (var = mean of the squared deviations)
//
// The residual stream stays float32 whatever the storage type T of the activations is: r is
// written back unrounded, and y is rounded once to T.  With `rows` given only those rows are
// read and nothing is written back (the last norm before the logits).  One block per row; the
// row is kept in shared memory between the passes (mean, then deviations: two passes, so that
// the variance is not a difference of large numbers).
#include "common.cuh"

template <typename T>
__global__ void add_layernorm_kernel(T* __restrict__ out, float* __restrict__ residual, const T* __restrict__ d1,
                                     const T* __restrict__ d2, const float* __restrict__ partial, int parts,
                                     long part_stride, const float* __restrict__ w, float eps, int hidden,
                                     const int* __restrict__ rows, int write_residual) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int i_out = blockIdx.x;
  const int r = rows ? rows[i_out] : i_out;
  float* res = residual + (size_t)r * hidden;
  const T* a = d1 ? d1 + (size_t)r * hidden : nullptr;
  const T* b = d2 ? d2 + (size_t)r * hidden : nullptr;
  const float* par = partial ? partial + (size_t)r * hidden : nullptr;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = res[i];
    if (a || b || par) {
      float d = a ? to_f32<T>(a[i]) : 0.f;
      if (b) d += to_f32<T>(b[i]);
      if (par) {
        float ps = 0.f;
        for (int q = 0; q < parts; ++q) ps += par[(size_t)q * part_stride + i];
        d += round_to<T>(ps);
      }
      v += d;
      if (write_residual) res[i] = v;
    }
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float c = row[i] - mean;
    ss += c * c;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  T* o = out + (size_t)i_out * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>((row[i] - mean) * inv * w[i]);
}

// out: [n_out, hidden] of T; residual: float32 [tokens, hidden]; d1, d2: T [tokens, hidden] or null.
extern "C" int ll_add_layernorm(int dtype, void* out, float* residual, const void* d1, const void* d2,
                                const float* partial, int parts, long part_stride, const float* w, float eps, int n_out,
                                int hidden, const int* rows, int write_residual, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (hidden <= 0) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (size_t)hidden;
  const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(add_layernorm_kernel<T>, dim3(n_out), dim3(threads), smem, stream, (T*)out, residual, (const T*)d1,
              (const T*)d2, partial, parts, part_stride, w, eps, hidden, rows, write_residual);
  });
  return LL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------------------------------
// Layer norm on a sublayer's *output*, added into a float32 residual stream:
//
//   residual += (y - mean(y)) / sqrt(var(y) + eps) * w          (float32, written back unrounded)
//   copy      = residual rounded to T                           (what the next sublayer's products read)
//
// y comes as T [tokens, hidden], or as float32 partial sums [parts, tokens, hidden] of a product that was
// split over its inner dimension; those are added up in a fixed order and not rounded.  `copy` may be null
// (float32 storage: the next reader takes the residual itself).  One block a row, two passes over the row
// in shared memory (mean, then deviations).
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void layernorm_into_residual_kernel(T* __restrict__ copy, float* __restrict__ residual,
                                               const T* __restrict__ y, const float* __restrict__ partial, int parts,
                                               long part_stride, const float* __restrict__ w, float eps, int hidden) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int r = blockIdx.x;
  float* res = residual + (size_t)r * hidden;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v;
    if (partial) {
      v = 0.f;
      for (int q = 0; q < parts; ++q) v += partial[(size_t)q * part_stride + (size_t)r * hidden + i];
    } else {
      v = to_f32<T>(y[(size_t)r * hidden + i]);
    }
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float c = row[i] - mean;
    ss += c * c;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = res[i] + (row[i] - mean) * inv * w[i];
    res[i] = v;
    if (copy) copy[(size_t)r * hidden + i] = from_f32<T>(v);
  }
}

// The same, four values a thread at a time (hidden a multiple of 4, so that every row starts on a 16-byte
// boundary of the float32 arrays and an 8-byte one of the bfloat16 ones).
template <typename T> __device__ __forceinline__ float4 ln_load4(const T* p);
template <> __device__ __forceinline__ float4 ln_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ln_load4<bf16>(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void ln_store4(T* p, float4 v);
template <> __device__ __forceinline__ void ln_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void ln_store4<bf16>(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&a);
  u.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename T>
__global__ void layernorm_into_residual_vec4_kernel(T* __restrict__ copy, float* __restrict__ residual,
                                                    const T* __restrict__ y, const float* __restrict__ partial,
                                                    int parts, long part_stride, const float* __restrict__ w,
                                                    float eps, int hidden) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const int r = blockIdx.x;
  float* res = residual + (size_t)r * hidden;
  float s = 0.f;
  for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
    float4 v;
    if (partial) {
      v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < parts; ++q) {
        const float4 a = *reinterpret_cast<const float4*>(partial + (size_t)q * part_stride + (size_t)r * hidden + i);
        v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
      }
    } else {
      v = ln_load4<T>(y + (size_t)r * hidden + i);
    }
    *reinterpret_cast<float4*>(row + i) = v;
    s += (v.x + v.y) + (v.z + v.w);
  }
  const float mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
    ss += (a * a + b * b) + (c * c + d * d);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    const float4 g = *reinterpret_cast<const float4*>(w + i);
    float4 o = *reinterpret_cast<const float4*>(res + i);
    o.x += (v.x - mean) * inv * g.x;
    o.y += (v.y - mean) * inv * g.y;
    o.z += (v.z - mean) * inv * g.z;
    o.w += (v.w - mean) * inv * g.w;
    *reinterpret_cast<float4*>(res + i) = o;
    if (copy) ln_store4<T>(copy + (size_t)r * hidden + i, o);
  }
}

// copy: [tokens, hidden] of T or null; residual: float32 [tokens, hidden]; y: T [tokens, hidden] or null when
// `partial` (float32 [parts, tokens, hidden], part_stride = tokens * hidden) is given.
extern "C" int ll_layernorm_into_residual(int dtype, void* copy, float* residual, const void* y, const float* partial,
                                          int parts, long part_stride, const float* w, float eps, int tokens,
                                          int hidden, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden <= 0 || (y == nullptr) == (partial == nullptr)) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (size_t)hidden;
  const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
  const uintptr_t ptrs = (uintptr_t)copy | (uintptr_t)residual | (uintptr_t)y | (uintptr_t)partial | (uintptr_t)w;
  if (hidden % 4 == 0 && ptrs % 16 == 0 && part_stride % 4 == 0) {
    const int vthreads = hidden >= 4096 ? 512 : hidden >= 1024 ? 256 : 128;
    LL_DISPATCH_DTYPE(dtype, {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(layernorm_into_residual_vec4_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
      ll_launch(layernorm_into_residual_vec4_kernel<T>, dim3(tokens), dim3(vthreads), smem, stream, (T*)copy, residual,
                (const T*)y, partial, parts, part_stride, w, eps, hidden);
    });
    return LL_LAUNCH_RESULT();
  }
  LL_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(layernorm_into_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ll_launch(layernorm_into_residual_kernel<T>, dim3(tokens), dim3(threads), smem, stream, (T*)copy, residual,
              (const T*)y, partial, parts, part_stride, w, eps, hidden);
  });
  return LL_LAUNCH_RESULT();
}

// copy[t, i] = residual[t, i] rounded to T: the float32 residual stream as the operand of a product.
template <typename T>
__global__ void round_rows_kernel(T* __restrict__ copy, const float* __restrict__ x, long total) {
  LL_PDL_TRIGGER();
  LL_PDL_WAIT();
  const long step = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) copy[i] = from_f32<T>(x[i]);
}

extern "C" int ll_round_rows(int dtype, void* copy, const float* x, long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)min((total + 255) / 256, (long)148 * 16);
  LL_DISPATCH_DTYPE(dtype, ll_launch(round_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)copy, x, total));
  return LL_LAUNCH_RESULT();
}
