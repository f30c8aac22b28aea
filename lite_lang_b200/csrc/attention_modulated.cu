// Paged attention whose scores are shaped before the softmax: any sizes, float32 or bfloat16 storage, all
// arithmetic in float32.  The kernel of the true 32-bit path, and of the shapes the tensor-core kernels of
// this family do not take.
//
// For the query at position p of a request and a key at position j of the same request:
//   raw_h[j]  = scale * temp[h] * f(p) * (q_h . k_(h / group))   temp optional (a number a head); f(p) = 1 + coef *
//                                                                 ln(floor((p + 1) / every) + 1), optional
//   raw_h[j] <- cap * tanh(raw_h[j] / cap)                        cap optional
//   raw_h[j] <- raw_h[j] + rel[min(p - j, nd - 1), h]             rel optional: a bias by distance, [nd, nh]
//   s_h[j]    = sum_g mix[h, g] raw_g[j]                          mix optional ([nh, nh], mixes all heads' scores)
//   visible   : mask 0: j <= p;  1: p - j < size (a window) or j < keep (the request's first tokens stay
//               visible);  2: j / size == p / size (chunks counted from position 0 of the request), always j <= p
//   w_h[j]    = exp(s_h[j]) / (sink + sum_j' exp(s_h[j']))        sink 0: softmax; 1: one more key of score 0
//                                                                 that has no value; with sink_val, of score
//                                                                 sink_val[h]
//   o_h       = sum_j w_h[j] v_(h / group)[j]  (* sigmoid(gate[h]) with a gate a head, or every channel of the
//               head times the sigmoid of its own gate input)
//
// One block a token.  Without `mix` a block works on one kv head and its query heads; with it, on all heads
// at once, since every head's score needs every other head's.  Keys are walked in tiles that start at
// multiples of the tile size, so the order of every sum depends on the position only: the result for a
// position is the same bits however the tokens were cut into steps or batched.  Online softmax (running
// maximum, sum, accumulator) with expf; the sink starts the maximum at 0 and the sum at 1.  Rows of V of
// keys that are not visible are read as zeros, so what a page held before does not matter.
#include "common.cuh"

#define AM_THREADS 256
#define AM_WARPS 8

template <typename T, int ACC>
__global__ void __launch_bounds__(AM_THREADS)
attention_modulated_kernel(T* __restrict__ out, long out_stride, const T* __restrict__ q, long q_stride,
                           const T* __restrict__ gate, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                           const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
                           const int* __restrict__ req_slot, const int* __restrict__ positions, int nh, int nkv, int hd,
                           int vd, int page_size, int num_pages, int mask, int mask_size, int sink, float scale,
                           const float* __restrict__ temp, const float* __restrict__ mix, int tk, int* status,
                           const float* __restrict__ sink_val, const float* __restrict__ rel, int nd, int keep,
                           float cap, float qt_coef, int qt_every, long gate_stride, int gate_channels,
                           float out_scale) {
  extern __shared__ float smem[];
  LL_PDL_WAIT();
  LL_PDL_TRIGGER();
  const int t = blockIdx.x;
  const int group = nh / nkv;
  // heads and kv heads of this block
  const int nkb = mix ? nkv : 1;
  const int kv0 = mix ? 0 : blockIdx.y;
  const int hb = mix ? nh : group;
  const int head0 = kv0 * group;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  float* qs = smem;                               // [hb][hd]
  float* ks = qs + hb * hd;                       // [tk][nkb][hd + 1]
  float* vs = ks + tk * nkb * (hd + 1);           // [tk][nkb][vd]
  float* raw = vs + tk * nkb * vd;                // [hb][32]
  float* ps = raw + hb * 32;                      // [hb][32]
  float* m_s = ps + hb * 32;                      // [hb]
  float* l_s = m_s + hb;                          // [hb]
  float* alpha_s = l_s + hb;                      // [hb]
  float* mix_s = alpha_s + hb;                    // [hb][hb] with mix

  const int entry = token_req[t];
  const int slot = entry >= 0 ? req_slot[entry] : -1;
  const int p = positions[t];
  T* o_row = out + (size_t)t * out_stride + (size_t)head0 * vd;
  if (slot < 0 || p < 0) {  // padding entry of a captured batch: defined output, no reads
    for (int i = tid; i < hb * vd; i += AM_THREADS) o_row[i] = from_f32<T>(0.f);
    return;
  }
  const int* bt = block_table + (size_t)slot * bt_stride;
  int lo = 0;
  if (mask == 1 && mask_size > 0) lo = max(0, p - mask_size + 1);
  if (mask == 2 && mask_size > 0) lo = (p / mask_size) * mask_size;
  if (mask != 1) keep = 0;
  const float qf = qt_every > 0 ? 1.0f + qt_coef * logf((float)((p + 1) / qt_every) + 1.0f) : 1.0f;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head0 * hd;
  for (int i = tid; i < hb * hd; i += AM_THREADS) qs[i] = to_f32<T>(q_row[i]);
  for (int i = tid; i < hb; i += AM_THREADS) {
    m_s[i] = sink ? (sink_val ? sink_val[head0 + i] : 0.f) : -INFINITY;
    l_s[i] = sink ? 1.f : 0.f;
  }
  if (mix)
    for (int i = tid; i < hb * hb; i += AM_THREADS) mix_s[i] = mix[i];

  float acc[ACC];
#pragma unroll
  for (int c = 0; c < ACC; ++c) acc[c] = 0.f;
  const int outs = hb * vd;

  // tiles start at multiples of the tile size; with kept first tokens the tiles that hold them come first, then
  // the walk jumps to the window's first tile
  const int win0 = (lo / tk) * tk;
  for (int tile0 = keep > 0 ? 0 : win0; tile0 <= p; tile0 = (tile0 + tk < win0 && tile0 + tk >= keep) ? win0 : tile0 + tk) {
    __syncthreads();  // previous tile fully consumed (also orders the loads above before their first use)
    // ---- the K and V rows of this tile, all kv heads of the block ----
    for (int r = warp; r < tk * nkb; r += AM_WARPS) {
      const int j = r / nkb, kl = r - j * nkb;
      const int pos = tile0 + j;
      const bool valid = ((pos >= lo || pos < keep) && pos <= p);
      long base = -1;
      if (valid) {
        const int page = bt[pos / page_size];
        if (page < 0 || page >= num_pages) {
          if (lane == 0) set_status(status, LL_ERR_PAGE_RANGE);
        } else {
          base = ((long)page * nkv + kv0 + kl) * page_size + (pos % page_size);
        }
      }
      float* kd = ks + (size_t)r * (hd + 1);
      float* vdst = vs + (size_t)r * vd;
      for (int d = lane; d < hd; d += 32) kd[d] = base >= 0 ? to_f32<T>(k_cache[base * hd + d]) : 0.f;
      for (int d = lane; d < vd; d += 32) vdst[d] = base >= 0 ? to_f32<T>(v_cache[base * vd + d]) : 0.f;
    }
    __syncthreads();
    // ---- raw scores: a warp a head in turn, lane = key ----
    const int pos = tile0 + lane;
    const bool valid = lane < tk && (pos >= lo || pos < keep) && pos <= p;
    for (int h = warp; h < hb; h += AM_WARPS) {
      float s = 0.f;
      if (lane < tk) {
        const float* qh = qs + (size_t)h * hd;
        const float* kj = ks + ((size_t)lane * nkb + h / group) * (hd + 1);
        for (int d = 0; d < hd; ++d) s = fmaf(qh[d], kj[d], s);
        s *= (temp ? scale * temp[head0 + h] : scale) * qf;
        if (cap > 0.f) s = cap * tanhf(s / cap);
        if (rel && valid) s += rel[(size_t)min(p - pos, nd - 1) * nh + head0 + h];
      }
      raw[h * 32 + lane] = s;
    }
    if (mix) __syncthreads();
    // ---- mixing over heads, online softmax ----
    for (int h = warp; h < hb; h += AM_WARPS) {
      float s;
      if (mix) {
        s = 0.f;
        for (int g = 0; g < hb; ++g) s = fmaf(mix_s[h * hb + g], raw[g * 32 + lane], s);
      } else {
        s = raw[h * 32 + lane];
      }
      s = valid ? s : -INFINITY;
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float pj = valid ? expf(s - m_new) : 0.f;
      const float alpha = expf(m_old - m_new);
      const float l_new = l_s[h] * alpha + warp_sum(pj);
      ps[h * 32 + lane] = pj;
      __syncwarp();
      if (lane == 0) {
        m_s[h] = m_new;
        l_s[h] = l_new;
        alpha_s[h] = alpha;
      }
    }
    __syncthreads();
    // ---- accumulate P V: a thread owns outputs tid, tid + 256, ... of [hb][vd] ----
#pragma unroll
    for (int c = 0; c < ACC; ++c) {
      const int idx = tid + c * AM_THREADS;
      if (idx < outs) {
        const int h = idx / vd, d = idx - h * vd;
        const float* pg = ps + h * 32;
        const float* vcol = vs + (size_t)(h / group) * vd + d;
        float a = acc[c] * alpha_s[h];
        for (int j = 0; j < tk; ++j) a = fmaf(pg[j], vcol[(size_t)j * nkb * vd], a);
        acc[c] = a;
      }
    }
  }
  __syncthreads();
  // ---- normalise, gate and write ----
  const T* g_row = gate ? gate + (size_t)t * gate_stride + (gate_channels ? (size_t)head0 * vd : (size_t)head0) : nullptr;
#pragma unroll
  for (int c = 0; c < ACC; ++c) {
    const int idx = tid + c * AM_THREADS;
    if (idx < outs) {
      const int h = idx / vd;
      float o = acc[c] / l_s[h] * out_scale;
      if (g_row) o *= 1.0f / (1.0f + expf(-to_f32<T>(g_row[gate_channels ? idx : h])));
      o_row[idx] = from_f32<T>(o);
    }
  }
}

// Keys a tile for these sizes: the largest of 32, 16, 8 whose tile fits in shared memory.  It depends on the
// sizes only, never on the step, so a position's sums keep their order.
static int am_tile_keys(int hb, int nkb, int hd, int vd, size_t* smem_out) {
  for (int tk = 32; tk >= 8; tk >>= 1) {
    const size_t floats = (size_t)hb * hd + (size_t)tk * nkb * (hd + 1 + vd) + (size_t)hb * 64 + 3 * (size_t)hb +
                          (size_t)hb * hb;
    if (floats * sizeof(float) <= 200 * 1024) {
      *smem_out = floats * sizeof(float);
      return tk;
    }
  }
  return 0;
}

// q: rows of the step's tokens, head h of token t at q + t*q_stride + h*hd; gate (optional): a number a head
// and token at gate + t*gate_stride + h, through a sigmoid onto the head's output; with gate_channels a number a
// channel of every head, at gate + t*gate_stride + h*vd + c.
// sink_val: float32 [nh] or null (with sink: the score of the key without a value); rel: float32 [nd, nh] or null;
// keep: with mask 1, positions below it stay visible; cap > 0: scores through cap * tanh(s / cap);
// qt_every > 0: the query's factor 1 + qt_coef * ln(floor((p + 1) / qt_every) + 1).  out_scale: a constant on the
// output (before its one rounding).
// out: [num_tokens, nh*vd] with row stride out_stride.
// k_cache [num_pages, nkv, page_size, hd] and v_cache [num_pages, nkv, page_size, vd]: one cache plane.
// block_table: int32 [request slots, bt_stride]; token_req: int32 [num_tokens] entry of each token;
// req_slot: int32 [entries] request slot of each entry (-1: padding); positions: int32 [num_tokens].
// temp: float32 [nh] or null; mix: float32 [nh, nh] or null.
extern "C" int ll_attention_modulated(int dtype, void* out, long out_stride, const void* q, long q_stride,
                                      const void* gate, const void* k_cache, const void* v_cache,
                                      const int* block_table, int bt_stride, const int* token_req, const int* req_slot,
                                      const int* positions, int num_tokens, int nh, int nkv, int hd, int vd,
                                      int page_size, int num_pages, int mask, int mask_size, int sink, float scale,
                                      const float* temp, const float* mix, int* status, const float* sink_val,
                                      const float* rel, int nd, int keep, float cap, float qt_coef, int qt_every,
                                      long gate_stride, int gate_channels, float out_scale, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hd <= 0 || vd <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || mask < 0 || mask > 2 ||
      (rel != nullptr && nd <= 0) || keep < 0)
    return (int)cudaErrorInvalidValue;
  const int group = nh / nkv;
  const int hb = mix ? nh : group, nkb = mix ? nkv : 1;
  size_t smem = 0;
  const int tk = am_tile_keys(hb, nkb, hd, vd, &smem);
  const int per_thread = (hb * vd + AM_THREADS - 1) / AM_THREADS;
  if (tk == 0 || per_thread > 32) return (int)cudaErrorInvalidValue;
  dim3 grid(num_tokens, mix ? 1 : nkv);
#define AM_LAUNCH(ACC)                                                                                              \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(attention_modulated_kernel<T, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                           (int)smem);                                                                              \
    ll_launch(attention_modulated_kernel<T, ACC>, grid, dim3(AM_THREADS), smem, stream, (T*)out, out_stride,        \
              (const T*)q, q_stride, (const T*)gate, (const T*)k_cache, (const T*)v_cache, block_table, bt_stride,  \
              token_req, req_slot, positions, nh, nkv, hd, vd, page_size, num_pages, mask, mask_size, sink, scale,  \
              temp, mix, tk, status, sink_val, rel, nd, keep, cap, qt_coef, qt_every, gate_stride, gate_channels,   \
              out_scale);                                                                                           \
  } while (0)
  LL_DISPATCH_DTYPE(dtype, {
    if (per_thread <= 4) AM_LAUNCH(4);
    else if (per_thread <= 8) AM_LAUNCH(8);
    else if (per_thread <= 16) AM_LAUNCH(16);
    else AM_LAUNCH(32);
  });
#undef AM_LAUNCH
  return LL_LAUNCH_RESULT();
}
