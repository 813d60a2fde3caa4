// Row and channel steps of layers that keep their residual stream in 32-bit while the products run in the
// model's type: a norm that reads one type and writes another, the norm on a branch's OUTPUT fused with the
// residual sum (and with a weighted average over the outputs of all earlier layers), a short causal
// convolution over time with a per-request state, the norm + page write of a latent that attention reads
// as keys and values alike, a sigmoid gate per head, and the xIELU activation.
//
// All arithmetic is float32 with one rounding at the output. None of these kernels depends on how a
// request's tokens were cut into steps: rows are independent, and the convolution takes the inputs that lie
// before a portion from the request's state.
#include "oi_api.h"

namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
// log(1 + e^x) without overflow
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// ---------------------------------------------------------------------------------------------
// out[r] = round( x[src] * rsqrt(mean(x[src]^2) + eps) * (w_offset + w) ), src = row_idx ? row_idx[r] : r
// ---------------------------------------------------------------------------------------------
template <typename TX, typename TO>
__global__ void rmsnorm_cast_kernel(TO* __restrict__ out, const TX* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                    const int* __restrict__ row_idx, int hidden, float eps, float w_offset) {
  pdl_start();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
  const TX* xr = x + src * hidden;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = to_f32(xr[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TO* o = out + (size_t)r * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x)
    o[d] = from_f32<TO>(to_f32(xr[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d)));
}

// ---------------------------------------------------------------------------------------------
// v = h[r] + a[r] * rsqrt(mean(a[r]^2) + eps) * (w_offset + w)         (the branch's output, normed, joins the stream)
// without history:  h[r] = v
// with history:     hist[n_prev][r] = v;  h[r] = sum_{j < n_prev} coef[j] * hist[j][r] + coef[n_prev] * v
// low != null:      low[r] = round(h[r]) in bfloat16, for the product that reads the stream next
// ---------------------------------------------------------------------------------------------
template <typename TA>
__global__ void branch_norm_add_kernel(float* __restrict__ h, const TA* __restrict__ a, const void* __restrict__ w, int w_dtype,
                                       int hidden, float eps, float w_offset, float* __restrict__ hist, long long hist_stride,
                                       int n_prev, const void* __restrict__ coef, int coef_dtype, bf16* __restrict__ low) {
  pdl_start();
  __shared__ float red[32];
  const size_t row = (size_t)blockIdx.x * hidden;
  const TA* ar = a + row;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = to_f32(ar[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    const float v = h[row + d] + to_f32(ar[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d));
    float next = v;
    if (hist != nullptr) {
      hist[(size_t)n_prev * hist_stride + row + d] = v;
      float acc = 0.f;
      for (int j = 0; j < n_prev; ++j) acc += load_as_f32(coef, coef_dtype, j) * hist[(size_t)j * hist_stride + row + d];
      next = acc + load_as_f32(coef, coef_dtype, n_prev) * v;
    }
    h[row + d] = next;
    if (low != nullptr) low[row + d] = __float2bfloat16_rn(next);
  }
}

// the average alone (a layer without any branch norm in front of it): hist[n_prev] = h, h = sum_j coef[j] hist[j]
__global__ void history_average_kernel(float* __restrict__ h, float* __restrict__ hist, long long hist_stride, int n_prev,
                                       const void* __restrict__ coef, int coef_dtype, long long n) {
  pdl_start();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = h[i];
    hist[(size_t)n_prev * hist_stride + i] = v;
    float acc = 0.f;
    for (int j = 0; j < n_prev; ++j) acc += load_as_f32(coef, coef_dtype, j) * hist[(size_t)j * hist_stride + i];
    h[i] = acc + load_as_f32(coef, coef_dtype, n_prev) * v;
  }
}

// ---------------------------------------------------------------------------------------------
// out[t, c] = x[t, c] + sum_{j < taps} w[c, j] * x_(t - taps + 1 + j)[c]: inputs before the portion's first row come
// from the request's state (the last taps - 1 inputs of earlier steps, zeros before the sequence's start). The state
// holds two copies per request, [slots][2][taps - 1][channels]: a step reads copy state_phase[request] and leaves the
// state as it stands after the step in the other copy (the host turns the phase over when the step is committed), so
// that rows which read the old state and rows which write the new one can run in one kernel.
// ---------------------------------------------------------------------------------------------
template <typename TX, typename TO>
__global__ void short_conv_kernel(TO* __restrict__ out, const TX* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                  float* __restrict__ state, long long state_stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ token_req, const int* __restrict__ state_slots,
                                  const int* __restrict__ state_phase, int channels, int taps, int add_input,
                                  long long x_stride, long long out_stride, int act, int tokens) {
  pdl_start();
  if ((int)blockIdx.x >= tokens) {
    // behind the filter's blocks, one block per request (and chunk of channels) leaves the new state in the other copy:
    // the last taps - 1 inputs of (current copy, this step's rows)
    const int b = blockIdx.x - tokens, keep = taps - 1;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    if (n <= 0 || token_req[start] < 0) return;   // a padding request of a recorded step owns no state
    const int phase = state_phase[b];
    const float* old = state + (size_t)state_slots[b] * state_stride + (size_t)phase * keep * channels;
    float* st = state + (size_t)state_slots[b] * state_stride + (size_t)(1 - phase) * keep * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x)
      for (int k = 0; k < keep; ++k) {
        const int s = n + k - keep;
        st[(size_t)k * channels + c] = s >= 0 ? to_f32(x[(size_t)(start + s) * x_stride + c]) : old[(size_t)(k + n) * channels + c];
      }
    return;
  }
  const int t = blockIdx.x;
  const int req = token_req[t];
  const int start = req >= 0 ? cu_seqlens[req] : t;
  const int rel = t - start;
  const int keep = taps - 1;
  const float* st = (req >= 0 && keep > 0) ? state + (size_t)state_slots[req] * state_stride + (size_t)state_phase[req] * keep * channels
                                           : nullptr;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float cur = to_f32(x[(size_t)t * x_stride + c]);
    float acc = add_input ? cur : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int s = rel - keep + j;
      float v;
      if (s >= 0)
        v = to_f32(x[(size_t)(start + s) * x_stride + c]);
      else
        v = st ? st[(size_t)(keep + s) * channels + c] : 0.f;
      acc += load_as_f32(w, w_dtype, (size_t)c * taps + j) * v;
    }
    if (act == OI_ACT_SILU) acc = acc / (1.f + expf(-acc));
    out[(size_t)t * out_stride + c] = from_f32<TO>(acc);
  }
}

// ---------------------------------------------------------------------------------------------
// latent[t] = round( z * rsqrt(mean(z^2) + eps) * (w_offset + w) ), z = src[t, 0..rank), stored at the row's slot of
// the pages (rows of `row_elems` >= rank elements, the rest zero)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_store_kernel(T* __restrict__ pages, long long page_stride, int page_size, int row_elems,
                                    const T* __restrict__ src, long long src_stride, const void* __restrict__ w, int w_dtype,
                                    const int* __restrict__ slots, int rank, float eps, float w_offset) {
  pdl_start();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;     // whole block leaves
  const T* z = src + (size_t)t * src_stride;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_f32(z[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)rank + eps);
  T* dst = pages + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * row_elems;
  for (int d = threadIdx.x; d < row_elems; d += blockDim.x)
    dst[d] = d < rank ? from_f32<T>(to_f32(z[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d))) : from_f32<T>(0.f);
}

// o[t, h, :] *= sigmoid(g[t, h])
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ o, long long o_stride, const T* __restrict__ g, long long g_stride, int heads,
                                 int head_elems, long long n) {
  pdl_start();
  const int per_row = heads * head_elems;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int r = (int)(i - t * per_row);
    const float gate = sigmoid_f(to_f32(g[t * g_stride + r / head_elems]));
    T* p = o + t * o_stride + r;
    *p = from_f32<T>(to_f32(*p) * gate);
  }
}

// xIELU with learned shape: z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2
template <typename T>
__global__ void xielu_kernel(T* out, const T* in, const void* __restrict__ pq, int pq_dtype, long long n) {
  pdl_start();
  const float ap = softplus_f(load_as_f32(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(load_as_f32(pq, pq_dtype, 1));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float z = to_f32(in[i]);
    const float v = z > 0.f ? ap * z * z + 0.5f * z : an * (expm1f(z) - z) + 0.5f * z;
    out[i] = from_f32<T>(v);
  }
}

// ---------------------------------------------------------------------------------------------
// The same steps moving 16 bytes (or four elements) per access, for rows and pointers that allow it. A thread
// keeps its part of the row in registers between the sum of squares and the output.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void load4(const float* p, float v[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void load4(const bf16* p, float v[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}
__device__ __forceinline__ void load4(const void* p, int dtype, size_t i, float v[4]) {
  if (dtype == OI_F32) load4(reinterpret_cast<const float*>(p) + i, v);
  else load4(reinterpret_cast<const bf16*>(p) + i, v);
}
__device__ __forceinline__ void store4(float* p, const float v[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(bf16* p, const float v[4]) {
  uint2 t;
  *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = t;
}

constexpr int kMaxCoef = 256;   // terms of an average the vector kernel keeps in shared memory

template <typename TA, int VPT>
__global__ void branch_norm_add_vec_kernel(float* __restrict__ h, const TA* __restrict__ a, const void* __restrict__ w, int w_dtype,
                                           int hidden, float eps, float w_offset, float* __restrict__ hist, long long hist_stride,
                                           int n_prev, const void* __restrict__ coef, int coef_dtype, bf16* __restrict__ low) {
  pdl_trigger();
  __shared__ float red[32];
  __shared__ float cf[kMaxCoef];
  const int nvec = hidden / 4;
  float wv[VPT][4];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {     // weights and coefficients do not depend on the kernels ahead on the stream
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) load4(w, w_dtype, (size_t)v * 4, wv[k]);
  }
  if (hist != nullptr)
    for (int j = threadIdx.x; j <= n_prev; j += blockDim.x) cf[j] = load_as_f32(coef, coef_dtype, j);
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * hidden;
  float av[VPT][4], hv[VPT][4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      load4(a + row + (size_t)v * 4, av[k]);
      load4(h + row + (size_t)v * 4, hv[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += av[k][e] * av[k][e];
    }
  }
  ss = block_sum(ss, red);      // its barriers also publish cf
  const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v >= nvec) continue;
    const size_t at = row + (size_t)v * 4;
    float x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = hv[k][e] + av[k][e] * inv * (w_offset + wv[k][e]);
    if (hist != nullptr) {
      store4(hist + (size_t)n_prev * hist_stride + at, x);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
      for (int j = 0; j < n_prev; ++j) {
        float p[4];
        load4(hist + (size_t)j * hist_stride + at, p);
        const float c = cf[j];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] += c * p[e];
      }
      const float c = cf[n_prev];
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = acc[e] + c * x[e];
    }
    store4(h + at, x);
    if (low != nullptr) store4(low + at, x);
  }
}

// kConvRows consecutive rows and four channels per thread: a row's earlier inputs stay in registers while the thread
// walks down its rows (rows of one request are consecutive), the taps' weights are read once, and only a request's
// first rows of the step go to its state. The same launch leaves the new state: blocks behind the filter's own, one per
// request, write the copy of the state that the step does not read.
constexpr int kConvRows = 4;
constexpr int kConvMaxTaps = 8;
template <typename TX, typename TO, int kTaps>     // kTaps: 2, 4 or 8, at least the taps
__global__ void __launch_bounds__(256) short_conv_vec_kernel(
    TO* __restrict__ out, const TX* __restrict__ x, const void* __restrict__ w, int w_dtype, float* __restrict__ state,
    long long state_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ token_req,
    const int* __restrict__ state_slots, const int* __restrict__ state_phase, int tokens, int channels, int taps, int add_input,
    int conv_blocks, long long x_stride, long long out_stride, int act) {
  pdl_trigger();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const int keep = taps - 1;
  if ((int)blockIdx.x >= conv_blocks) {
    // The blocks behind the filter's own: one per request, they leave the state as it stands after the step in the copy
    // that the step does not read (the filter's blocks read the other one, so the two kinds of block never meet).
    pdl_wait();
    const int b = blockIdx.x - conv_blocks;
    const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
    if (c >= channels || n <= 0 || token_req[start] < 0) return;   // a padding request of a recorded step owns no state
    const int phase = state_phase[b];
    const float* old = state + (size_t)state_slots[b] * state_stride + (size_t)phase * keep * channels;
    float* nx = state + (size_t)state_slots[b] * state_stride + (size_t)(1 - phase) * keep * channels;
    for (int k = 0; k < keep; ++k) {
      const int s = n + k - keep;
      float v[4];
      if (s >= 0) load4(x + (size_t)(start + s) * x_stride + c, v);
      else load4(old + (size_t)(k + n) * channels + c, v);
      store4(nx + (size_t)k * channels + c, v);
    }
    return;
  }
  const int t0 = blockIdx.x * kConvRows;
  float wt[kTaps][4];
  if (c < channels) {
#pragma unroll
    for (int j = 0; j < kTaps; ++j)
      if (j < taps) {
#pragma unroll
        for (int e = 0; e < 4; ++e) wt[j][e] = load_as_f32(w, w_dtype, (size_t)(c + e) * taps + keep - j);   // of the input j rows above
      }
  }
  pdl_wait();
  if (c >= channels) return;
  // ring[i]: the input i + 1 rows above the current one
  float ring[kTaps][4];
#pragma unroll
  for (int j = 0; j < kTaps; ++j) {
    const int r = t0 - 1 - j;
    if (j < keep && r >= 0) load4(x + (size_t)r * x_stride + c, ring[j]);
  }
  const int t_end = min(tokens, t0 + kConvRows);
  // The requests of the rows and of the taps - 1 rows above them, and the rows' inputs: all asked for before any is used.
  // A request's rows are consecutive, so a row's place in its portion shows in its neighbours' requests alone.
  int reqs[kConvRows + kTaps - 1];
  float curs[kConvRows][4];
#pragma unroll
  for (int i = 0; i < kConvRows + kTaps - 1; ++i) {
    const int r = t0 - (kTaps - 1) + i;
    reqs[i] = (r >= 0 && r < t_end && r >= t0 - keep) ? token_req[r] : -2;
  }
#pragma unroll
  for (int i = 0; i < kConvRows; ++i)
    if (t0 + i < t_end) load4(x + (size_t)(t0 + i) * x_stride + c, curs[i]);
#pragma unroll
  for (int i = 0; i < kConvRows; ++i) {
    const int t = t0 + i;
    if (t >= t_end) break;
    const int req = reqs[i + kTaps - 1];
    int rel = 0;                 // rows of the same request directly above, counted up to taps - 1
#pragma unroll
    for (int j = 1; j < kTaps; ++j)
      if (j <= keep && rel == j - 1 && reqs[i + kTaps - 1 - j] == req) rel = j;
    // a portion's first rows read the copy of the request's state that is current in this step
    const float* st = (req >= 0 && rel < keep)
                          ? state + (size_t)state_slots[req] * state_stride + (size_t)state_phase[req] * keep * channels : nullptr;
    float cur[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) cur[e] = curs[i][e];
    float acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = add_input ? cur[e] : 0.f;
#pragma unroll
    for (int j = 0; j < kTaps; ++j) {     // j = 0: the row itself; j > 0: the input j rows above
      if (j >= taps) break;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (j == 0) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = cur[e];
      } else if (rel - j >= 0) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = ring[j - 1][e];
      } else if (st) {
        load4(st + (size_t)(keep + rel - j) * channels + c, v);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] += wt[j][e] * v[e];
    }
    if (act == OI_ACT_SILU) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = acc[e] / (1.f + expf(-acc[e]));
    }
    store4(out + (size_t)t * out_stride + c, acc);
#pragma unroll
    for (int j = kTaps - 1; j > 0; --j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) ring[j][e] = ring[j - 1][e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) ring[0][e] = cur[e];
  }
}

// o[t, h, :] *= sigmoid(g[t, h]), 16 bytes per access (a head's elements are a multiple of the vector)
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ o, long long o_stride, const T* __restrict__ g, long long g_stride,
                                     int head_elems, int vecs_per_row) {
  pdl_start();
  constexpr int EPV = 16 / sizeof(T);
  const int t = blockIdx.x;
  for (int v = blockIdx.y * blockDim.x + threadIdx.x; v < vecs_per_row; v += gridDim.y * blockDim.x) {
    const float gate = sigmoid_f(to_f32(g[(size_t)t * g_stride + (v * EPV) / head_elems]));
    T* p = o + (size_t)t * o_stride + (size_t)v * EPV;
    float a[4], b[4] = {0.f, 0.f, 0.f, 0.f};
    load4(p, a);
    if (EPV == 8) load4(p + 4, b);
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] *= gate, b[e] *= gate;
    store4(p, a);
    if (EPV == 8) store4(p + 4, b);
  }
}

// 16 bytes per access
template <typename T>
__global__ void xielu_vec_kernel(T* out, const T* in, const void* __restrict__ pq, int pq_dtype, long long nvec) {
  pdl_start();
  constexpr int EPV = 16 / sizeof(T);
  const float ap = softplus_f(load_as_f32(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(load_as_f32(pq, pq_dtype, 1));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float z[8];
    load4(in + i * EPV, z);
    if (EPV == 8) load4(in + i * EPV + 4, z + 4);
#pragma unroll
    for (int e = 0; e < EPV; ++e) {
      // a bfloat16 result keeps 8 bits: the special-function unit's exponential (2 ulp of float32) is exact enough there
      const float em1 = sizeof(T) == 2 ? __expf(z[e]) - 1.f : expm1f(z[e]);
      z[e] = z[e] > 0.f ? ap * z[e] * z[e] + 0.5f * z[e] : an * (em1 - z[e]) + 0.5f * z[e];
    }
    store4(out + i * EPV, z);
    if (EPV == 8) store4(out + i * EPV + 4, z + 4);
  }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

int flat_blocks(long long n) {
  const long long b = (n + kRowThreads - 1) / kRowThreads;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

OI_API int oi_rmsnorm_cast(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, const int* row_idx,
                           int rows, int hidden, float eps, float w_offset, void* stream) {
  OI_REQUIRE(rows >= 0 && hidden > 0, "rmsnorm_cast: bad sizes rows=%d hidden=%d", rows, hidden);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define OI_CAST_CASE(XD, OD, TX, TO)                                                                                  \
  if (x_dtype == XD && out_dtype == OD) {                                                                             \
    oi_launch(rmsnorm_cast_kernel<TX, TO>, rows, kRowThreads, 0, s, (TO*)out, (const TX*)x, w, w_dtype, row_idx, hidden, eps, \
              w_offset);                                                                                              \
    OI_CHECK_LAUNCH();                                                                                                \
    return OI_OK;                                                                                                     \
  }
  OI_CAST_CASE(OI_F32, OI_F32, float, float)
  OI_CAST_CASE(OI_F32, OI_BF16, float, bf16)
  OI_CAST_CASE(OI_BF16, OI_F32, bf16, float)
  OI_CAST_CASE(OI_BF16, OI_BF16, bf16, bf16)
#undef OI_CAST_CASE
  OI_REQUIRE(false, "rmsnorm_cast: unknown dtype codes %d -> %d", x_dtype, out_dtype);
}

OI_API int oi_branch_norm_add(float* h, const void* a, int a_dtype, const void* w, int w_dtype, int rows, int hidden, float eps,
                              float w_offset, float* hist, long long hist_stride, int n_prev, const void* coef, int coef_dtype,
                              void* low, void* stream) {
  OI_REQUIRE(rows >= 0 && hidden > 0, "branch_norm_add: bad sizes rows=%d hidden=%d", rows, hidden);
  OI_REQUIRE(hist == nullptr || (coef != nullptr && n_prev >= 0 && hist_stride >= (long long)rows * hidden),
             "branch_norm_add: the history needs coefficients and a stride of at least rows * hidden");
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int nvec = hidden / 4;
  if (hidden % 4 == 0 && nvec <= 512 * 4 && aligned16(h) && aligned16(a) && aligned16(w) && (!hist || (aligned16(hist) && hist_stride % 4 == 0 &&
      n_prev < kMaxCoef)) && (!low || aligned16(low)) && (a_dtype == OI_F32 || a_dtype == OI_BF16)) {
    const int vpt = nvec <= 256 ? 1 : (nvec <= 1024 ? 2 : 4);
    const int threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32;
#define OI_BNA(TA, V)                                                                                                        \
  oi_launch(branch_norm_add_vec_kernel<TA, V>, rows, threads, 0, s, h, (const TA*)a, w, w_dtype, hidden, eps, w_offset, hist, \
            hist_stride, n_prev, coef, coef_dtype, (bf16*)low)
    if (a_dtype == OI_F32) {
      if (vpt == 1) OI_BNA(float, 1); else if (vpt == 2) OI_BNA(float, 2); else OI_BNA(float, 4);
    } else {
      if (vpt == 1) OI_BNA(bf16, 1); else if (vpt == 2) OI_BNA(bf16, 2); else OI_BNA(bf16, 4);
    }
#undef OI_BNA
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  if (a_dtype == OI_F32)
    oi_launch(branch_norm_add_kernel<float>, rows, kRowThreads, 0, s, h, (const float*)a, w, w_dtype, hidden, eps, w_offset, hist,
              hist_stride, n_prev, coef, coef_dtype, (bf16*)low);
  else if (a_dtype == OI_BF16)
    oi_launch(branch_norm_add_kernel<bf16>, rows, kRowThreads, 0, s, h, (const bf16*)a, w, w_dtype, hidden, eps, w_offset, hist,
              hist_stride, n_prev, coef, coef_dtype, (bf16*)low);
  else
    OI_REQUIRE(false, "branch_norm_add: unknown dtype code %d", a_dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_history_average(float* h, float* hist, long long hist_stride, int n_prev, const void* coef, int coef_dtype,
                              long long n, void* stream) {
  OI_REQUIRE(h && hist && coef && n_prev >= 0 && n >= 0 && hist_stride >= n, "history_average: bad arguments");
  if (n == 0) return OI_OK;
  oi_launch(history_average_kernel, flat_blocks(n), kRowThreads, 0, (cudaStream_t)stream, h, hist, hist_stride, n_prev, coef,
            coef_dtype, n);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// x_stride / out_stride: elements between rows (the channels of a row may be a slice of a wider buffer); act: OI_ACT_NONE
// or OI_ACT_SILU on the filter's result. The state keeps the INPUTS, so the activation does not touch it.
OI_API int oi_short_conv_strided(void* out, int out_dtype, long long out_stride, const void* x, int x_dtype, long long x_stride,
                                 const void* w, int w_dtype, float* state, long long state_stride, const int* cu_seqlens,
                                 const int* token_req, const int* state_slots, const int* state_phase, int tokens, int requests,
                                 int channels, int taps, int add_input, int update_state, int act, void* stream) {
  OI_REQUIRE(act == OI_ACT_NONE || act == OI_ACT_SILU, "short_conv: unknown activation code %d", act);
  OI_REQUIRE(x_stride >= channels && out_stride >= channels, "short_conv: rows narrower than the channels");
  OI_REQUIRE(tokens >= 0 && requests >= 0 && channels > 0 && taps >= 1, "short_conv: bad sizes tokens=%d channels=%d taps=%d",
             tokens, channels, taps);
  OI_REQUIRE(taps == 1 || (state != nullptr && state_phase != nullptr && state_stride >= 2LL * (taps - 1) * channels),
             "short_conv: %d taps need a state of two copies of %d rows per request, and the requests' phases", taps, taps - 1);
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int cy = (channels + kRowThreads - 1) / kRowThreads;
  const dim3 grid(tokens, cy);
  const bool vec = x_stride % 4 == 0 && out_stride % 4 == 0 && channels % 4 == 0 && taps <= kConvMaxTaps && aligned16(out) &&
                   aligned16(x) &&
                   (taps == 1 || (aligned16(state) && state_stride % 4 == 0));
  const int vthreads = channels / 4 >= 256 ? 256 : ((channels / 4 + 31) / 32) * 32;
  // the filter's blocks, and behind them one block per request (and chunk of channels) that leaves the new state
  const int conv_blocks = (tokens + kConvRows - 1) / kConvRows;
  const dim3 vgrid(conv_blocks + ((update_state && taps > 1) ? requests : 0), vec ? (channels / 4 + vthreads - 1) / vthreads : 1);
#define OI_CONV_VEC(TX, TO, KT)                                                                                          \
  oi_launch(short_conv_vec_kernel<TX, TO, KT>, vgrid, vthreads, 0, s, (TO*)out, (const TX*)x, w, w_dtype, state, state_stride, \
            cu_seqlens, token_req, state_slots, state_phase, tokens, channels, taps, add_input, conv_blocks, x_stride, out_stride, act)
#define OI_CONV_CASE(XD, OD, TX, TO)                                                                                     \
  if (x_dtype == XD && out_dtype == OD) {                                                                                \
    if (vec) {                                                                                                           \
      if (taps <= 2) OI_CONV_VEC(TX, TO, 2);                                                                             \
      else if (taps <= 4) OI_CONV_VEC(TX, TO, 4);                                                                        \
      else OI_CONV_VEC(TX, TO, 8);                                                                                       \
      OI_CHECK_LAUNCH();                                                                                                 \
      return OI_OK;                                                                                                      \
    }                                                                                                                    \
    /* the filter's blocks, and behind them one block per request (and chunk of channels) that leaves the new state */    \
    oi_launch(short_conv_kernel<TX, TO>, dim3(tokens + ((update_state && taps > 1) ? requests : 0), cy), kRowThreads, 0, s, \
              (TO*)out, (const TX*)x, w, w_dtype, state, state_stride, cu_seqlens, token_req, state_slots, state_phase,  \
              channels, taps, add_input, x_stride, out_stride, act, tokens);                                             \
    OI_CHECK_LAUNCH();                                                                                                   \
    return OI_OK;                                                                                                        \
  }
  OI_CONV_CASE(OI_F32, OI_F32, float, float)
  OI_CONV_CASE(OI_F32, OI_BF16, float, bf16)
  OI_CONV_CASE(OI_BF16, OI_BF16, bf16, bf16)
#undef OI_CONV_CASE
#undef OI_CONV_VEC
  OI_REQUIRE(false, "short_conv: dtype codes %d -> %d are not supported", x_dtype, out_dtype);
}

OI_API int oi_short_conv(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, float* state,
                         long long state_stride, const int* cu_seqlens, const int* token_req, const int* state_slots,
                         const int* state_phase, int tokens, int requests, int channels, int taps, int add_input, int update_state,
                         void* stream) {
  return oi_short_conv_strided(out, out_dtype, channels, x, x_dtype, channels, w, w_dtype, state, state_stride, cu_seqlens, token_req,
                               state_slots, state_phase, tokens, requests, channels, taps, add_input, update_state, OI_ACT_NONE, stream);
}

OI_API int oi_latent_store(void* pages, long long page_stride, int page_size, int row_elems, const void* src, long long src_stride,
                           int dtype, const void* w, int w_dtype, const int* slots, int tokens, int rank, float eps, float w_offset,
                           void* stream) {
  OI_REQUIRE(tokens >= 0 && rank > 0 && row_elems >= rank && page_size > 0, "latent_store: bad sizes rank=%d row=%d", rank, row_elems);
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = rank <= 64 ? 64 : (rank <= 128 ? 128 : kRowThreads);
  if (dtype == OI_F32)
    oi_launch(latent_store_kernel<float>, tokens, threads, 0, s, (float*)pages, page_stride, page_size, row_elems, (const float*)src,
              src_stride, w, w_dtype, slots, rank, eps, w_offset);
  else if (dtype == OI_BF16)
    oi_launch(latent_store_kernel<bf16>, tokens, threads, 0, s, (bf16*)pages, page_stride, page_size, row_elems, (const bf16*)src,
              src_stride, w, w_dtype, slots, rank, eps, w_offset);
  else
    OI_REQUIRE(false, "latent_store: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_head_gate(void* o, long long o_stride, const void* g, long long g_stride, int dtype, int tokens, int heads,
                        int head_elems, void* stream) {
  OI_REQUIRE(tokens >= 0 && heads > 0 && head_elems > 0, "head_gate: bad sizes");
  const long long n = (long long)tokens * heads * head_elems;
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int epv = dtype == OI_F32 ? 4 : 8;
  if ((dtype == OI_F32 || dtype == OI_BF16) && head_elems % epv == 0 && o_stride % epv == 0 && aligned16(o)) {
    const int vecs = heads * head_elems / epv;
    const int threads = vecs >= 256 ? 256 : ((vecs + 31) / 32) * 32;
    const dim3 grid(tokens, (vecs + threads - 1) / threads);
    if (dtype == OI_F32)
      oi_launch(head_gate_vec_kernel<float>, grid, threads, 0, s, (float*)o, o_stride, (const float*)g, g_stride, head_elems, vecs);
    else
      oi_launch(head_gate_vec_kernel<bf16>, grid, threads, 0, s, (bf16*)o, o_stride, (const bf16*)g, g_stride, head_elems, vecs);
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  if (dtype == OI_F32)
    oi_launch(head_gate_kernel<float>, flat_blocks(n), kRowThreads, 0, s, (float*)o, o_stride, (const float*)g, g_stride, heads,
              head_elems, n);
  else if (dtype == OI_BF16)
    oi_launch(head_gate_kernel<bf16>, flat_blocks(n), kRowThreads, 0, s, (bf16*)o, o_stride, (const bf16*)g, g_stride, heads,
              head_elems, n);
  else
    OI_REQUIRE(false, "head_gate: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_xielu(void* out, const void* in, int dtype, const void* pq, int pq_dtype, long long n, void* stream) {
  OI_REQUIRE(n >= 0 && pq != nullptr, "xielu: bad arguments");
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int epv = dtype == OI_F32 ? 4 : 8;
  if ((dtype == OI_F32 || dtype == OI_BF16) && n % epv == 0 && aligned16(out) && aligned16(in)) {
    if (dtype == OI_F32)
      oi_launch(xielu_vec_kernel<float>, flat_blocks(n / epv), kRowThreads, 0, s, (float*)out, (const float*)in, pq, pq_dtype, n / epv);
    else
      oi_launch(xielu_vec_kernel<bf16>, flat_blocks(n / epv), kRowThreads, 0, s, (bf16*)out, (const bf16*)in, pq, pq_dtype, n / epv);
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  if (dtype == OI_F32)
    oi_launch(xielu_kernel<float>, flat_blocks(n), kRowThreads, 0, s, (float*)out, (const float*)in, pq, pq_dtype, n);
  else if (dtype == OI_BF16)
    oi_launch(xielu_kernel<bf16>, flat_blocks(n), kRowThreads, 0, s, (bf16*)out, (const bf16*)in, pq, pq_dtype, n);
  else
    OI_REQUIRE(false, "xielu: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
