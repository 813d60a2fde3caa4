// Paged causal attention, general form: any head_dim that is a multiple of 8 (up to 512), any
// number of heads and groups, an optional window, float32 or bfloat16 storage; prompt portions
// and single decoded tokens alike. One warp per (token, query head).
//
// s[i,j] = (q_i . k_j) * scale for j <= pos_i (and j > pos_i - window, or j among the sequence's kept first keys),
// online softmax in float32,
// o_i = sum_j p[i,j] v_j; query head h reads kv head h / (nq / nkv)
// (pegainfer-kernels/csrc/shared/paged_attention.cu:439-567; pegainfer-kernels/src/ops/attention.rs:507).
// The keys of a request are visited in position order, 32 at a time, whatever else is in the
// batch, so a row's result does not depend on how the batch was cut.
//
// This is the kernel of the true 32-bit path and of every shape the tuned kernels refuse.
//
// Score modifiers (OiScoreMods, all optional): the score of a query at position p is multiplied by
// 1 + coef * ln(floor((p + 1) / every) + 1); then capped, s <- cap * tanh(s / cap); then slope_h * (i - j) is taken off;
// and the softmax's denominator gets one more term exp(sink_h), which has no key and no value (it enters as the state
// the online softmax starts from: maximum sink_h, sum 1, nothing accumulated).
#include "common.cuh"
#include "oi_api.h"

#define ATTN_MAX_HD 512   // heads of more than 256 elements (a wide latent read as keys and values) get a second instance

template <typename T>
struct Vec16;  // 16 bytes of T
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <>
struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      out[2 * k] = f.x; out[2 * k + 1] = f.y;
    }
  }
};

template <typename T, int kWarps, int kMaxHd>
__global__ void attention_generic_kernel(
    const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride, int page_size,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
    const int* __restrict__ positions, int nq, int nkv, int hd, float scale, int window, int tokens, OiScoreMods mods) {
  pdl_start();
  __shared__ float q_sh[kWarps][kMaxHd];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int head = blockIdx.y * kWarps + warp;
  if (head >= nq) return;  // whole warp leaves; no block-wide barrier below
  const int req = token_req[token];
  if (req < 0) return;     // padding row
  const int pos = positions[token];
  const int kvh = head / (nq / nkv);
  const int* bt = block_table + (size_t)req * bt_stride;

  const T* qp = q + (size_t)token * q_row_stride + (size_t)head * hd;
  for (int d = lane; d < hd; d += 32) q_sh[warp][d] = to_f32(qp[d]);
  __syncwarp();

  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t row_elems = (size_t)nkv * hd;
  constexpr int VN = Vec16<T>::N;
  constexpr int kAccs = kMaxHd / 32;
  float acc[kAccs];
#pragma unroll
  for (int r = 0; r < kAccs; ++r) acc[r] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (mods.sinks) { m = mods.sinks[head]; l = 1.f; }
  if (mods.qt_every > 0) scale *= 1.f + mods.qt_coef * logf((float)((pos + 1) / mods.qt_every) + 1.f);
  const float slope = mods.slopes ? mods.slopes[head] : 0.f;
  const float cap = mods.softcap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;

  // the keys a row sees: [first, pos], and with kept first keys also [0, min(keep_first, first)) behind the window
  const int kept_end = mods.keep_first > 0 ? min(mods.keep_first, first) : 0;
  for (int seg = kept_end > 0 ? 0 : 1; seg < 2; ++seg) {
  const int seg_lo = seg == 0 ? 0 : first, seg_hi = seg == 0 ? kept_end : pos + 1;
  for (int base = seg_lo; base < seg_hi; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    if (j < seg_hi) {
      const int page = bt[j / page_size];
      const T* kp = k_cache + (size_t)page * page_stride + (size_t)(j % page_size) * row_elems + (size_t)kvh * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; d += VN) {
        float kv[VN];
        Vec16<T>::load(kp + d, kv);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot += q_sh[warp][d + e] * kv[e];
      }
      s = dot * scale;
      if (cap > 0.f) s = cap * tanhf(s * inv_cap);
      s -= slope * (float)(pos - j);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (j < seg_hi) ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);  // m = -inf on the first tile gives 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < kAccs; ++r) acc[r] *= corr;
    const int n_valid = min(32, seg_hi - base);
    for (int jj = 0; jj < n_valid; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int jv = base + jj;
      const int page = bt[jv / page_size];
      const T* vp = v_cache + (size_t)page * page_stride + (size_t)(jv % page_size) * row_elems + (size_t)kvh * hd;
#pragma unroll
      for (int r = 0; r < kAccs; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) acc[r] += pj * to_f32(vp[d]);
      }
    }
    m = m_new;
  }
  }
  T* op = out + (size_t)token * out_row_stride + (size_t)head * hd;
  const float inv_l = 1.f / l;
#pragma unroll
  for (int r = 0; r < kAccs; ++r) {
    const int d = lane + 32 * r;
    if (d < hd) op[d] = from_f32<T>(acc[r] * inv_l);
  }
}

OI_API int oi_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride, int dtype,
                                const void* k_cache, const void* v_cache, long long page_stride,
                                int page_size, const int* block_table, int bt_stride,
                                const int* token_req, const int* positions, int tokens, int nq, int nkv,
                                int hd, float scale, int window, const OiScoreMods* mods_in, void* stream) {
  OI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  OI_REQUIRE(hd > 0 && hd % 8 == 0 && hd <= ATTN_MAX_HD,
             "attention: head_dim %d unsupported (multiples of 8 up to %d)", hd, ATTN_MAX_HD);
  OI_REQUIRE(q_row_stride % 8 == 0 && page_stride % 8 == 0, "attention: strides must be multiples of 8 elements");
  OI_REQUIRE(page_size > 0, "attention: page_size %d", page_size);
  if (tokens == 0) return OI_OK;
  OiScoreMods mods = {};
  if (mods_in) mods = *mods_in;
  constexpr int kWarps = 4;
  dim3 grid(tokens, (nq + kWarps - 1) / kWarps);
  cudaStream_t s = (cudaStream_t)stream;
#define OI_ATTN_GENERIC(T, MAXHD)                                                                                   \
  oi_launch(attention_generic_kernel<T, kWarps, MAXHD>, grid, kWarps * 32, 0, s, (const T*)q, q_row_stride, (T*)out,  \
            out_row_stride, (const T*)k_cache, (const T*)v_cache, page_stride, page_size, block_table, bt_stride,    \
            token_req, positions, nq, nkv, hd, scale, window, tokens, mods)
  if (dtype == OI_F32) {
    if (hd <= 256) OI_ATTN_GENERIC(float, 256); else OI_ATTN_GENERIC(float, 512);
  } else if (dtype == OI_BF16) {
    if (hd <= 256) OI_ATTN_GENERIC(bf16, 256); else OI_ATTN_GENERIC(bf16, 512);
  } else {
    OI_REQUIRE(false, "attention: unknown dtype code %d", dtype);
  }
#undef OI_ATTN_GENERIC
  OI_CHECK_LAUNCH();
  return OI_OK;
}
