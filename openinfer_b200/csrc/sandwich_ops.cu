// Kernels of blocks that norm a sublayer's input AND its output ("sandwich" blocks) with a Dynamic Tanh norm, and of an
// attention that rotates first and norms afterwards.
//
//   dyt(v; alpha, w, b) = tanh(alpha * v) * w + b       alpha a scalar tensor, w and b vectors; no mean, no variance
//
//   dyt_step_kernel        one pass over the float32 stream h [rows, width]:
//                            h <- h + dyt(branch; post)      when a sublayer's result (float32) is given
//                            out <- dyt(h; pre)              when the next sublayer's (or the head's) input is wanted, in the
//                                                            model's type, optionally only of the rows `row_idx` names
//                                                            (h is then left as it was: nothing reads it again)
//                          the place of residual add + norm in a pre-norm block: ONE kernel between two sublayers.
//   rope_norm_store_kernel one warp per (row, head) of the fused q | k | v projection (heads of `hd` numbers): adds the
//                          row's bias (a small table indexed by the row's position, see below), turns the first
//                          2 * rot_half numbers of q and k heads by the position's angles (pairs (d, d + rot_half)), divides
//                          q and k heads by their root mean square over `qk_dim` numbers (after the rotation, no weight),
//                          writes q back in place and k and v to the row's page slot.
//
// The bias table: a projection with a bias b that then passes a causal filter of `taps` taps (zeros before the sequence's
// start) equals the filter of the bias-free projection plus b * (sum of the taps that fall on positions >= 0), which
// depends on the position alone and is constant from position taps - 1 on: table[min(pos, n_tab - 1)][column].
#include "common.cuh"

namespace {

constexpr int kDytThreads = 256;

struct DytParams {
  const void* alpha;   // one number
  const void* w;       // [width]
  const void* b;       // [width]
  int dtype;
};

// four neighbouring numbers of a parameter vector (index a multiple of four), 8 or 16 bytes at a time
__device__ __forceinline__ void load4_as_f32(const void* p, int dtype, int i, float (&out)[4]) {
  if (dtype == OI_F32) {
    const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    out[0] = t.x, out[1] = t.y, out[2] = t.z, out[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    out[0] = a.x, out[1] = a.y, out[2] = b.x, out[3] = b.y;
  }
}
__device__ __forceinline__ void store4(float* o, const float (&v)[4]) { *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(bf16* o, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<unsigned*>(&a), t.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(o) = t;
}

// kVec: the width is a multiple of four and every pointer 16-byte aligned: four numbers a thread, 8- and 16-byte accesses
template <typename TO, bool kVec>
__global__ void dyt_step_kernel(float* __restrict__ h, const float* __restrict__ branch, DytParams post, DytParams pre,
                                TO* __restrict__ out, const int* __restrict__ row_idx, int width) {
  pdl_start();
  const int r = blockIdx.x;
  const int row = row_idx ? row_idx[r] : r;
  float* hr = h + (size_t)row * width;
  const float a_post = branch ? load_as_f32(post.alpha, post.dtype, 0) : 0.f;
  const float a_pre = out ? load_as_f32(pre.alpha, pre.dtype, 0) : 0.f;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < width; c += gridDim.y * blockDim.x * 4) {
    float v[4];
    if (kVec) {
      const float4 t = *reinterpret_cast<const float4*>(hr + c);
      v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = c + e < width ? hr[c + e] : 0.f;
    }
    if (branch) {
      const float* br = branch + (size_t)row * width;
      if (kVec) {
        const float4 t = *reinterpret_cast<const float4*>(br + c);
        const float y[4] = {t.x, t.y, t.z, t.w};
        float w[4], b[4];
        load4_as_f32(post.w, post.dtype, c, w);
        load4_as_f32(post.b, post.dtype, c, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += tanhf(a_post * y[e]) * w[e] + b[e];
        if (!row_idx) store4(hr + c, v);        // gathered rows: the stream is not read again, the sum stays in registers
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < width) {
            v[e] += tanhf(a_post * br[c + e]) * load_as_f32(post.w, post.dtype, c + e) + load_as_f32(post.b, post.dtype, c + e);
            if (!row_idx) hr[c + e] = v[e];
          }
      }
    }
    if (out) {
      TO* o = out + (size_t)r * width;
      if (kVec) {
        float w[4], b[4], y[4];
        load4_as_f32(pre.w, pre.dtype, c, w);
        load4_as_f32(pre.b, pre.dtype, c, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = tanhf(a_pre * v[e]) * w[e] + b[e];
        store4(o + c, y);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < width)
            o[c + e] = from_f32<TO>(tanhf(a_pre * v[e]) * load_as_f32(pre.w, pre.dtype, c + e) + load_as_f32(pre.b, pre.dtype, c + e));
      }
    }
  }
}

constexpr int kRopeWarps = 4;
constexpr int kRopeMaxHd = 512;

template <typename T>
__global__ void rope_norm_store_kernel(T* __restrict__ qkv, long long row_stride, int nq, int nkv, int hd, int qk_dim,
                                       const float* __restrict__ bias_tab, int n_tab, long long tab_stride,
                                       const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_half,
                                       int max_pos, int unit_norm, float eps, const int* __restrict__ positions,
                                       const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                       long long page_stride, int page_size, int write_kv, int tokens) {
  pdl_start();
  __shared__ float sh[kRopeWarps][kRopeMaxHd];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const int heads_total = write_kv ? nq + 2 * nkv : nq;
  const long long gw = (long long)blockIdx.x * kRopeWarps + wi;
  if (gw >= (long long)tokens * heads_total) return;       // whole warps leave; only warp-level barriers below
  const int token = (int)(gw / heads_total), head = (int)(gw - (long long)token * heads_total);
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
  T* src = qkv + (size_t)token * row_stride + (size_t)head * hd;
  T* dst = src;
  if (kind != 0) {
    const int slot = slots[token];
    if (slot < 0) return;                                    // a padding row stores nothing
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    dst = (kind == 1 ? k_cache : v_cache) + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * nkv * hd +
          (size_t)kvh * hd;
  }
  int pos = positions[token];
  pos = pos < 0 ? 0 : pos;
  const float* bias = bias_tab ? bias_tab + (size_t)min(pos, n_tab - 1) * tab_stride + (size_t)head * hd : nullptr;
  float* x = sh[wi];
  for (int d = lane; d < hd; d += 32) x[d] = to_f32(src[d]) + (bias ? bias[d] : 0.f);
  __syncwarp();
  if (kind == 2) {
    for (int d = lane; d < hd; d += 32) dst[d] = from_f32<T>(x[d]);
    return;
  }
  if (rot_half > 0) {
    const int p = pos >= max_pos ? max_pos - 1 : pos;        // admission bounds positions
    for (int i = lane; i < rot_half; i += 32) {
      const float c = cos_tab[(size_t)p * rot_half + i], s = sin_tab[(size_t)p * rot_half + i];
      const float a = x[i], b = x[i + rot_half];
      x[i] = a * c - b * s;
      x[i + rot_half] = b * c + a * s;
    }
    __syncwarp();
  }
  float inv = 1.f;
  if (unit_norm) {
    float ss = 0.f;
    for (int d = lane; d < qk_dim; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    inv = 1.f / sqrtf(ss / (float)qk_dim + eps);
  }
  for (int d = lane; d < hd; d += 32) dst[d] = from_f32<T>(x[d] * inv);
}

// The same for heads of 8, 16, 32, 64, 128 or 256 numbers whose rows can be read 16 bytes at a time and whose rotated
// halves are multiples of eight: eight neighbouring numbers a lane, hd / 8 lanes a head, 256 / hd heads a warp; a number's
// partner in the rotation comes from the lane rot_half / 8 further on (or back) by shuffles, the sum of squares is reduced
// over the head's lanes.
template <typename T>
__global__ void __launch_bounds__(128)
rope_norm_store_vec_kernel(T* __restrict__ qkv, long long row_stride, int nq, int nkv, int hd, int qk_dim,
                           const float* __restrict__ bias_tab, int n_tab, long long tab_stride,
                           const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int rot_half, int max_pos,
                           int unit_norm, float eps, const int* __restrict__ positions, const int* __restrict__ slots,
                           T* __restrict__ k_cache, T* __restrict__ v_cache, long long page_stride, int page_size, int write_kv,
                           int tokens) {
  pdl_start();
  const int lane = threadIdx.x & 31;
  const int lph = hd >> 3, per_warp = 32 / lph;               // lanes per head, heads per warp
  const int sub = lane / lph, l = lane - sub * lph;
  const int heads_total = write_kv ? nq + 2 * nkv : nq;
  const long long total = (long long)tokens * heads_total;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  long long item = gw * per_warp + sub;
  const bool active = item < total;
  if (!active) item = total - 1;                               // idle lanes follow along (the shuffles want every lane) and store nothing
  const int token = (int)(item / heads_total), head = (int)(item - (long long)token * heads_total);
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
  const int d0 = l * 8;
  T* src = qkv + (size_t)token * row_stride + (size_t)head * hd + d0;
  T* dst = src;
  bool store = active;
  if (kind != 0) {
    const int slot = slots[token];
    store = store && slot >= 0;
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    if (slot >= 0)
      dst = (kind == 1 ? k_cache : v_cache) + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * nkv * hd +
            (size_t)kvh * hd + d0;
  }
  int pos = positions[token];
  pos = pos < 0 ? 0 : pos;
  float x[8];
  if (sizeof(T) == 2) {
    const uint4 t = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      x[2 * e] = f.x, x[2 * e + 1] = f.y;
    }
  } else {
    const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
    x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
  }
  if (bias_tab) {
    const float4* b4 = reinterpret_cast<const float4*>(bias_tab + (size_t)min(pos, n_tab - 1) * tab_stride + (size_t)head * hd + d0);
    const float4 a = b4[0], b = b4[1];
    x[0] += a.x, x[1] += a.y, x[2] += a.z, x[3] += a.w, x[4] += b.x, x[5] += b.y, x[6] += b.z, x[7] += b.w;
  }
  // the rotation: numbers [0, rot_half) and [rot_half, 2 rot_half) of q and k heads are partners
  const bool turns = kind != 2 && d0 < 2 * rot_half;
  const bool low = d0 < rot_half;
  const int partner = turns ? (low ? lane + (rot_half >> 3) : lane - (rot_half >> 3)) : lane;
  float c[8], sn[8];
  if (turns) {
    const int p = pos >= max_pos ? max_pos - 1 : pos;
    const int i0 = low ? d0 : d0 - rot_half;
    const float4* c4 = reinterpret_cast<const float4*>(cos_tab + (size_t)p * rot_half + i0);
    const float4* s4 = reinterpret_cast<const float4*>(sin_tab + (size_t)p * rot_half + i0);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    c[0] = ca.x, c[1] = ca.y, c[2] = ca.z, c[3] = ca.w, c[4] = cb.x, c[5] = cb.y, c[6] = cb.z, c[7] = cb.w;
    sn[0] = sa.x, sn[1] = sa.y, sn[2] = sa.z, sn[3] = sa.w, sn[4] = sb.x, sn[5] = sb.y, sn[6] = sb.z, sn[7] = sb.w;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float other = __shfl_sync(0xffffffffu, x[e], partner);
    if (turns) x[e] = low ? x[e] * c[e] - other * sn[e] : x[e] * c[e] + other * sn[e];
  }
  float inv = 1.f;
  if (unit_norm) {
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += d0 + e < qk_dim ? x[e] * x[e] : 0.f;
    for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (kind != 2) inv = 1.f / sqrtf(ss / (float)qk_dim + eps);
  }
  if (!store) return;
  if (sizeof(T) == 2) {
    uint4 t;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
    for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(x[2 * e] * inv, x[2 * e + 1] * inv);
    *reinterpret_cast<uint4*>(dst) = t;
  } else {
    reinterpret_cast<float4*>(dst)[0] = make_float4(x[0] * inv, x[1] * inv, x[2] * inv, x[3] * inv);
    reinterpret_cast<float4*>(dst)[1] = make_float4(x[4] * inv, x[5] * inv, x[6] * inv, x[7] * inv);
  }
}

}  // namespace

// h [*, width] float32 (the stream; updated in place when `branch` is given); branch float32 [rows, width] or null;
// out [rows, width] of `out_dtype` or null; row_idx: the rows of h (and of branch) that `out` is formed from, or null.
// post_* / pre_*: alpha (one number), weight and bias of the two norms, all three of one dtype code each.
OI_API int oi_dyt_step(float* h, const float* branch, const void* post_alpha, const void* post_w, const void* post_b, int post_dtype,
                       const void* pre_alpha, const void* pre_w, const void* pre_b, int pre_dtype, void* out, int out_dtype,
                       const int* row_idx, int rows, int width, void* stream) {
  OI_REQUIRE(rows >= 0 && width > 0 && h != nullptr, "dyt_step: bad sizes rows=%d width=%d", rows, width);
  OI_REQUIRE(!branch || (post_alpha && post_w && post_b), "dyt_step: a branch needs the norm of its output");
  OI_REQUIRE(!out || (pre_alpha && pre_w && pre_b), "dyt_step: an output needs its norm");
  OI_REQUIRE(!row_idx || out, "dyt_step: gathered rows need an output");
  if (rows == 0 || (!branch && !out)) return OI_OK;
  const DytParams post{post_alpha, post_w, post_b, post_dtype}, pre{pre_alpha, pre_w, pre_b, pre_dtype};
  const int quads = (width + 3) / 4;
  const int threads = quads >= kDytThreads ? kDytThreads : ((quads + 31) / 32) * 32;
  const dim3 grid(rows, (quads + threads - 1) / threads);
  cudaStream_t s = (cudaStream_t)stream;
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = width % 4 == 0 && al(h) && al(branch) && al(out) && al(post_w) && al(post_b) && al(pre_w) && al(pre_b);
#define OI_DYT(T)                                                                                                        \
  do {                                                                                                                   \
    if (vec) oi_launch(dyt_step_kernel<T, true>, grid, threads, 0, s, h, branch, post, pre, (T*)out, row_idx, width);    \
    else oi_launch(dyt_step_kernel<T, false>, grid, threads, 0, s, h, branch, post, pre, (T*)out, row_idx, width);       \
  } while (0)
  if (!out || out_dtype == OI_F32) OI_DYT(float);
  else if (out_dtype == OI_BF16) OI_DYT(bf16);
  else
    OI_REQUIRE(false, "dyt_step: unknown dtype code %d", out_dtype);
#undef OI_DYT
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// qkv [tokens, row_stride]: heads of hd numbers, nq query heads, then (write_kv) nkv key heads and nkv value heads.
// bias_tab float32 [n_tab, tab_stride] or null; cos / sin float32 [max_pos, rot_half] or null (rot_half 0).
OI_API int oi_rope_norm_store(void* qkv, int dtype, long long row_stride, int tokens, int nq, int nkv, int hd, int qk_dim,
                              const float* bias_tab, int n_tab, long long tab_stride, const float* cos_tab, const float* sin_tab,
                              int rot_half, int max_pos, int unit_norm, float eps, const int* positions, const int* slots,
                              void* k_cache, void* v_cache, long long page_stride, int page_size, int write_kv, void* stream) {
  OI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && hd > 0 && hd <= kRopeMaxHd && qk_dim > 0 && qk_dim <= hd,
             "rope_norm_store: bad sizes nq=%d nkv=%d hd=%d qk_dim=%d", nq, nkv, hd, qk_dim);
  OI_REQUIRE(rot_half >= 0 && 2 * rot_half <= hd && (rot_half == 0 || (cos_tab && sin_tab && max_pos > 0)),
             "rope_norm_store: %d rotated pairs in a head of %d numbers, or no tables", rot_half, hd);
  OI_REQUIRE(positions && (!write_kv || (slots && k_cache && v_cache && page_size > 0)), "rope_norm_store: the step's positions and slots are missing");
  OI_REQUIRE(!bias_tab || n_tab > 0, "rope_norm_store: an empty bias table");
  if (tokens == 0) return OI_OK;
  const long long warps = (long long)tokens * (write_kv ? nq + 2 * nkv : nq);
  const unsigned blocks = (unsigned)((warps + kRopeWarps - 1) / kRopeWarps);
  cudaStream_t s = (cudaStream_t)stream;
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const int elem = dtype == OI_F32 ? 4 : 2;
  const bool vec = (hd == 8 || hd == 16 || hd == 32 || hd == 64 || hd == 128 || hd == 256) && rot_half % 8 == 0 && al(qkv) &&
                   (row_stride * elem) % 16 == 0 && (!bias_tab || (al(bias_tab) && tab_stride % 4 == 0)) &&
                   (rot_half == 0 || (al(cos_tab) && al(sin_tab))) &&
                   (!write_kv || (al(k_cache) && al(v_cache) && (page_stride * elem) % 16 == 0)) && (dtype == OI_F32 || dtype == OI_BF16);
  if (vec) {
    const int per_warp = 32 / (hd / 8);
    const long long vwarps = (warps + per_warp - 1) / per_warp;
    const unsigned vblocks = (unsigned)((vwarps + 3) / 4);
#define OI_RNSV(T)                                                                                                           \
  oi_launch(rope_norm_store_vec_kernel<T>, vblocks, 128, 0, s, (T*)qkv, row_stride, nq, nkv, hd, qk_dim, bias_tab, n_tab,     \
            tab_stride, cos_tab, sin_tab, rot_half, max_pos, unit_norm, eps, positions, slots, (T*)k_cache, (T*)v_cache,      \
            page_stride, page_size, write_kv, tokens)
    if (dtype == OI_F32) OI_RNSV(float); else OI_RNSV(bf16);
#undef OI_RNSV
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
#define OI_RNS(T)                                                                                                          \
  oi_launch(rope_norm_store_kernel<T>, blocks, kRopeWarps * 32, 0, s, (T*)qkv, row_stride, nq, nkv, hd, qk_dim, bias_tab, n_tab, \
            tab_stride, cos_tab, sin_tab, rot_half, max_pos, unit_norm, eps, positions, slots, (T*)k_cache, (T*)v_cache,    \
            page_stride, page_size, write_kv, tokens)
  if (dtype == OI_F32) OI_RNS(float);
  else if (dtype == OI_BF16) OI_RNS(bf16);
  else OI_REQUIRE(false, "rope_norm_store: unknown dtype code %d", dtype);
#undef OI_RNS
  OI_CHECK_LAUNCH();
  return OI_OK;
}
