// Kernels of blocks whose mixer and feed-forward read ONE norm and are added together, and of a latent attention whose
// keys carry a rotated part beside the latent.
//
//   latent_rope_store_kernel   one row of the fused input product [queries | latent, rotated key part | ...]: the latent's
//                              RMS norm, the rotation of the shared key part, both written to the row's page slot as one
//                              cached row [latent, rotated part, zeros]; and the rotation of every head's rotated query
//                              part in place. Rotate-half pairs (i, i + half) with float32 cos / sin tables per position.
//   add2_cast_kernel           x <- x + a (+ b) on the float32 stream, and the new x rounded to the model's type for the
//                              product that reads it next.
//   token_gate_kernel          g <- gelu_tanh(g) * E[token, off .. off + dim): a small gate times a per-token embedding.
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_rope_store_kernel(T* __restrict__ pages, long long page_stride, int page_size, int row_elems,
                                         T* __restrict__ proj, long long proj_stride, int latent_off, int rank,
                                         const void* __restrict__ w, int w_dtype, float eps, float w_offset, int rot_half,
                                         const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int max_pos,
                                         const int* __restrict__ positions, const int* __restrict__ slots, int heads,
                                         int q_head_stride, int q_rot_off, int store) {
  pdl_start();
  __shared__ float red[32];
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * proj_stride;
  int pos = positions[t];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const float* cs = cos_tab + (size_t)pos * rot_half;
  const float* sn = sin_tab + (size_t)pos * rot_half;
  // the heads' rotated query parts, in place
  for (int i = threadIdx.x; i < heads * rot_half; i += blockDim.x) {
    const int h = i / rot_half, d = i - h * rot_half;
    T* q = row + (size_t)h * q_head_stride + q_rot_off;
    const float a = to_f32(q[d]), b = to_f32(q[d + rot_half]);
    q[d] = from_f32<T>(a * cs[d] - b * sn[d]);
    q[d + rot_half] = from_f32<T>(b * cs[d] + a * sn[d]);
  }
  const int slot = (store && slots) ? slots[t] : -1;
  if (slot < 0) return;     // whole block leaves: a padding row, or a layer that reads another's pages
  const T* z = row + latent_off;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_f32(z[d]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)rank + eps);
  T* dst = pages + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * row_elems;
  for (int d = threadIdx.x; d < row_elems; d += blockDim.x) {
    float v = 0.f;
    if (d < rank) {
      v = to_f32(z[d]) * inv * (w_offset + load_as_f32(w, w_dtype, d));
    } else if (d < rank + 2 * rot_half) {
      const int r = d - rank;
      const int i = r < rot_half ? r : r - rot_half;
      const float a = to_f32(z[rank + i]), b = to_f32(z[rank + i + rot_half]);
      v = r < rot_half ? a * cs[i] - b * sn[i] : b * cs[i] + a * sn[i];
    }
    dst[d] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void add2_cast_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ low,
                                 long long n) {
  pdl_start();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i] + (b ? a[i] + b[i] : a[i]);
    x[i] = v;
    if (low) low[i] = from_f32<T>(v);
  }
}

// four elements a thread, 16-byte accesses on the float32 operands
template <typename T>
__global__ void add2_cast_vec_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ low,
                                     long long n4) {
  pdl_start();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(x)[i];
    const float4 av = reinterpret_cast<const float4*>(a)[i];
    if (b) {
      const float4 bv = reinterpret_cast<const float4*>(b)[i];
      v.x += av.x + bv.x, v.y += av.y + bv.y, v.z += av.z + bv.z, v.w += av.w + bv.w;
    } else {
      v.x += av.x, v.y += av.y, v.z += av.z, v.w += av.w;
    }
    reinterpret_cast<float4*>(x)[i] = v;
    if (low) {
      low[4 * i] = from_f32<T>(v.x), low[4 * i + 1] = from_f32<T>(v.y);
      low[4 * i + 2] = from_f32<T>(v.z), low[4 * i + 3] = from_f32<T>(v.w);
    }
  }
}

template <typename T>
__global__ void token_gate_kernel(T* __restrict__ g, long long g_stride, const int* __restrict__ token_ids, const void* __restrict__ table,
                                  int table_dtype, long long table_stride, int vocab, int off, int dim, long long n) {
  pdl_start();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dim;
    const int d = (int)(i - t * dim);
    int tok = token_ids[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float z = to_f32(g[t * g_stride + d]);
    const float act = 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    g[t * g_stride + d] = from_f32<T>(act * load_as_f32(table, table_dtype, (size_t)tok * table_stride + off + d));
  }
}

inline int grid_for(long long n) {
  const long long b = (n + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

// proj [tokens, proj_stride] in `dtype`: head h's rotated query part lies at h * q_head_stride + q_rot_off, the latent at
// latent_off (rank numbers) with the shared rotated key part (2 * rot_half numbers) directly behind it. pages
// [pages, page_size, row_elems >= rank + 2 * rot_half]. store 0: only the queries are rotated.
OI_API int oi_latent_rope_store(void* pages, long long page_stride, int page_size, int row_elems, void* proj, long long proj_stride,
                                int dtype, int tokens, int latent_off, int rank, const void* w, int w_dtype, float eps, float w_offset,
                                int rot_half, const float* cos_tab, const float* sin_tab, int max_pos, const int* positions,
                                const int* slots, int heads, int q_head_stride, int q_rot_off, int store, void* stream) {
  OI_REQUIRE(tokens >= 0 && rank > 0 && rot_half > 0 && heads > 0 && page_size > 0, "latent_rope_store: bad sizes");
  OI_REQUIRE(row_elems >= rank + 2 * rot_half, "latent_rope_store: a cached row of %d numbers cannot hold %d + %d", row_elems, rank,
             2 * rot_half);
  OI_REQUIRE(cos_tab && sin_tab && max_pos > 0 && positions, "latent_rope_store: the rotation needs tables and positions");
  OI_REQUIRE(!store || (pages && slots && w), "latent_rope_store: the store needs pages, slots and the norm's weight");
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_elems <= 64 ? 64 : (row_elems <= 128 ? 128 : 256);
  if (dtype == OI_F32)
    oi_launch(latent_rope_store_kernel<float>, tokens, threads, 0, s, (float*)pages, page_stride, page_size, row_elems, (float*)proj,
              proj_stride, latent_off, rank, w, w_dtype, eps, w_offset, rot_half, cos_tab, sin_tab, max_pos, positions, slots, heads,
              q_head_stride, q_rot_off, store);
  else if (dtype == OI_BF16)
    oi_launch(latent_rope_store_kernel<bf16>, tokens, threads, 0, s, (bf16*)pages, page_stride, page_size, row_elems, (bf16*)proj,
              proj_stride, latent_off, rank, w, w_dtype, eps, w_offset, rot_half, cos_tab, sin_tab, max_pos, positions, slots, heads,
              q_head_stride, q_rot_off, store);
  else
    OI_REQUIRE(false, "latent_rope_store: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// x [n] float32 <- x + a (+ b, when given); low [n] in `low_dtype` (or null) gets the new x rounded once.
OI_API int oi_add2_cast(float* x, const float* a, const float* b, void* low, int low_dtype, long long n, void* stream) {
  OI_REQUIRE(n >= 0 && x && a, "add2_cast: bad arguments");
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = n % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)a % 16 == 0 && (!b || (uintptr_t)b % 16 == 0);
  if (low_dtype == OI_F32) {
    if (vec) oi_launch(add2_cast_vec_kernel<float>, grid_for(n / 4), 256, 0, s, x, a, b, (float*)low, n / 4);
    else oi_launch(add2_cast_kernel<float>, grid_for(n), 256, 0, s, x, a, b, (float*)low, n);
  } else if (low_dtype == OI_BF16) {
    if (vec) oi_launch(add2_cast_vec_kernel<bf16>, grid_for(n / 4), 256, 0, s, x, a, b, (bf16*)low, n / 4);
    else oi_launch(add2_cast_kernel<bf16>, grid_for(n), 256, 0, s, x, a, b, (bf16*)low, n);
  } else {
    OI_REQUIRE(false, "add2_cast: unknown dtype code %d", low_dtype);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// g [tokens, dim] (row stride g_stride) in `dtype` <- gelu_tanh(g) * table[token_ids[t], off .. off + dim)
OI_API int oi_token_gate(void* g, long long g_stride, int dtype, const int* token_ids, const void* table, int table_dtype,
                         long long table_stride, int vocab, int off, int dim, int tokens, void* stream) {
  OI_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0 && off >= 0 && g && token_ids && table, "token_gate: bad arguments");
  const long long n = (long long)tokens * dim;
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32)
    oi_launch(token_gate_kernel<float>, grid_for(n), 256, 0, s, (float*)g, g_stride, token_ids, table, table_dtype, table_stride, vocab,
              off, dim, n);
  else if (dtype == OI_BF16)
    oi_launch(token_gate_kernel<bf16>, grid_for(n), 256, 0, s, (bf16*)g, g_stride, token_ids, table, table_dtype, table_stride, vocab,
              off, dim, n);
  else
    OI_REQUIRE(false, "token_gate: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
