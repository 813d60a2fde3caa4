// Recurrent mixers whose memory is a matrix per head: a scan over the rows of a step, request by request.
//
// Both kinds keep, per request and head, C [D keys x V values] in float32 and update it token by token:
//
//   kMatrixMemory (the mLSTM cell):  m' = max(f + m, i);  C' = e^(f + m - m') C + e^(i - m') k v^T;  n' likewise with k;
//                                    o = C'^T q / (max(|n' . q|, e^(-m')) + 1e-6);  i = cap tanh(zi / cap),
//                                    f = logsigmoid(cap tanh(zf / cap)); q arrives unscaled and is multiplied by q_scale
//   kGatedDelta (gated delta rule):  C <- diag(g) C;  d = beta (v - C^T k);  C <- C + k d^T;  o = C^T q, with k and q made
//                                    unit vectors (1e-6 inside the root), q times q_scale, beta = sigmoid(zb) and one decay
//                                    per key channel g = exp(-exp(A_h) softplus(a + dt))
//   kLinearDecay (linear attention with one fixed decay per head, "lightning attention"):
//                                    C <- lambda_h C + k v^T;  o = C^T q, with q, k and v through silu first and no other scale
//
// Prompts and single decoded tokens take the same two launches. A first kernel forms, for all rows at once, what does
// not depend on earlier rows (gates, decays, unit vectors); then block (request, head, slice of value columns) walks the
// request's rows of the step in order, its slice of C in registers (a column's D numbers spread over 4 to 16 lanes), the
// rows' records staged in shared memory a chunk at a time (cp.async, two buffers), so that the loop over rows is the recurrence alone. The state
// lives in two copies that take turns ([slots][2][heads][elems], C stored column by column, then n and m): a step reads
// copy state_phase[request] and leaves the other, so no block reads what another writes. Everything is float32: the
// inputs are the float32 sums of the projections.
#include "common.cuh"

namespace {

enum : int { kMatrixMemory = 0, kGatedDelta = 1, kLinearDecay = 2 };
constexpr int kThreads = 128;
constexpr int kMaxRegs = 16;   // key channels a thread holds of its column

struct ScanArgs {
  const float* qkv;            // [tokens, ld_qkv]: queries, keys (kv head major, D each) and values (head major, V each)
  long long ld_qkv;
  int q_off, k_off, v_off;
  const float* gates;          // [tokens, ld_gates]: matrix memory: zi at i_off + h, zf at f_off + h; delta: zb at i_off + h
  long long ld_gates;
  int i_off, f_off;
  const float* decay;          // delta: a [tokens, ld_decay], head major, D each
  long long ld_decay;
  const void* p0;              // matrix memory: bias of zi [H]; delta: dt [H * D]; linear decay: lambda [H]
  const void* p1;              // matrix memory: bias of zf [H]; delta: A [H]
  int p_dtype;
  float cap, q_scale;
  float* prep;                 // [tokens, H, rec]: what the scan reads per row and head (see recurrent_prepare_kernel)
  int rec;
  float* state;
  long long state_stride;      // floats between slots (two copies inside)
  const int* cu_seqlens;
  const int* token_req;
  const int* state_slots;
  const int* state_phase;
  float* out;                  // [tokens, ld_out], head major, V each
  long long ld_out;
  int tokens, H, G, D, V;
};

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// Everything of a row that does not depend on the rows before it, one warp per (row, head), so that the scan's loop is
// the recurrence alone. Record of rec >= 3 D + 2 floats: keys [D], queries [D], decays [D], two scalars, padding.
//   matrix memory: keys as they are, queries times q_scale, (no decays), the log gates i and f
//   delta rule:    unit keys, unit queries times q_scale, g = exp(-exp(A) softplus(a + dt)), beta
//   linear decay:  silu of the keys, silu of the queries times q_scale; the head's values get their silu in place
template <int kMode>
__global__ void recurrent_prepare_kernel(ScanArgs a) {
  pdl_start();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= a.tokens * a.H) return;
  const int t = warp / a.H, h = warp - t * a.H, D = a.D;
  const int g = h / (a.H / a.G);
  const float* r = a.qkv + (size_t)t * a.ld_qkv;
  float* rec = a.prep + ((size_t)t * a.H + h) * a.rec;
  const float* gr = a.gates + (size_t)t * a.ld_gates;
  if (kMode == kLinearDecay) {
    for (int d = lane; d < D; d += 32) {
      const float k = r[a.k_off + g * D + d], q = r[a.q_off + g * D + d];
      rec[d] = k / (1.f + expf(-k));
      rec[D + d] = q / (1.f + expf(-q)) * a.q_scale;
    }
    float* v = const_cast<float*>(r) + a.v_off + (size_t)h * a.V;      // only this warp touches the head's values of the row
    for (int c = lane; c < a.V; c += 32) v[c] = v[c] / (1.f + expf(-v[c]));
  } else if (kMode == kMatrixMemory) {
    for (int d = lane; d < D; d += 32) {
      rec[d] = r[a.k_off + g * D + d];
      rec[D + d] = r[a.q_off + g * D + d] * a.q_scale;
    }
    if (lane == 0) {
      const float zi = gr[a.i_off + h] + load_as_f32(a.p0, a.p_dtype, h), zf = gr[a.f_off + h] + load_as_f32(a.p1, a.p_dtype, h);
      const float fx = a.cap * tanhf(zf / a.cap);
      rec[3 * D] = a.cap * tanhf(zi / a.cap);
      rec[3 * D + 1] = fminf(fx, 0.f) - log1pf(expf(-fabsf(fx)));     // logsigmoid
    }
  } else {
    float k2 = 0.f, q2 = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float k = r[a.k_off + g * D + d], q = r[a.q_off + g * D + d];
      k2 += k * k;
      q2 += q * q;
    }
    k2 = warp_sum(k2);
    q2 = warp_sum(q2);
    const float kn = 1.f / sqrtf(k2 + 1e-6f), qn = a.q_scale / sqrtf(q2 + 1e-6f);
    const float rate = expf(load_as_f32(a.p1, a.p_dtype, h));
    for (int d = lane; d < D; d += 32) {
      rec[d] = r[a.k_off + g * D + d] * kn;
      rec[D + d] = r[a.q_off + g * D + d] * qn;
      const float x = a.decay[(size_t)t * a.ld_decay + (size_t)h * D + d] + load_as_f32(a.p0, a.p_dtype, (size_t)h * D + d);
      rec[2 * D + d] = expf(-rate * softplus_f(x));
    }
    if (lane == 0) rec[3 * D] = 1.f / (1.f + expf(-gr[a.i_off + h]));
  }
}

template <int kBytes>
__device__ __forceinline__ void cp_async(float* smem, const float* global) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  if (kBytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(global) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(global) : "memory");
}

template <int kLanes>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block (request, head, slice of kThreads / kLanes value columns): the request's rows of the step in order, the slice of
// C in registers (a column's D numbers spread over kLanes lanes, R each), the rows' records staged in shared memory a
// chunk at a time.
// Which key channel register i of lane j holds, and a row's D numbers into a thread's R registers. kVec4 (D a multiple of
// four): a lane holds runs of four neighbours, d = 4 (j + (i / 4) kLanes) + i % 4, and reads them 16 bytes at a time;
// otherwise d = j + i kLanes.
template <int kLanes, bool kVec4>
__device__ __forceinline__ int channel_of(int i, int j) {
  return kVec4 ? 4 * (j + (i >> 2) * kLanes) + (i & 3) : j + i * kLanes;
}
template <int kLanes, int R, bool kVec4>
__device__ __forceinline__ void load_channels(float (&dst)[R], const float* __restrict__ row, int D, int j) {
  if (kVec4) {
#pragma unroll
    for (int q = 0; q < R / 4; ++q) {
      const int d = 4 * (j + q * kLanes);
      const float4 v = d < D ? *reinterpret_cast<const float4*>(row + d) : make_float4(0.f, 0.f, 0.f, 0.f);
      dst[4 * q] = v.x, dst[4 * q + 1] = v.y, dst[4 * q + 2] = v.z, dst[4 * q + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int d = j + i * kLanes;
      dst[i] = d < D ? row[d] : 0.f;
    }
  }
}

template <int kMode, int kLanes, int R, bool kVec4>
__global__ void __launch_bounds__(kThreads) recurrent_scan_kernel(ScanArgs a, int chunk) {
  pdl_wait();    // no early trigger: the blocks of the kernel behind this one would wait on the SMs this latency-bound loop needs
  extern __shared__ __align__(16) float stage[];   // two buffers of [chunk][rec] records, then [chunk][cols] values
  constexpr int kCols = kThreads / kLanes;
  const int b = blockIdx.x, h = blockIdx.y;
  const int start = a.cu_seqlens[b], n_rows = a.cu_seqlens[b + 1] - start;
  if (n_rows <= 0 || a.token_req[start] < 0) return;    // a padding request of a recorded step owns no state
  const int j = threadIdx.x % kLanes, cl = threadIdx.x / kLanes;
  const int c = blockIdx.z * kCols + cl;
  const bool col = c < a.V;
  const int D = a.D, V = a.V, rec = a.rec;
  const int elems = D * V + (kMode == kMatrixMemory ? D + 1 : 0);
  const int phase = a.state_phase[b];
  const float* old = a.state + (size_t)a.state_slots[b] * a.state_stride + ((size_t)phase * a.H + h) * elems;
  float* fresh = a.state + (size_t)a.state_slots[b] * a.state_stride + ((size_t)(1 - phase) * a.H + h) * elems;
  float C[R], nn[R];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = channel_of<kLanes, kVec4>(i, j);
    C[i] = (col && d < D) ? old[(size_t)c * D + d] : 0.f;
    nn[i] = (kMode == kMatrixMemory && d < D) ? old[(size_t)D * V + d] : 0.f;
  }
  if (kMode == kMatrixMemory) m = old[(size_t)D * V + D];
  const float lam = kMode == kLinearDecay ? load_as_f32(a.p0, a.p_dtype, h) : 0.f;

  // two buffers: the next chunk's records are on their way (cp.async) while this one is worked on
  const int buf_floats = chunk * (rec + kCols);
  auto request = [&](int t0, int buf) {
    const int n = min(chunk, n_rows - t0), rec4 = rec / 4;
    float* st = stage + (size_t)buf * buf_floats;
    float* vl = st + (size_t)chunk * rec;
    for (int i = threadIdx.x; i < n * rec4; i += kThreads) {
      const int tt = i / rec4, e = (i - tt * rec4) * 4;
      cp_async<16>(st + (size_t)tt * rec + e, a.prep + ((size_t)(start + t0 + tt) * a.H + h) * rec + e);
    }
    for (int i = threadIdx.x; i < n * kCols; i += kThreads) {
      const int tt = i / kCols, cc = blockIdx.z * kCols + (i - tt * kCols);
      if (cc < V) cp_async<4>(vl + i, a.qkv + (size_t)(start + t0 + tt) * a.ld_qkv + a.v_off + h * V + cc);
      else vl[i] = 0.f;
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  request(0, 0);
  int turn = 0;
  for (int t0 = 0; t0 < n_rows; t0 += chunk, turn ^= 1) {
    const int n = min(chunk, n_rows - t0);
    if (t0 + chunk < n_rows) {
      request(t0 + chunk, turn ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const float* stage_now = stage + (size_t)turn * buf_floats;
    const float* vals = stage_now + (size_t)chunk * rec;
    int tt = 0;
    if (kMode == kGatedDelta) {
      // Two rows at a time. With A = g1 C (the state behind the first row's decay) everything the two rows need of the
      // state is four dot products with A that do not wait for one another:
      //   d1 = b1 (v1 - A^T k1),  o1 = A^T q1 + (k1 . q1) d1,
      //   d2 = b2 (v2 - (g2 A)^T k2 - ((g2 k1) . k2) d1),  o2 = (g2 A)^T q2 + ((g2 k1) . q2) d1 + (k2 . q2) d2,
      //   C <- g2 A + (g2 k1) d1 + k2 d2,
      // so the chain from state to state holds one tree of shuffles a pair instead of two a row.
      for (; tt + 1 < n; tt += 2) {
        const float* r1 = stage_now + (size_t)tt * rec;
        const float* r2 = r1 + rec;
        const float v1 = vals[tt * kCols + cl], v2 = vals[(tt + 1) * kCols + cl];
        const float b1 = r1[3 * D], b2 = r2[3 * D];
        float k1[R], q1[R], k2[R], q2[R], g[R];
        load_channels<kLanes, R, kVec4>(g, r1 + 2 * D, D, j);
        load_channels<kLanes, R, kVec4>(k1, r1, D, j);
        load_channels<kLanes, R, kVec4>(q1, r1 + D, D, j);
        float ak1[4] = {0.f, 0.f, 0.f, 0.f}, aq1[4] = {0.f, 0.f, 0.f, 0.f}, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] *= g[i];
          ak1[i & 3] += C[i] * k1[i];
          aq1[i & 3] += C[i] * q1[i];
          s1 += k1[i] * q1[i];
        }
        load_channels<kLanes, R, kVec4>(g, r2 + 2 * D, D, j);
        load_channels<kLanes, R, kVec4>(k2, r2, D, j);
        load_channels<kLanes, R, kVec4>(q2, r2 + D, D, j);
        float ak2[4] = {0.f, 0.f, 0.f, 0.f}, aq2[4] = {0.f, 0.f, 0.f, 0.f}, s2 = 0.f, s3 = 0.f, s4 = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] *= g[i];                 // g2 A
          k1[i] *= g[i];                // g2 k1
          ak2[i & 3] += C[i] * k2[i];
          aq2[i & 3] += C[i] * q2[i];
          s2 += k1[i] * k2[i];
          s3 += k1[i] * q2[i];
          s4 += k2[i] * q2[i];
        }
        const float A_k1 = lanes_sum<kLanes>((ak1[0] + ak1[1]) + (ak1[2] + ak1[3]));
        const float A_q1 = lanes_sum<kLanes>((aq1[0] + aq1[1]) + (aq1[2] + aq1[3]));
        const float A_k2 = lanes_sum<kLanes>((ak2[0] + ak2[1]) + (ak2[2] + ak2[3]));
        const float A_q2 = lanes_sum<kLanes>((aq2[0] + aq2[1]) + (aq2[2] + aq2[3]));
        s1 = lanes_sum<kLanes>(s1), s2 = lanes_sum<kLanes>(s2), s3 = lanes_sum<kLanes>(s3), s4 = lanes_sum<kLanes>(s4);
        const float d1 = b1 * (v1 - A_k1);
        const float d2 = b2 * (v2 - (A_k2 + s2 * d1));
#pragma unroll
        for (int i = 0; i < R; ++i) C[i] += k1[i] * d1 + k2[i] * d2;
        if (j == 0 && col) {
          float* o_row = a.out + (size_t)(start + t0 + tt) * a.ld_out + (size_t)h * V + c;
          o_row[0] = A_q1 + s1 * d1;
          o_row[a.ld_out] = A_q2 + s3 * d1 + s4 * d2;
        }
      }
    }
    if (kMode == kLinearDecay) {
      // Four rows at a time. The read-out does not feed the state, so the chain from row to row is one multiply-add a
      // register; the four rows' sums over the lanes of a column are four shuffle trees that do not wait for one another.
      for (; tt + 3 < n; tt += 4) {
        float o4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float* r = stage_now + (size_t)(tt + u) * rec;
          const float v = vals[(tt + u) * kCols + cl];
          float k[R], q[R];
          load_channels<kLanes, R, kVec4>(k, r, D, j);
          load_channels<kLanes, R, kVec4>(q, r + D, D, j);
          float num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < R; ++i) {
            C[i] = fmaf(lam, C[i], k[i] * v);
            num[i & 3] += C[i] * q[i];
          }
          o4[u] = (num[0] + num[1]) + (num[2] + num[3]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) o4[u] = lanes_sum<kLanes>(o4[u]);
        if (j == 0 && col) {
          float* o_row = a.out + (size_t)(start + t0 + tt) * a.ld_out + (size_t)h * V + c;
#pragma unroll
          for (int u = 0; u < 4; ++u) o_row[(size_t)u * a.ld_out] = o4[u];
        }
      }
    }
#pragma unroll 2
    for (; tt < n; ++tt) {
      const float* r = stage_now + (size_t)tt * rec;
      const float v = vals[tt * kCols + cl];
      float o;
      if (kMode == kMatrixMemory) {
        const float gi = r[3 * D], gf = r[3 * D + 1];
        const float m_new = fmaxf(gf + m, gi);
        const float keep = expf(gf + m - m_new), put = expf(gi - m_new);
        m = m_new;
        float k[R], q[R];
        load_channels<kLanes, R, kVec4>(k, r, D, j);
        load_channels<kLanes, R, kVec4>(q, r + D, D, j);
        float num[4] = {0.f, 0.f, 0.f, 0.f}, nq[4] = {0.f, 0.f, 0.f, 0.f};     // four partial sums: short dependent chains
        const float pv = put * v;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] = keep * C[i] + pv * k[i];
          nn[i] = keep * nn[i] + put * k[i];
          num[i & 3] += C[i] * q[i];
          nq[i & 3] += nn[i] * q[i];
        }
        const float ns = lanes_sum<kLanes>((num[0] + num[1]) + (num[2] + num[3]));
        const float qs = lanes_sum<kLanes>((nq[0] + nq[1]) + (nq[2] + nq[3]));
        o = ns / (fmaxf(fabsf(qs), expf(-m)) + 1e-6f);
      } else if (kMode == kLinearDecay) {
        // the read-out does not feed the state: the chain from row to row is one multiply-add a register
        float k[R], q[R];
        load_channels<kLanes, R, kVec4>(k, r, D, j);
        load_channels<kLanes, R, kVec4>(q, r + D, D, j);
        float num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] = fmaf(lam, C[i], k[i] * v);
          num[i & 3] += C[i] * q[i];
        }
        o = lanes_sum<kLanes>((num[0] + num[1]) + (num[2] + num[3]));
      } else {
        const float beta = r[3 * D];
        float k[R], g[R], q[R];
        load_channels<kLanes, R, kVec4>(k, r, D, j);
        load_channels<kLanes, R, kVec4>(g, r + 2 * D, D, j);
        float kv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] *= g[i];
          kv[i & 3] += C[i] * k[i];
        }
        load_channels<kLanes, R, kVec4>(q, r + D, D, j);
        const float dlt = beta * (v - lanes_sum<kLanes>((kv[0] + kv[1]) + (kv[2] + kv[3])));
        float num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R; ++i) {
          C[i] += k[i] * dlt;
          num[i & 3] += C[i] * q[i];
        }
        o = lanes_sum<kLanes>((num[0] + num[1]) + (num[2] + num[3]));
      }
      if (j == 0 && col) a.out[(size_t)(start + t0 + tt) * a.ld_out + (size_t)h * V + c] = o;
    }
    __syncthreads();                           // everyone has read this buffer before the chunk after next is requested into it
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = channel_of<kLanes, kVec4>(i, j);
    if (col && d < D) fresh[(size_t)c * D + d] = C[i];
    if (kMode == kMatrixMemory && blockIdx.z == 0 && cl == 0 && d < D) fresh[(size_t)D * V + d] = nn[i];
  }
  if (kMode == kMatrixMemory && blockIdx.z == 0 && threadIdx.x == 0) fresh[(size_t)D * V + D] = m;
}

// out[t, h, c] = o[t, h, c] * rsqrt(mean_c o[t, h, :]^2 + eps) * w[h * w_stride + c] * sigmoid(gate[t, h, c]) * scale:
// the per-head unit norm, the weight and the output gate of a recurrent mixer, one warp per (row, head).
template <typename TO>
__global__ void head_norm_gate_kernel(TO* __restrict__ out, long long ld_out, const float* __restrict__ o, long long ld_o,
                                      const float* __restrict__ gate, long long ld_gate, const void* __restrict__ w,
                                      int w_dtype, int w_stride, int tokens, int H, int V, float eps, float scale) {
  pdl_start();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* row = o + (size_t)t * ld_o + (size_t)h * V;
  float ss = 0.f;
  for (int c = lane; c < V; c += 32) ss += row[c] * row[c];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)V + eps);
  for (int c = lane; c < V; c += 32) {
    const float gz = gate[(size_t)t * ld_gate + (size_t)h * V + c];
    const float val = row[c] * r * load_as_f32(w, w_dtype, (size_t)h * w_stride + c) * (1.f / (1.f + expf(-gz))) * scale;
    out[(size_t)t * ld_out + (size_t)h * V + c] = from_f32<TO>(val);
  }
}

// The same for ONE norm over a whole row of many numbers (H = 1: a norm over all heads together): one block a row.
template <typename TO>
__global__ void row_norm_gate_kernel(TO* __restrict__ out, long long ld_out, const float* __restrict__ o, long long ld_o,
                                     const float* __restrict__ gate, long long ld_gate, const void* __restrict__ w, int w_dtype,
                                     int V, float eps, float scale) {
  pdl_start();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * ld_o;
  float ss = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) ss += row[c] * row[c];
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)V + eps);
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    const float gz = gate[(size_t)t * ld_gate + c];
    out[(size_t)t * ld_out + c] = from_f32<TO>(row[c] * r * load_as_f32(w, w_dtype, c) * (1.f / (1.f + expf(-gz))) * scale);
  }
}

}  // namespace

// floats of scratch the scan wants per row: oi_recurrent_scan's `prep` is [tokens, H, that]
OI_API int oi_recurrent_record(int D) { return (3 * D + 2 + 3) & ~3; }   // a multiple of four floats: 16-byte copies

// mode 0: matrix memory (p0, p1: the two gate biases [H]); mode 1: gated delta rule (p0: dt [H * D], p1: A [H];
// decay: a [tokens, ld_decay]); mode 2: linear attention with a fixed decay per head (p0: lambda [H]; qkv is written: the
// values get their silu in place). State: [slots][2][H][D * V (+ D + 1 in mode 0)] floats. prep: scratch, see above.
OI_API int oi_recurrent_scan(int mode, const float* qkv, long long ld_qkv, int q_off, int k_off, int v_off, const float* gates,
                             long long ld_gates, int i_off, int f_off, const float* decay, long long ld_decay, const void* p0,
                             const void* p1, int p_dtype, float cap, float q_scale, float* prep, float* state,
                             long long state_stride, const int* cu_seqlens, const int* token_req, const int* state_slots,
                             const int* state_phase, float* out, long long ld_out, int tokens, int requests, int H, int G, int D,
                             int V, void* stream) {
  OI_REQUIRE(mode == kMatrixMemory || mode == kGatedDelta || mode == kLinearDecay, "recurrent_scan: unknown mode %d", mode);
  OI_REQUIRE(requests >= 0 && tokens >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0,
             "recurrent_scan: bad sizes H=%d G=%d D=%d V=%d", H, G, D, V);
  OI_REQUIRE(D <= 32 * kMaxRegs, "recurrent_scan: %d key channels per head, at most %d", D, 32 * kMaxRegs);
  OI_REQUIRE(mode != kGatedDelta || decay != nullptr, "recurrent_scan: the delta rule needs its decays");
  OI_REQUIRE(prep != nullptr, "recurrent_scan: the scratch for the rows' records is missing");
  const long long elems = (long long)D * V + (mode == kMatrixMemory ? D + 1 : 0);
  OI_REQUIRE(state != nullptr && state_stride >= 2 * H * elems, "recurrent_scan: the state needs two copies of %lld floats per head", elems);
  if (requests == 0 || tokens == 0) return OI_OK;
  ScanArgs a;
  a.qkv = qkv, a.ld_qkv = ld_qkv, a.q_off = q_off, a.k_off = k_off, a.v_off = v_off;
  a.gates = gates, a.ld_gates = ld_gates, a.i_off = i_off, a.f_off = f_off;
  a.decay = decay, a.ld_decay = ld_decay, a.p0 = p0, a.p1 = p1, a.p_dtype = p_dtype, a.cap = cap, a.q_scale = q_scale;
  a.prep = prep, a.rec = oi_recurrent_record(D);
  a.state = state, a.state_stride = state_stride, a.cu_seqlens = cu_seqlens, a.token_req = token_req;
  a.state_slots = state_slots, a.state_phase = state_phase, a.out = out, a.ld_out = ld_out;
  a.tokens = tokens, a.H = H, a.G = G, a.D = D, a.V = V;
  cudaStream_t s = (cudaStream_t)stream;
  const int warps = tokens * H;
  if (mode == kMatrixMemory) oi_launch(recurrent_prepare_kernel<kMatrixMemory>, (warps + 3) / 4, 128, 0, s, a);
  else if (mode == kLinearDecay) oi_launch(recurrent_prepare_kernel<kLinearDecay>, (warps + 3) / 4, 128, 0, s, a);
  else oi_launch(recurrent_prepare_kernel<kGatedDelta>, (warps + 3) / 4, 128, 0, s, a);
  OI_CHECK_LAUNCH();
  // rows per buffer: two buffers of at most 13 KB; the linear decay, which walks four rows at a time, takes more (up to 44 KB)
  const int chunk = mode == kLinearDecay ? (D <= 64 ? 24 : (D <= 128 ? 12 : (D <= 256 ? 4 : 2)))
                                         : (D <= 64 ? 16 : (D <= 128 ? 8 : (D <= 256 ? 4 : 2)));
#define OI_SCAN_AS(MODE, LANES, REGS)                                                                                   \
  do {                                                                                                                  \
    constexpr int cols = kThreads / LANES;                                                                              \
    const dim3 grid(requests, H, (V + cols - 1) / cols);                                                                \
    const size_t smem = 2 * (size_t)chunk * (a.rec + cols) * sizeof(float);                                                 \
    /* plain stream order: launched early, the few long-lived blocks would be packed onto the SMs that the kernel */     \
    /* before frees first and share their issue slots (measured 2.1 against 0.9 ms for 2,048 rows) */                   \
    oi_fence_next_launch();                                                                                              \
    if (D % 4 == 0) oi_launch(recurrent_scan_kernel<MODE, LANES, REGS, true>, grid, kThreads, smem, s, a, chunk);        \
    else oi_launch(recurrent_scan_kernel<MODE, LANES, REGS, false>, grid, kThreads, smem, s, a, chunk);                 \
  } while (0)
  // (a column over 32 lanes of four registers instead of 8 of sixteen: 0.84 against 0.79 ms for 2,048 rows of 128 channels:
  // the deeper shuffle tree costs what the shorter loops save)
#define OI_SCAN(MODE)                                 \
  do {                                                \
    if (D <= 16) OI_SCAN_AS(MODE, 4, 4);              \
    else if (D <= 64) OI_SCAN_AS(MODE, 4, 16);        \
    else if (D <= 128) OI_SCAN_AS(MODE, 8, 16);       \
    else if (D <= 256) OI_SCAN_AS(MODE, 16, 16);      \
    else OI_SCAN_AS(MODE, 32, 16);                    \
  } while (0)
  // (the linear decay's sums over a column's lanes are off the chain from row to row: more lanes a column, fewer columns a
  // block and so more blocks)
  if (mode == kMatrixMemory) OI_SCAN(kMatrixMemory);
  else if (mode == kLinearDecay) {
    if (D <= 16) OI_SCAN_AS(kLinearDecay, 4, 4);
    else if (D <= 32) OI_SCAN_AS(kLinearDecay, 8, 4);
    else if (D <= 64) OI_SCAN_AS(kLinearDecay, 16, 4);
    else if (D <= 128) OI_SCAN_AS(kLinearDecay, 16, 8);   // (32 lanes of four registers, twice the blocks: 422 against 357 us for 2,048 rows)
    else if (D <= 256) OI_SCAN_AS(kLinearDecay, 32, 8);
    else OI_SCAN_AS(kLinearDecay, 32, 16);
  } else OI_SCAN(kGatedDelta);
#undef OI_SCAN
#undef OI_SCAN_AS
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_head_norm_gate(void* out, int out_dtype, long long ld_out, const float* o, long long ld_o, const float* gate,
                             long long ld_gate, const void* w, int w_dtype, int w_stride, int tokens, int H, int V, float eps,
                             float scale, void* stream) {
  OI_REQUIRE(tokens >= 0 && H > 0 && V > 0, "head_norm_gate: bad sizes");
  if (tokens == 0) return OI_OK;
  const int warps = tokens * H, blocks = (warps + 7) / 8;
  cudaStream_t s = (cudaStream_t)stream;
  if (H == 1 && V >= 256 && (out_dtype == OI_F32 || out_dtype == OI_BF16)) {     // one long row: a block a row, not a warp
    const int threads = V >= 1024 ? 256 : 128;
    if (out_dtype == OI_F32)
      oi_launch(row_norm_gate_kernel<float>, tokens, threads, 0, s, (float*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, V, eps, scale);
    else
      oi_launch(row_norm_gate_kernel<bf16>, tokens, threads, 0, s, (bf16*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, V, eps, scale);
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  if (out_dtype == OI_F32)
    oi_launch(head_norm_gate_kernel<float>, blocks, 256, 0, s, (float*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, w_stride, tokens, H, V, eps, scale);
  else if (out_dtype == OI_BF16)
    oi_launch(head_norm_gate_kernel<bf16>, blocks, 256, 0, s, (bf16*)out, ld_out, o, ld_o, gate, ld_gate, w, w_dtype, w_stride, tokens, H, V, eps, scale);
  else
    OI_REQUIRE(false, "head_norm_gate: unknown dtype code %d", out_dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
