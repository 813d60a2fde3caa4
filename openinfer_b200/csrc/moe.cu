// Routed experts: a feed-forward of `experts` small gated layers of which every row uses `top`.
//
//   1. moe_router_kernel   z = W_r x in float32 (one block a row), the `top` largest logits (ties to the lower index),
//                          their softmax -> ids [rows, top], weights [rows, top]. Scoring 1 ("sigmoid, corrected, by groups"):
//                          s = sigmoid(z); the choice goes by s + correction, among the experts of the `keep_groups` best of
//                          `n_groups` equal groups of neighbours (a group's score: the sum of its two largest choice scores);
//                          the weights are the chosen experts' s divided by their sum (+ 1e-20)
//   2. moe_group_kernel    the (row, choice) pairs sorted by expert (stable, so the order never depends on timing), and
//                          the list of row tiles (expert, first sorted place, rows) the products run over
//   3. moe_gemm_kernel     per tile: act(x W_gate_e^T, x W_up_e^T) for the rows of the tile, gathered by their pair's row;
//                          then the down projection, each row written to its pair's place
//   4. moe_combine_kernel  out[row] = sum_j weight[row, j] * y[row * top + j], j ascending
//
// Steps of few rows (at most two pairs an expert on average) skip 2 and run 3 pair by pair (moe_gemv_kernel: a warp per
// output row, the expert's rows read 16 bytes at a time); larger steps take the tiles.
// Everything a step needs is found on the device (no sizes travel back to the host), so a step of single tokens can be
// recorded and replayed. A row's sums are formed in the same order whatever else shares its tile: the result of a row does
// not depend on the batch. The tiles' products run on the tensor cores for bfloat16 operands (mma.sync, float32
// accumulation) and on the ordinary pipes for float32 and for rows that cannot be read 16 bytes at a time.
#include "common.cuh"

namespace {

constexpr int kTileM = 32, kTileN = 64, kTileK = 32;
constexpr int kMaxTop = 32;

template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ x, long long ldx, const void* __restrict__ w, int w_dtype, int rows, int K,
                                  int E, int top, int* __restrict__ ids, float* __restrict__ wts, int scoring,
                                  const float* __restrict__ correction, int n_groups, int keep_groups) {
  pdl_start();
  extern __shared__ float smem[];              // the row's logits [E], scores [E], group scores [E], then which are taken [E bytes]
  const int warps = blockDim.x >> 5, wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* z = smem;
  float* sc = smem + E;
  float* gs = smem + 2 * E;
  unsigned char* taken = reinterpret_cast<unsigned char*>(smem + 3 * E);
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * ldx;
  constexpr int kVec = 16 / (int)sizeof(T);
  const bool vec = w_dtype == (sizeof(T) == 2 ? OI_BF16 : OI_F32) && K % kVec == 0 && ldx % kVec == 0 && (uintptr_t)x % 16 == 0 &&
                   (uintptr_t)w % 16 == 0;
  // one block a row; a warp takes four experts at a time, so that their loads are in flight together
  for (int e0 = wi * 4; e0 < E; e0 += warps * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec) {       // a lane takes 16 bytes of the row and of each expert's weights at a time
      const T* wt = reinterpret_cast<const T*>(w);
      // (experts beyond the last read the last one's row again and are not stored: loads without a condition can all be
      // in flight at once, where a load behind a test waits for the one before it: 8 rows of width 2,048 21.8 -> 8.2 us)
      const T* wrow[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) wrow[i] = wt + (size_t)min(e0 + i, E - 1) * K;
#pragma unroll 2
      for (int k = lane * kVec; k < K; k += 32 * kVec) {
        T xv[kVec], wv[4][kVec];
        *reinterpret_cast<uint4*>(xv) = *reinterpret_cast<const uint4*>(xr + k);
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(wv[i]) = *reinterpret_cast<const uint4*>(wrow[i] + k);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < kVec; ++e) acc[i] += to_f32(wv[i][e]) * to_f32(xv[e]);
      }
    } else {
#pragma unroll 4
      for (int k = lane; k < K; k += 32) {
        const float xv = to_f32(xr[k]);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (e0 + i < E) acc[i] += load_as_f32(w, w_dtype, (size_t)(e0 + i) * K + k) * xv;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sum = warp_sum(acc[i]);
      if (lane == 0 && e0 + i < E) {
        z[e0 + i] = sum;
        taken[e0 + i] = 0;
      }
    }
  }
  __syncthreads();
  if (wi != 0) return;
  if (scoring == 1) {
    for (int e = lane; e < E; e += 32) {
      const float sg = 1.f / (1.f + expf(-z[e]));
      sc[e] = sg;
      z[e] = sg + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
      const int per = E / n_groups;
      for (int g = lane; g < n_groups; g += 32) {
        float a = -INFINITY, b = -INFINITY;          // the group's two largest choice scores
        for (int i = 0; i < per; ++i) {
          const float v = z[g * per + i];
          if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
        }
        gs[g] = per > 1 ? a + b : a;
      }
      __syncwarp();
      for (int e = lane; e < E; e += 32) taken[e] = 1;
      __syncwarp();
      for (int kept = 0; kept < keep_groups; ++kept) {
        float best = -INFINITY;
        int bg = 0x7fffffff;
        // (a group is kept already when its experts are open; the first open candidate stands whatever its score is, so
        // that rows of a padded step, whose numbers mean nothing and may be NaN, still name experts that exist)
        for (int g = lane; g < n_groups; g += 32) {
          const float v = gs[g];
          if (taken[g * per] && (bg == 0x7fffffff || v > best)) { best = v; bg = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, o);
          const int og = __shfl_xor_sync(0xffffffffu, bg, o);
          if (og != 0x7fffffff && (bg == 0x7fffffff || ov > best || (ov == best && og < bg))) { best = ov; bg = og; }
        }
        if (bg == 0x7fffffff) break;
        for (int i = lane; i < per; i += 32) taken[bg * per + i] = 0;
        __syncwarp();
      }
    }
  }
  float chosen_z[kMaxTop];
  int chosen_e[kMaxTop];
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      if (taken[e]) continue;
      const float v = z[e];
      if (be == 0x7fffffff || v > best) {
        best = v;
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > best || (ov == best && oe < be))) {
        best = ov;
        be = oe;
      }
    }
    if (be >= E) be = j;          // nothing open (cannot happen with sizes the entry point accepts): still an expert that exists
    if (lane == 0) taken[be] = 1;
    __syncwarp();
    chosen_z[j] = best;
    chosen_e[j] = be;
  }
  if (lane == 0 && scoring == 1) {
    float sum = 0.f;
    for (int j = 0; j < top; ++j) sum += sc[chosen_e[j]];
    for (int j = 0; j < top; ++j) {
      ids[(size_t)row * top + j] = chosen_e[j];
      wts[(size_t)row * top + j] = sc[chosen_e[j]] / (sum + 1e-20f);
    }
  } else if (lane == 0) {
    float mx = chosen_z[0], sum = 0.f;
    for (int j = 1; j < top; ++j) mx = fmaxf(mx, chosen_z[j]);
    for (int j = 0; j < top; ++j) {
      chosen_z[j] = expf(chosen_z[j] - mx);
      sum += chosen_z[j];
    }
    for (int j = 0; j < top; ++j) {
      ids[(size_t)row * top + j] = chosen_e[j];
      wts[(size_t)row * top + j] = chosen_z[j] / sum;
    }
  }
}

// One block per expert e. sorted[first_e + i] = the i-th pair (in ascending pair number) that chose e; tiles of tile_m
// sorted places that belong to one expert: tile_info[3 * t] = expert, first place, rows. tile_info's last word
// (at 3 * max_tiles) is the number of tiles.
__global__ void moe_group_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ sorted, int* __restrict__ tile_info,
                                 int max_tiles, int tile_m) {
  pdl_start();
  extern __shared__ int hist[];       // [E] counts, then [warps] scan scratch
  __shared__ int s_first, s_tile0, s_count;
  const int e = blockIdx.x;
  for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int id = ids[p];
    if (id >= 0 && id < E) atomicAdd(&hist[id], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int first = 0, tile0 = 0, total = 0;
    for (int i = 0; i < E; ++i) {
      const int tiles = (hist[i] + tile_m - 1) / tile_m;
      if (i < e) {
        first += hist[i];
        tile0 += tiles;
      }
      total += tiles;
    }
    s_first = first, s_tile0 = tile0, s_count = hist[e];
    if (e == 0) tile_info[3 * max_tiles] = total < max_tiles ? total : max_tiles;
  }
  __syncthreads();
  const int first = s_first, tile0 = s_tile0, count = s_count;
  for (int t = threadIdx.x; t * tile_m < count; t += blockDim.x) {
    if (tile0 + t < max_tiles) {
      tile_info[3 * (tile0 + t)] = e;
      tile_info[3 * (tile0 + t) + 1] = first + t * tile_m;
      tile_info[3 * (tile0 + t) + 2] = count - t * tile_m < tile_m ? count - t * tile_m : tile_m;
    }
  }
  // stable compaction of the pairs that chose e
  int* wsum = hist + E;
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, warps = blockDim.x >> 5;
  int running = 0;
  for (int base = 0; base < pairs; base += blockDim.x) {
    const int p = base + threadIdx.x;
    const bool mine = p < pairs && ids[p] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    __syncthreads();
    if (lane == 0) wsum[wi] = __popc(ballot);
    __syncthreads();
    int before = 0, all = 0;
    for (int w = 0; w < warps; ++w) {
      if (w < wi) before += wsum[w];
      all += wsum[w];
    }
    if (mine) sorted[first + running + before + __popc(ballot & ((1u << lane) - 1))] = p;
    running += all;
  }
}

// out rows of one tile: C[i, n] = sum_k A[src(i), k] * W_e[n, k] (k ascending), i over the tile's sorted places.
// kGlu: W_e holds N gate rows and then N up rows; the result is the gated activation `act` of the two sums (glu_act:
// act(g) * u, or with OI_ACT_SWIGLU_CLAMP g' sigmoid(1.702 g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)). a_div: the source row of place i is sorted[i] / a_div (a_div 0: the place itself).
// scatter: the result of place i goes to row sorted[i] (else to row i).
template <typename T, typename TO, bool kGlu>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const T* __restrict__ A, long long lda, int a_div, const T* __restrict__ Wt,
                                                       long long w_expert_stride, TO* __restrict__ out, long long ld_out, int scatter,
                                                       const int* __restrict__ sorted, const int* __restrict__ tile_info,
                                                       int max_tiles, int N, int K, float limit, int act) {
  pdl_wait();    // no early trigger: waiting blocks of the next kernel would share the SMs with this product
  const int tile = blockIdx.x;
  if (tile >= tile_info[3 * max_tiles]) return;
  // a block takes kTileM rows: of a longer tile, the part that blockIdx.z names
  const int e = tile_info[3 * tile], place0 = tile_info[3 * tile + 1] + (int)blockIdx.z * kTileM;
  const int m_rows = min(tile_info[3 * tile + 2] - (int)blockIdx.z * kTileM, kTileM);
  if (m_rows <= 0) return;
  const int n0 = blockIdx.y * kTileN;
  __shared__ float As[kTileK][kTileM + 1];
  __shared__ float Wg[kTileK][kTileN + 1];
  __shared__ float Wu[kGlu ? kTileK : 1][kTileN + 1];
  __shared__ int src[kTileM];
  if (threadIdx.x < kTileM) {
    int r = -1;
    if ((int)threadIdx.x < m_rows) {
      const int place = place0 + threadIdx.x;
      r = a_div > 0 ? sorted[place] / a_div : place;
    }
    src[threadIdx.x] = r;
  }
  __syncthreads();
  const T* We = Wt + (size_t)e * w_expert_stride;
  const int tn = threadIdx.x % 16, tm = threadIdx.x / 16;   // thread: rows tm, tm + 16; columns tn + 16 j, j < 4
  float acc[2][4] = {}, accu[2][4] = {};
  // operands that can be read 16 bytes at a time (rows that start on 16-byte boundaries, K a multiple of the vector)
  constexpr int kVec = 16 / (int)sizeof(T);
  const bool vec = K % kVec == 0 && lda % kVec == 0 && ((uintptr_t)A % 16 == 0) && ((uintptr_t)We % 16 == 0) &&
                   ((size_t)N * K) % kVec == 0;
  for (int k0 = 0; k0 < K; k0 += kTileK) {
    if (vec) {
      constexpr int kChunks = kTileK / kVec;     // 16-byte pieces of a tile's row
      for (int i = threadIdx.x; i < kTileM * kChunks; i += 256) {
        const int m = i / kChunks, k = (i % kChunks) * kVec;
        const int r = src[m];
        T v[kVec] = {};
        if (r >= 0 && k0 + k < K) *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(A + (size_t)r * lda + k0 + k);
#pragma unroll
        for (int e = 0; e < kVec; ++e) As[k + e][m] = (r >= 0 && k0 + k < K) ? to_f32(v[e]) : 0.f;
      }
      for (int i = threadIdx.x; i < kTileN * kChunks; i += 256) {
        const int n = i / kChunks, k = (i % kChunks) * kVec;
        const bool ok = n0 + n < N && k0 + k < K;
        T v[kVec] = {}, u[kVec] = {};
        if (ok) {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(We + (size_t)(n0 + n) * K + k0 + k);
          if (kGlu) *reinterpret_cast<uint4*>(u) = *reinterpret_cast<const uint4*>(We + (size_t)(N + n0 + n) * K + k0 + k);
        }
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          Wg[k + e][n] = ok ? to_f32(v[e]) : 0.f;
          if (kGlu) Wu[k + e][n] = ok ? to_f32(u[e]) : 0.f;
        }
      }
    } else {
      for (int i = threadIdx.x; i < kTileM * kTileK; i += 256) {
        const int m = i / kTileK, k = i % kTileK;
        const int r = src[m];
        As[k][m] = (r >= 0 && k0 + k < K) ? to_f32(A[(size_t)r * lda + k0 + k]) : 0.f;
      }
      for (int i = threadIdx.x; i < kTileN * kTileK; i += 256) {
        const int n = i / kTileK, k = i % kTileK;
        const bool ok = n0 + n < N && k0 + k < K;
        Wg[k][n] = ok ? to_f32(We[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
        if (kGlu) Wu[k][n] = ok ? to_f32(We[(size_t)(N + n0 + n) * K + k0 + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTileK; ++k) {
      const float a0 = As[k][tm], a1 = As[k][tm + 16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w = Wg[k][tn + 16 * j];
        acc[0][j] += a0 * w;
        acc[1][j] += a1 * w;
        if (kGlu) {
          const float u = Wu[k][tn + 16 * j];
          accu[0][j] += a0 * u;
          accu[1][j] += a1 * u;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = tm + 16 * i;
    if (m >= m_rows) continue;
    const int place = place0 + m;
    const size_t row = scatter ? (size_t)sorted[place] : (size_t)place;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + 16 * j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (kGlu) {
        v = glu_act<false>(v, accu[i][j], act, limit);
      }
      out[row * ld_out + n] = from_f32<TO>(v);
    }
  }
}

// The tiles' products on the tensor cores for bfloat16 operands that can be read 16 bytes at a time (mma.sync m16n8k16,
// float32 accumulation): 8 warps, warp w the 16 rows (w & 1) x the 16 columns (w >> 1) of the 32 x 64 tile (and the same
// columns of the up rows). Operand tiles lie in shared memory as they lie in global memory (rows of 32 k, padded to 40).
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const unsigned (&a)[4], const unsigned (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename TO, bool kGlu>
__global__ void __launch_bounds__(256) moe_gemm_mma_kernel(const bf16* __restrict__ A, long long lda, int a_div, const bf16* __restrict__ Wt,
                                                           long long w_expert_stride, TO* __restrict__ out, long long ld_out,
                                                           int scatter, const int* __restrict__ sorted,
                                                           const int* __restrict__ tile_info, int max_tiles, int N, int K, float limit, int act) {
  pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= tile_info[3 * max_tiles]) return;
  // a block takes kTileM rows: of a longer tile, the part that blockIdx.z names
  const int e = tile_info[3 * tile], place0 = tile_info[3 * tile + 1] + (int)blockIdx.z * kTileM;
  const int m_rows = min(tile_info[3 * tile + 2] - (int)blockIdx.z * kTileM, kTileM);
  if (m_rows <= 0) return;
  const int n0 = blockIdx.y * kTileN;
  constexpr int kPad = kTileK + 8;
  __shared__ __align__(16) bf16 As[kTileM][kPad];
  __shared__ __align__(16) bf16 Bg[kTileN][kPad];
  __shared__ __align__(16) bf16 Bu[kGlu ? kTileN : 1][kPad];
  __shared__ int src[kTileM];
  if (threadIdx.x < kTileM) {
    int r = -1;
    if ((int)threadIdx.x < m_rows) {
      const int place = place0 + threadIdx.x;
      r = a_div > 0 ? sorted[place] / a_div : place;
    }
    src[threadIdx.x] = r;
  }
  __syncthreads();
  const bf16* We = Wt + (size_t)e * w_expert_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int wm = (warp & 1) * 16, wn = (warp >> 1) * 16;
  float acc[2][4] = {}, accu[2][4] = {};
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int k0 = 0; k0 < K; k0 += kTileK) {
    if (threadIdx.x < kTileM * 4) {
      const int m = threadIdx.x >> 2, k = (threadIdx.x & 3) * 8;
      const int r = src[m];
      *reinterpret_cast<uint4*>(&As[m][k]) = (r >= 0 && k0 + k < K) ? *reinterpret_cast<const uint4*>(A + (size_t)r * lda + k0 + k) : zero;
    }
    {
      const int n = threadIdx.x >> 2, k = (threadIdx.x & 3) * 8;
      const bool ok = n0 + n < N && k0 + k < K;
      *reinterpret_cast<uint4*>(&Bg[n][k]) = ok ? *reinterpret_cast<const uint4*>(We + (size_t)(n0 + n) * K + k0 + k) : zero;
      if (kGlu) *reinterpret_cast<uint4*>(&Bu[n][k]) = ok ? *reinterpret_cast<const uint4*>(We + (size_t)(N + n0 + n) * K + k0 + k) : zero;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; kk += 16) {
      unsigned a[4];
      a[0] = *reinterpret_cast<const unsigned*>(&As[wm + g][kk + 2 * tg]);
      a[1] = *reinterpret_cast<const unsigned*>(&As[wm + g + 8][kk + 2 * tg]);
      a[2] = *reinterpret_cast<const unsigned*>(&As[wm + g][kk + 2 * tg + 8]);
      a[3] = *reinterpret_cast<const unsigned*>(&As[wm + g + 8][kk + 2 * tg + 8]);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        unsigned b[2];
        b[0] = *reinterpret_cast<const unsigned*>(&Bg[wn + 8 * j + g][kk + 2 * tg]);
        b[1] = *reinterpret_cast<const unsigned*>(&Bg[wn + 8 * j + g][kk + 2 * tg + 8]);
        mma_bf16_16816(acc[j], a, b);
        if (kGlu) {
          b[0] = *reinterpret_cast<const unsigned*>(&Bu[wn + 8 * j + g][kk + 2 * tg]);
          b[1] = *reinterpret_cast<const unsigned*>(&Bu[wn + 8 * j + g][kk + 2 * tg + 8]);
          mma_bf16_16816(accu[j], a, b);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int m = wm + g + (c >> 1) * 8, n = n0 + wn + 8 * j + 2 * tg + (c & 1);
      if (m >= m_rows || n >= N) continue;
      const int place = place0 + m;
      const size_t row = scatter ? (size_t)sorted[place] : (size_t)place;
      float v = acc[j][c];
      if (kGlu) {
        v = glu_act<false>(v, accu[j][c], act, limit);
      }
      out[row * ld_out + n] = from_f32<TO>(v);
    }
}

// The same products for steps whose experts have many rows each: tiles of kBigM sorted places (see oi_moe_tile_rows), so
// that an expert's weights are read from the second-level cache once per 128 rows and not once per 32. 8 warps, warp w
// the 32 rows (w & 3) x the 32 columns (w >> 2) of the 128 x 64 tile (and the same columns of the up rows); operand tiles
// of 32 k arrive by cp.async in two buffers, so that a tile's copies run beside the products of the one before. A row's
// sums are formed in the same order as in the kernel above.
constexpr int kBigM = 128;

__device__ __forceinline__ void moe_cp16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;          // 0: the 16 bytes are filled with zeros and src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}

__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

template <typename TO, bool kGlu>
__global__ void __launch_bounds__(256) moe_gemm_mma_big_kernel(const bf16* __restrict__ A, long long lda, int a_div, const bf16* __restrict__ Wt,
                                                               long long w_expert_stride, TO* __restrict__ out, long long ld_out,
                                                               int scatter, const int* __restrict__ sorted,
                                                               const int* __restrict__ tile_info, int max_tiles, int N, int K, float limit,
                                                               int act) {
  pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= tile_info[3 * max_tiles]) return;
  const int e = tile_info[3 * tile], place0 = tile_info[3 * tile + 1], m_rows = min(tile_info[3 * tile + 2], kBigM);
  const int n0 = blockIdx.y * kTileN;
  constexpr int kPad = kTileK + 8;
  __shared__ __align__(16) bf16 As[2][kBigM][kPad];
  __shared__ __align__(16) bf16 Bg[2][kTileN][kPad];
  __shared__ __align__(16) bf16 Bu[2][kGlu ? kTileN : 1][kPad];
  __shared__ int src[kBigM];
  if (threadIdx.x < kBigM) {
    int r = -1;
    if ((int)threadIdx.x < m_rows) {
      const int place = place0 + threadIdx.x;
      r = a_div > 0 ? sorted[place] / a_div : place;
    }
    src[threadIdx.x] = r;
  }
  __syncthreads();
  const bf16* We = Wt + (size_t)e * w_expert_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const int wm = (warp & 3) * 32, wn = (warp >> 2) * 32;
  // this thread's 16-byte pieces of a stage: two of A (rows m, m + 64), one of the gate rows and one of the up rows
  const int lm = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 8;
  const int r0 = src[lm], r1 = src[lm + 64];
  const bool n_ok = n0 + lm < N;
  auto load = [&](int k0, int buf) {
    const bool k_ok = k0 + lk < K;
    moe_cp16(&As[buf][lm][lk], (r0 >= 0 && k_ok) ? A + (size_t)r0 * lda + k0 + lk : A, r0 >= 0 && k_ok);
    moe_cp16(&As[buf][lm + 64][lk], (r1 >= 0 && k_ok) ? A + (size_t)r1 * lda + k0 + lk : A, r1 >= 0 && k_ok);
    const bool ok = n_ok && k_ok;
    moe_cp16(&Bg[buf][lm][lk], ok ? We + (size_t)(n0 + lm) * K + k0 + lk : We, ok);
    if (kGlu) moe_cp16(&Bu[buf][lm][lk], ok ? We + (size_t)(N + n0 + lm) * K + k0 + lk : We, ok);
    asm volatile("cp.async.commit_group;\n" ::);
  };
  float acc[2][4][4] = {}, accu[kGlu ? 2 : 1][4][4] = {};
  load(0, 0);
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += kTileK, buf ^= 1) {
    if (k0 + kTileK < K) {
      load(k0 + kTileK, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; kk += 16) {
      // ldmatrix: lanes 8 q .. 8 q + 7 name the rows of the q-th 8 x 8 piece. A: pieces (rows 0-7, k 0-7), (rows 8-15,
      // k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15); weights: (columns 0-7, k 0-7), (0-7, k 8-15), (8-15, k 0-7), (8-15, k 8-15)
      unsigned a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldsm4(a[i], &As[buf][wm + 16 * i + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        unsigned b[4];
        ldsm4(b, &Bg[buf][wn + 8 * (j + (lane >> 4)) + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
        mma_bf16_16816(acc[0][j], a[0], *reinterpret_cast<const unsigned(*)[2]>(&b[0]));
        mma_bf16_16816(acc[1][j], a[1], *reinterpret_cast<const unsigned(*)[2]>(&b[0]));
        mma_bf16_16816(acc[0][j + 1], a[0], *reinterpret_cast<const unsigned(*)[2]>(&b[2]));
        mma_bf16_16816(acc[1][j + 1], a[1], *reinterpret_cast<const unsigned(*)[2]>(&b[2]));
        if (kGlu) {
          ldsm4(b, &Bu[buf][wn + 8 * (j + (lane >> 4)) + (lane & 7)][kk + ((lane >> 3) & 1) * 8]);
          mma_bf16_16816(accu[0][j], a[0], *reinterpret_cast<const unsigned(*)[2]>(&b[0]));
          mma_bf16_16816(accu[kGlu ? 1 : 0][j], a[1], *reinterpret_cast<const unsigned(*)[2]>(&b[0]));
          mma_bf16_16816(accu[0][j + 1], a[0], *reinterpret_cast<const unsigned(*)[2]>(&b[2]));
          mma_bf16_16816(accu[kGlu ? 1 : 0][j + 1], a[1], *reinterpret_cast<const unsigned(*)[2]>(&b[2]));
        }
      }
    }
    __syncthreads();       // the buffer is free for the copies of the stage after the next
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = wm + 16 * i + g + 8 * h;
      if (m >= m_rows) continue;
      const int place = place0 + m;
      const size_t row = scatter ? (size_t)sorted[place] : (size_t)place;
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn + 8 * j + 2 * tg + c;
          if (n >= N) continue;
          float v = acc[i][j][2 * h + c];
          if (kGlu) v = glu_act<false>(v, accu[kGlu ? i : 0][j][2 * h + c], act, limit);
          out[row * ld_out + n] = from_f32<TO>(v);
        }
    }
}

// The same two products for steps of few rows (at most two pairs an expert on average): one block per (pair, 16 output
// rows), a warp per output row at a time, the pair's input row in shared memory as float32, the expert's rows read 16 bytes
// at a time. No grouping is needed: pair p reads row p / a_div (a_div 0: row p) and writes row p.
template <typename T, typename TO, bool kGlu>
__global__ void __launch_bounds__(128) moe_gemv_kernel(const T* __restrict__ A, long long lda, int a_div, const T* __restrict__ Wt,
                                                       long long w_expert_stride, TO* __restrict__ out, long long ld_out,
                                                       const int* __restrict__ ids, int N, int K, float limit, int act) {
  pdl_wait();    // no early trigger: waiting blocks of the next kernel would share the SMs with this product
  extern __shared__ __align__(16) float xs[];
  constexpr int kVec = 16 / (int)sizeof(T), kRows = 16;
  const int p = blockIdx.x, lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const T* xr = A + (size_t)(a_div > 0 ? p / a_div : p) * lda;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32(xr[k]);
  __syncthreads();
  const T* We = Wt + (size_t)ids[p] * w_expert_stride;
  const bool vec = K % kVec == 0 && ((uintptr_t)We % 16 == 0);
  const int n_end = min(N, (int)(blockIdx.y + 1) * kRows);
  if (vec) {
    // two output rows of the warp at a time, two steps along K unrolled: eight 16-byte loads in flight a lane (a row beyond
    // the block's last reads that one again and is not stored)
    for (int n = blockIdx.y * kRows + wi; n < n_end; n += 8) {
      const int n1 = n + 4 < n_end ? n + 4 : n;
      const T* wg0 = We + (size_t)n * K;
      const T* wg1 = We + (size_t)n1 * K;
      const T* wu0 = wg0 + (size_t)N * K;
      const T* wu1 = wg1 + (size_t)N * K;
      float g0 = 0.f, u0 = 0.f, g1 = 0.f, u1 = 0.f;
#pragma unroll 2
      for (int k = lane * kVec; k < K; k += 32 * kVec) {
        T a0[kVec], b0[kVec], a1[kVec], b1[kVec];
        *reinterpret_cast<uint4*>(a0) = *reinterpret_cast<const uint4*>(wg0 + k);
        *reinterpret_cast<uint4*>(a1) = *reinterpret_cast<const uint4*>(wg1 + k);
        if (kGlu) {
          *reinterpret_cast<uint4*>(b0) = *reinterpret_cast<const uint4*>(wu0 + k);
          *reinterpret_cast<uint4*>(b1) = *reinterpret_cast<const uint4*>(wu1 + k);
        }
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          const float xv = xs[k + e];
          g0 += to_f32(a0[e]) * xv;
          g1 += to_f32(a1[e]) * xv;
          if (kGlu) {
            u0 += to_f32(b0[e]) * xv;
            u1 += to_f32(b1[e]) * xv;
          }
        }
      }
      g0 = warp_sum(g0), g1 = warp_sum(g1);
      if (kGlu) u0 = warp_sum(u0), u1 = warp_sum(u1);
      if (lane == 0) {
        out[(size_t)p * ld_out + n] = from_f32<TO>(kGlu ? glu_act<false>(g0, u0, act, limit) : g0);
        if (n1 != n) out[(size_t)p * ld_out + n1] = from_f32<TO>(kGlu ? glu_act<false>(g1, u1, act, limit) : g1);
      }
    }
    return;
  }
  for (int n = blockIdx.y * kRows + wi; n < n_end; n += 4) {
    const T* wg = We + (size_t)n * K;
    const T* wu = We + (size_t)(N + n) * K;
    float g = 0.f, u = 0.f;
    for (int k = lane; k < K; k += 32) {
      g += to_f32(wg[k]) * xs[k];
      if (kGlu) u += to_f32(wu[k]) * xs[k];
    }
    g = warp_sum(g);
    if (kGlu) u = warp_sum(u);
    if (lane == 0) out[(size_t)p * ld_out + n] = from_f32<TO>(kGlu ? glu_act<false>(g, u, act, limit) : g);
  }
}

// add (or null): a float32 term per output number that every row gets beside its experts' sum (an expert all rows share)
__global__ void moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const float* __restrict__ wts, int top, int W,
                                   size_t n, const float* __restrict__ add) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / W, c = i - t * W;
    float acc = 0.f;
    for (int j = 0; j < top; ++j) acc += wts[t * top + j] * y[(t * top + j) * W + c];
    out[i] = add ? acc + add[i] : acc;
  }
}

}  // namespace

OI_API int oi_moe_max_tiles(int pairs, int experts) { return pairs / kTileM + experts; }

// Sorted places per tile: 128 where the experts have 64 rows and more on average (the weights are then read once per 128
// rows), otherwise 32 (fewer rows that are computed for nothing). A function of the step's size alone.
OI_API int oi_moe_tile_rows(int pairs, int experts) { return (long long)pairs >= 64LL * experts ? kBigM : kTileM; }

// Steps of at most this many (row, choice) pairs take the row-by-row products and need no grouping.
OI_API int oi_moe_small(int pairs, int experts) { return pairs <= 2 * experts && pairs <= 64; }

// x [rows, K] (row stride ldx) in `dtype`; router weights [E, K]; ids, wts [rows, top]; sorted [rows * top];
// tile_info [3 * max_tiles + 1] with max_tiles = oi_moe_max_tiles(rows * top, E).
OI_API int oi_moe_route_scored(const void* x, int dtype, long long ldx, const void* w_router, int w_dtype, int rows, int K, int E,
                               int top, int scoring, const float* correction, int n_groups, int keep_groups, int* ids, float* wts,
                               int* sorted, int* tile_info, void* stream);

OI_API int oi_moe_route(const void* x, int dtype, long long ldx, const void* w_router, int w_dtype, int rows, int K, int E, int top,
                        int* ids, float* wts, int* sorted, int* tile_info, void* stream) {
  return oi_moe_route_scored(x, dtype, ldx, w_router, w_dtype, rows, K, E, top, 0, nullptr, 1, 1, ids, wts, sorted, tile_info, stream);
}

// scoring 0: the `top` largest logits, weighted by their softmax. scoring 1: sigmoid scores; the choice goes by score +
// correction (float32 [E] or null) among the experts of the `keep_groups` best of `n_groups` equal groups of neighbours;
// weights: the chosen scores (without the correction) divided by their sum.
OI_API int oi_moe_route_scored(const void* x, int dtype, long long ldx, const void* w_router, int w_dtype, int rows, int K, int E,
                               int top, int scoring, const float* correction, int n_groups, int keep_groups, int* ids, float* wts,
                               int* sorted, int* tile_info, void* stream) {
  OI_REQUIRE(rows >= 0 && K > 0 && E > 0 && top > 0 && top <= E && top <= kMaxTop, "moe_route: bad sizes experts=%d top=%d (at most %d)", E,
             top, kMaxTop);
  OI_REQUIRE(E <= 4096, "moe_route: %d experts, at most 4096", E);
  OI_REQUIRE(scoring == 0 || scoring == 1, "moe_route: unknown scoring %d", scoring);
  OI_REQUIRE(n_groups >= 1 && keep_groups >= 1 && keep_groups <= n_groups && E % n_groups == 0 && (E / n_groups) * keep_groups >= top,
             "moe_route: %d experts in %d groups of which %d are kept cannot give %d choices", E, n_groups, keep_groups, top);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = 3 * (size_t)E * sizeof(float) + (size_t)E + 16;
  if (dtype == OI_F32)
    oi_launch(moe_router_kernel<float>, rows, 128, smem, s, (const float*)x, ldx, w_router, w_dtype, rows, K, E, top, ids, wts, scoring,
              correction, n_groups, keep_groups);
  else if (dtype == OI_BF16)
    oi_launch(moe_router_kernel<bf16>, rows, 128, smem, s, (const bf16*)x, ldx, w_router, w_dtype, rows, K, E, top, ids, wts, scoring,
              correction, n_groups, keep_groups);
  else
    OI_REQUIRE(false, "moe_route: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  const int pairs = rows * top;
  if (oi_moe_small(pairs, E)) return OI_OK;      // few rows: the products go pair by pair and need no grouping
  oi_launch(moe_group_kernel, E, 256, (size_t)(E + 8) * sizeof(int), s, (const int*)ids, pairs, E, sorted, tile_info, oi_moe_max_tiles(pairs, E), oi_moe_tile_rows(pairs, E));
  OI_CHECK_LAUNCH();
  return OI_OK;
}

namespace {
// Routing without a router: row t uses the experts table[token_ids[t], :], each with the same weight.
__global__ void moe_table_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int rows, int vocab, int E, int top,
                                 float weight, int* __restrict__ ids, float* __restrict__ wts) {
  pdl_start();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * top) return;
  int tok = token_ids[i / top];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  int e = table[(size_t)tok * top + i % top];
  ids[i] = e < 0 ? 0 : (e >= E ? E - 1 : e);
  wts[i] = weight;
}
}  // namespace

// The same outputs as oi_moe_route for a layer whose experts are chosen by the token id: table [vocab, top] int32 (the
// entries of a row differ), every chosen expert weighted 1 / top.
OI_API int oi_moe_route_table(const int* token_ids, const int* table, int rows, int vocab, int E, int top, int* ids, float* wts,
                              int* sorted, int* tile_info, void* stream) {
  OI_REQUIRE(rows >= 0 && vocab > 0 && E > 0 && top > 0 && top <= E && top <= kMaxTop, "moe_route_table: bad sizes experts=%d top=%d (at most %d)",
             E, top, kMaxTop);
  OI_REQUIRE(E <= 4096, "moe_route_table: %d experts, at most 4096", E);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int pairs = rows * top;
  oi_launch(moe_table_kernel, (pairs + 127) / 128, 128, 0, s, token_ids, table, rows, vocab, E, top, 1.f / (float)top, ids, wts);
  OI_CHECK_LAUNCH();
  if (oi_moe_small(pairs, E)) return OI_OK;
  oi_launch(moe_group_kernel, E, 256, (size_t)(E + 8) * sizeof(int), s, (const int*)ids, pairs, E, sorted, tile_info, oi_moe_max_tiles(pairs, E), oi_moe_tile_rows(pairs, E));
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// act [rows * top, F] (scratch, `dtype`), y [rows * top, W] float32 (scratch), out [rows, W] float32; add [rows, W] float32
// or null: added to the weighted sum (out may be add itself).
// w_gate_up [E, 2 F, W] (F gate rows, then F up rows), w_down [E, W, F], both in `dtype`.
OI_API int oi_moe_experts(const void* x, int dtype, long long ldx, const void* w_gate_up, const void* w_down, int rows, int W, int F,
                          int E, int top, float limit, int glu, const int* ids, const int* sorted, const int* tile_info, const float* wts,
                          void* act, float* y, float* out, const float* add, void* stream) {
  OI_REQUIRE(rows >= 0 && W > 0 && F > 0 && E > 0 && top > 0, "moe_experts: bad sizes");
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int pairs = rows * top, max_tiles = oi_moe_max_tiles(pairs, E);
  const size_t n_out = (size_t)rows * W;
  const int cblocks = (int)((n_out + 255) / 256 > 148 * 16 ? 148 * 16 : (n_out + 255) / 256);
  if (oi_moe_small(pairs, E) && (size_t)(W > F ? W : F) * sizeof(float) <= 48 * 1024) {
    const dim3 v1(pairs, (F + 15) / 16), v2(pairs, (W + 15) / 16);
    if (dtype == OI_F32) {
      oi_launch(moe_gemv_kernel<float, float, true>, v1, 128, (size_t)W * 4, s, (const float*)x, ldx, top, (const float*)w_gate_up,
                (long long)2 * F * W, (float*)act, (long long)F, ids, F, W, limit, glu);
      OI_CHECK_LAUNCH();
      oi_launch(moe_gemv_kernel<float, float, false>, v2, 128, (size_t)F * 4, s, (const float*)act, (long long)F, 0, (const float*)w_down,
                (long long)W * F, y, (long long)W, ids, W, F, 0.f, 0);
    } else if (dtype == OI_BF16) {
      oi_launch(moe_gemv_kernel<bf16, bf16, true>, v1, 128, (size_t)W * 4, s, (const bf16*)x, ldx, top, (const bf16*)w_gate_up,
                (long long)2 * F * W, (bf16*)act, (long long)F, ids, F, W, limit, glu);
      OI_CHECK_LAUNCH();
      oi_launch(moe_gemv_kernel<bf16, float, false>, v2, 128, (size_t)F * 4, s, (const bf16*)act, (long long)F, 0, (const bf16*)w_down,
                (long long)W * F, y, (long long)W, ids, W, F, 0.f, 0);
    } else {
      OI_REQUIRE(false, "moe_experts: unknown dtype code %d", dtype);
    }
    OI_CHECK_LAUNCH();
    oi_launch(moe_combine_kernel, cblocks, 256, 0, s, out, (const float*)y, wts, top, W, n_out, add);
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  const int tile_rows = oi_moe_tile_rows(pairs, E), subs = tile_rows / kTileM;
  const bool big = tile_rows == kBigM;
  const dim3 g1(max_tiles, (F + kTileN - 1) / kTileN, subs), g2(max_tiles, (W + kTileN - 1) / kTileN, subs);
  const dim3 b1(max_tiles, (F + kTileN - 1) / kTileN), b2(max_tiles, (W + kTileN - 1) / kTileN);
  if (dtype == OI_F32) {
    oi_launch(moe_gemm_kernel<float, float, true>, g1, 256, 0, s, (const float*)x, ldx, top, (const float*)w_gate_up, (long long)2 * F * W,
              (float*)act, (long long)F, 0, sorted, tile_info, max_tiles, F, W, limit, glu);
    OI_CHECK_LAUNCH();
    oi_launch(moe_gemm_kernel<float, float, false>, g2, 256, 0, s, (const float*)act, (long long)F, 0, (const float*)w_down, (long long)W * F,
              y, (long long)W, 1, sorted, tile_info, max_tiles, W, F, 0.f, 0);
  } else if (dtype == OI_BF16) {
    // tensor cores when every row of the operands starts on a 16-byte boundary
    const bool tc1 = W % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w_gate_up % 16 == 0;
    const bool tc2 = F % 8 == 0 && (uintptr_t)act % 16 == 0 && (uintptr_t)w_down % 16 == 0;
    if (tc1 && big)
      oi_launch(moe_gemm_mma_big_kernel<bf16, true>, b1, 256, 0, s, (const bf16*)x, ldx, top, (const bf16*)w_gate_up, (long long)2 * F * W,
                (bf16*)act, (long long)F, 0, sorted, tile_info, max_tiles, F, W, limit, glu);
    else if (tc1)
      oi_launch(moe_gemm_mma_kernel<bf16, true>, g1, 256, 0, s, (const bf16*)x, ldx, top, (const bf16*)w_gate_up, (long long)2 * F * W,
                (bf16*)act, (long long)F, 0, sorted, tile_info, max_tiles, F, W, limit, glu);
    else
      oi_launch(moe_gemm_kernel<bf16, bf16, true>, g1, 256, 0, s, (const bf16*)x, ldx, top, (const bf16*)w_gate_up, (long long)2 * F * W,
                (bf16*)act, (long long)F, 0, sorted, tile_info, max_tiles, F, W, limit, glu);
    OI_CHECK_LAUNCH();
    if (tc2 && big)
      oi_launch(moe_gemm_mma_big_kernel<float, false>, b2, 256, 0, s, (const bf16*)act, (long long)F, 0, (const bf16*)w_down, (long long)W * F,
                y, (long long)W, 1, sorted, tile_info, max_tiles, W, F, 0.f, 0);
    else if (tc2)
      oi_launch(moe_gemm_mma_kernel<float, false>, g2, 256, 0, s, (const bf16*)act, (long long)F, 0, (const bf16*)w_down, (long long)W * F,
                y, (long long)W, 1, sorted, tile_info, max_tiles, W, F, 0.f, 0);
    else
      oi_launch(moe_gemm_kernel<bf16, float, false>, g2, 256, 0, s, (const bf16*)act, (long long)F, 0, (const bf16*)w_down, (long long)W * F,
                y, (long long)W, 1, sorted, tile_info, max_tiles, W, F, 0.f, 0);
  } else {
    OI_REQUIRE(false, "moe_experts: unknown dtype code %d", dtype);
  }
  OI_CHECK_LAUNCH();
  const size_t n = (size_t)rows * W;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  oi_launch(moe_combine_kernel, blocks, 256, 0, s, out, (const float*)y, wts, top, W, n, add);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
