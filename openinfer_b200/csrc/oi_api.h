// The C interface of the library: every entry point, and the structures of its host-side step code.
//
// All entry points return 0 on success or an error code (common.cuh); oi_last_error() gives the
// message. Pointers are device pointers unless said otherwise; `stream` is a cudaStream_t. Element
// type codes: OI_F32 = 0, OI_BF16 = 1. Activation codes: OI_ACT_NONE / OI_ACT_SILU / OI_ACT_GELU_TANH / OI_ACT_XIELU /
// OI_ACT_SWIGLU_CLAMP.
#pragma once

#include "common.cuh"

// What the streaming product can do where it adds up its K slices, to take the norm kernels out of a decode layer
// (gemm_stream.cu). All pointers are device pointers; a null `ssq_in` / `residual` switches the part off.
typedef struct OiStreamEpilogue {
  // the product FOLLOWS a norm whose weight is already in its input: row m of the sums is multiplied by
  // rsqrt(sum_u ssq_in[m * ssq_stride + u] * inv_width + eps), u < ssq_units
  const float* ssq_in;
  int ssq_units;
  int ssq_stride;              // floats between rows of the partial squares (both directions), a multiple of 4
  float inv_width, eps;
  // the product ENDS a residual branch: out[m, n] = round(residual[m, n] + sum) (out may be the residual itself), and
  // for the norm that reads the row next (xs null: none): xs[m, n] = round(out[m, n] * (w_offset + norm_w[n])) and
  // ssq_out[m * ssq_stride + tile * slices + slice] = the sum of out[m, n]^2 over the columns that slice of that tile owns
  const __nv_bfloat16* residual;
  long long ld_residual;
  const void* norm_w;
  int norm_w_bf16;
  float w_offset;
  __nv_bfloat16* xs;
  long long ld_xs;
  float* ssq_out;
} OiStreamEpilogue;

// What an attention layer may do to its scores beyond scale, mask and softmax; everything off when zero / null.
typedef struct OiScoreMods {
  const float* sinks;    // [nq] float32: one more term exp(sinks[h]) in the softmax's denominator, without a key or a value
  const float* slopes;   // [nq] float32: slopes[h] * (i - j) is taken off the score of key j for the query at position i
  float softcap;         // > 0: score <- softcap * tanh(score / softcap), before the slope
  float qt_coef;         // qt_every > 0: the score of the query at position p is multiplied by
  int qt_every;          //   1 + qt_coef * ln(floor((p + 1) / qt_every) + 1), before the cap
  int keep_first;        // > 0, with a window: the first keep_first keys of a sequence stay visible behind the window
} OiScoreMods;

#ifdef __CUDACC__
constexpr float kLog2e = 1.4426950408889634f;

// What a tensor-core attention kernel instantiated with MODS does to the raw dot products of one query row, leaving them in units of log2: the row's
// temperature and the softmax scale, the cap (tanh through one exp2 and one division: 1 - 2 / (e^(2x) + 1), whose
// absolute error stays near 1e-7 for every x), and the distance slope.
struct RowMods {
  float mul;      // no cap: scale * temperature * log2(e); with a cap: scale * temperature * 2 log2(e) / cap
  float cap_l2;   // cap * log2(e), 0 without a cap
  float slope_l2; // slope * log2(e)
  __device__ __forceinline__ void init(const OiScoreMods& mods, float scale, int head, int pos) {
    float sc = scale;
    if (mods.qt_every > 0) sc *= 1.f + mods.qt_coef * logf((float)((pos + 1) / mods.qt_every) + 1.f);
    cap_l2 = mods.softcap > 0.f ? mods.softcap * kLog2e : 0.f;
    mul = mods.softcap > 0.f ? sc * (2.f * kLog2e) / mods.softcap : sc * kLog2e;
    slope_l2 = mods.slopes ? mods.slopes[head] * kLog2e : 0.f;
  }
  __device__ __forceinline__ float apply(float s, int dist) const {
    float x = s * mul;
    if (cap_l2 > 0.f) {
      float e;
      asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(x));
      x = cap_l2 - __fdividef(2.f * cap_l2, e + 1.f);
    }
    return fmaf(-slope_l2, (float)dist, x);
  }
};
#endif

// argmax_noalloc.cu
OI_API int oi_argmax_noalloc(int* out, const float* logits, int rows, int vocab, long long row_stride, void* stream);

// attention_generic.cu
OI_API int oi_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride, int dtype, const void*
       k_cache, const void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride,
       const int* token_req, const int* positions, int tokens, int nq, int nkv, int hd, float scale, int window,
       const OiScoreMods* mods, void* stream);

// attention_mma.cu
OI_API int oi_attention_decode(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
       const void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int merge_in_kernel,
       void* stream);
OI_API int oi_attention_decode_mods(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
       const void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int merge_in_kernel,
       const OiScoreMods* mods, void* stream);
OI_API int oi_attention_mma_mods(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache, const
       void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int* cu_seqlens,
       const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int any_split, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int rows_per_cta,
       const OiScoreMods* mods, void* stream);
OI_API int oi_attention_decode_rope(const void* qkv, int q_row_stride, void* out, int out_row_stride, void* k_cache,
       void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int merge_in_kernel,
       const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps, float w_offset, const float* cos_tab,
       const float* sin_tab, int rot_half, int max_pos, const int* positions, const int* slots, int write_kv, void*
       stream);
OI_API int oi_attention_mma(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache, const
       void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int
       any_split, int nq, int nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits,
       int rows_per_cta, void* stream);

// attention_tcgen05.cu
OI_API int oi_attention_tcgen05(const void* q, long long q_row_stride, int tokens, void* out, int out_row_stride,
       const void* k_cache, const void* v_cache, long long page_stride, int page_size, int num_pages, const int*
       block_table, int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items, int num_items, int nq,
       int nkv, int hd, float scale, int window, const int* row_splits, int any_split, float* part_o, float* part_lse,
       int max_splits, void* stream);
OI_API int oi_attention_merge_slices(void* out, int out_row_stride, const float* part_o, const float* part_lse,
       const int* row_splits, int nq, int max_splits, int tokens, int hd, void* stream);
OI_API int oi_attention_tcgen05_status(int* status);

// branch_ops.cu: steps of layers that keep the residual stream in 32-bit (see the file's head)
OI_API int oi_rmsnorm_cast(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, const int*
       row_idx, int rows, int hidden, float eps, float w_offset, void* stream);
OI_API int oi_branch_norm_add(float* h, const void* a, int a_dtype, const void* w, int w_dtype, int rows, int hidden,
       float eps, float w_offset, float* hist, long long hist_stride, int n_prev, const void* coef, int coef_dtype,
       void* low, void* stream);
OI_API int oi_history_average(float* h, float* hist, long long hist_stride, int n_prev, const void* coef, int
       coef_dtype, long long n, void* stream);
OI_API int oi_short_conv(void* out, int out_dtype, const void* x, int x_dtype, const void* w, int w_dtype, float*
       state, long long state_stride, const int* cu_seqlens, const int* token_req, const int* state_slots, const int*
       state_phase, int tokens, int requests, int channels, int taps, int add_input, int update_state, void* stream);
OI_API int oi_short_conv_strided(void* out, int out_dtype, long long out_stride, const void* x, int x_dtype, long long
       x_stride, const void* w, int w_dtype, float* state, long long state_stride, const int* cu_seqlens, const int*
       token_req, const int* state_slots, const int* state_phase, int tokens, int requests, int channels, int taps, int
       add_input, int update_state, int act, void* stream);

// elementwise.cu: every gated activation, the ones with a limit included (OI_ACT_SWIGLU_CLAMP)
OI_API int oi_glu_act(void* out, const void* gate_up, int dtype, int rows, int inter, int block, int act, float limit,
       void* stream);

// recurrent.cu: mixers with a matrix memory per head (mode 0: the mLSTM cell, 1: the gated delta rule, 2: linear attention
// with one fixed decay per head, p0 = the decays [H]; q, k and v get their silu there, v in place in `qkv`)
OI_API int oi_recurrent_record(int D);
OI_API int oi_recurrent_scan(int mode, const float* qkv, long long ld_qkv, int q_off, int k_off, int v_off, const float*
       gates, long long ld_gates, int i_off, int f_off, const float* decay, long long ld_decay, const void* p0, const
       void* p1, int p_dtype, float cap, float q_scale, float* prep, float* state, long long state_stride, const int*
       cu_seqlens, const int* token_req, const int* state_slots, const int* state_phase, float* out, long long ld_out,
       int tokens, int requests, int H, int G, int D, int V, void* stream);
OI_API int oi_head_norm_gate(void* out, int out_dtype, long long ld_out, const float* o, long long ld_o, const float*
       gate, long long ld_gate, const void* w, int w_dtype, int w_stride, int tokens, int H, int V, float eps, float
       scale, void* stream);

// sandwich_ops.cu: a Dynamic Tanh norm, dyt(v) = tanh(alpha v) w + b, between two sublayers of a float32 stream
// (h += dyt(branch; post); out = dyt(h; pre), either half optional; row_idx: out is read from these rows of h), and the
// step of an attention that adds the projections' bias (a table by position), rotates, THEN divides q and k heads by their
// root mean square over qk_dim numbers, and stores k and v in their pages
OI_API int oi_dyt_step(float* h, const float* branch, const void* post_alpha, const void* post_w, const void* post_b, int
       post_dtype, const void* pre_alpha, const void* pre_w, const void* pre_b, int pre_dtype, void* out, int out_dtype,
       const int* row_idx, int rows, int width, void* stream);
OI_API int oi_rope_norm_store(void* qkv, int dtype, long long row_stride, int tokens, int nq, int nkv, int hd, int qk_dim,
       const float* bias_tab, int n_tab, long long tab_stride, const float* cos_tab, const float* sin_tab, int rot_half,
       int max_pos, int unit_norm, float eps, const int* positions, const int* slots, void* k_cache, void* v_cache,
       long long page_stride, int page_size, int write_kv, void* stream);

// hyper.cu: several residual streams
OI_API int oi_hyper_step(float* X, int rows, int S, int W, const float* y, const float* y2, float c1, float c2, const
       void* mix, const void* b_out, const void* a_in, int p_dtype, const void* norm_w, int nw_dtype, float eps, float
       w_offset, void* out, int out_dtype, const int* row_idx, void* stream);
OI_API int oi_hyper_fanout(float* X, const void* h, int h_dtype, int rows, int S, int W, void* stream);
OI_API int oi_scaled_sum(float* out, const float* a, const float* b, float ca, float cb, long long n, void* stream);

// moe.cu: routed experts
OI_API int oi_moe_max_tiles(int pairs, int experts);
OI_API int oi_moe_small(int pairs, int experts);
OI_API int oi_moe_tile_rows(int pairs, int experts);
OI_API int oi_moe_route(const void* x, int dtype, long long ldx, const void* w_router, int w_dtype, int rows, int K, int
       E, int top, int* ids, float* wts, int* sorted, int* tile_info, void* stream);
OI_API int oi_moe_experts(const void* x, int dtype, long long ldx, const void* w_gate_up, const void* w_down, int rows,
       int W, int F, int E, int top, float limit, int glu, const int* ids, const int* sorted, const int* tile_info, const float*
       wts, void* act, float* y, float* out, const float* add, void* stream);

// oi_moe_route with the way of scoring as an argument. scoring 0: the `top` largest logits weighted by their softmax.
// scoring 1: sigmoid scores; the choice goes by score + correction (float32 [E] or null) among the experts of the
// `keep_groups` best of `n_groups` equal groups of neighbours (a group's score: the sum of its two largest choice scores);
// the weights are the chosen experts' scores, without the correction, divided by their sum.
OI_API int oi_moe_route_scored(const void* x, int dtype, long long ldx, const void* w_router, int w_dtype, int rows, int K, int E,
                               int top, int scoring, const float* correction, int n_groups, int keep_groups, int* ids, float* wts,
                               int* sorted, int* tile_info, void* stream);
OI_API int oi_moe_route_table(const int* token_ids, const int* table, int rows, int vocab, int E, int top, int* ids, float*
       wts, int* sorted, int* tile_info, void* stream);

// parallel_ops.cu: a latent with a rotated key part, the joint residual add, a gate times a per-token embedding
OI_API int oi_latent_rope_store(void* pages, long long page_stride, int page_size, int row_elems, void* proj, long long
       proj_stride, int dtype, int tokens, int latent_off, int rank, const void* w, int w_dtype, float eps, float
       w_offset, int rot_half, const float* cos_tab, const float* sin_tab, int max_pos, const int* positions, const int*
       slots, int heads, int q_head_stride, int q_rot_off, int store, void* stream);
OI_API int oi_add2_cast(float* x, const float* a, const float* b, void* low, int low_dtype, long long n, void* stream);
OI_API int oi_token_gate(void* g, long long g_stride, int dtype, const int* token_ids, const void* table, int table_dtype,
       long long table_stride, int vocab, int off, int dim, int tokens, void* stream);

// gemm_stream.cu / gemm_tcgen05.cu: the gate/up product with a gated activation that takes a limit
OI_API int oi_gemm_stream_glu(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long
       long ldw, int M, int N, int K, int cluster_size, int act, float limit, void* stream);
OI_API int oi_gemm_tcgen05_glu(void* C, long long ldc, const void* A, long long lda, const void* W, long long ldw, int M,
       int N, int K, int pair, int act, float limit, void* stream);

OI_API int oi_latent_store(void* pages, long long page_stride, int page_size, int row_elems, const void* src, long
       long src_stride, int dtype, const void* w, int w_dtype, const int* slots, int tokens, int rank, float eps,
       float w_offset, void* stream);
OI_API int oi_head_gate(void* o, long long o_stride, const void* g, long long g_stride, int dtype, int tokens, int
       heads, int head_elems, void* stream);
OI_API int oi_xielu(void* out, const void* in, int dtype, const void* pq, int pq_dtype, long long n, void* stream);

// elementwise.cu
OI_API int oi_embedding(void* out, int out_dtype, const void* table, int table_dtype, const int* ids, int tokens, int
       hidden, int vocab, void* stream);
OI_API int oi_gather_tokens(int* ids, const int* src, const int* from, int n, int n_from, void* stream);
OI_API int oi_copy_words(int* dst, const int* src, int n, int ids_off, int src_off, int n_ids, const int* from, int
       n_from, void* stream);
OI_API int oi_rmsnorm(void* out, void* x, const void* delta, int dtype, const void* w, int w_dtype, const int*
       row_idx, int rows, int hidden, float eps, float w_offset, void* stream);
OI_API int oi_add_inplace(void* x, const void* delta, int dtype, long long n, void* stream);
OI_API int oi_scale_cap(void* x, int dtype, long long n, float scale, float cap, void* stream);
OI_API int oi_silu_mul(void* out, const void* gate_up, int dtype, int rows, int inter, int block, int act, void*
       stream);

// gemm_generic.cu
OI_API int oi_gemm_generic(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
       int K, long long lda, long long ldw, long long ldc, void* stream);

// gemm_skinny.cu
OI_API int oi_gemm_skinny(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long
       long ldw, int M, int N, int K, int silu_mul, int act, int cluster_size, void* stream);

// gemm_stream.cu
OI_API int oi_gemm_stream(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long
       long ldw, int M, int N, int K, int cluster_size, int act, void* stream);
OI_API int oi_gemm_stream_fused(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
       long long ldw, int M, int N, int K, int cluster_size, int act, const OiStreamEpilogue* epilogue, void* stream);
OI_API int oi_gemm_stream_unary(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
       long long ldw, int M, int N, int K, int cluster_size, int act, float p0, float p1, void* stream);
OI_API int oi_gemm_stream_status(int* status);

// gemm_tcgen05.cu
OI_API int oi_gemm_tcgen05(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W, long long
       ldw, int M, int N, int K, int tile_n, int act, void* stream);
OI_API int oi_gemm_tcgen05_pair(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W, long
       long ldw, int M, int N, int K, int act, void* stream);
OI_API int oi_gemm_tcgen05_unary(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W, long
       long ldw, int M, int N, int K, int pair, int act, float p0, float p1, void* stream);
OI_API int oi_gemm_tcgen05_status(int* status);

// rope_kv.cu
OI_API int oi_qk_norm_rope_kv(void* qkv, int dtype, int row_stride, int tokens, int nq, int nkv, int hd, const void*
       q_norm_w, const void* k_norm_w, int norm_dtype, float eps, float w_offset, const float* cos_tab, const float*
       sin_tab, int rot_half, int max_pos, const int* positions, const int* slots, void* k_cache, void* v_cache, long
       long page_stride, int page_size, int write_kv, int interleaved, void* stream);

// runtime.cu
OI_API const char* oi_last_error();
OI_API int oi_abi_version();
OI_API unsigned long long oi_launches();
OI_API int oi_launch_fence();   // the next kernel launched by this library gets plain stream order (once)
OI_API int oi_set_pdl(int enabled);
OI_API int oi_device_info(int device, int* sm_major, int* sm_minor, int* sm_count, long long* l2_bytes);

// sampling.cu
OI_API int oi_argmax_chunks(int vocab);
OI_API int oi_argmax(int* out, const float* logits, int rows, int vocab, long long row_stride, float* partial_vals,
       int* partial_idx, void* stream);
OI_API int oi_sample_use_clusters(int on);
OI_API int oi_sample(int* out, const float* logits, long long row_stride, float* probs, int rows, int vocab, const
       float* temperature, const int* top_k, const float* top_p, const float* min_p, const float* uniform, void*
       stream);
OI_API int oi_token_logprobs(const float* logits, long long row_stride, int vocab, const int* rows, const int* picked,
       const int* ks, int n, int k_max, float* out_lp, float* top_vals, int* top_ids, void* stream);

// library_gemm.cu
OI_API int oi_library_gemm_ready();
OI_API int oi_library_gemm_init(const char* path, void* workspace, long long workspace_bytes);
OI_API int oi_library_gemm(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
       long long ldw, int M, int N, int K, void* stream);

// ------------------------------------------------------------------------------------------------
// host_step.cu: the host side of a step in native code. Which kernel takes which product, the gated
// feed-forward, one layer's attention, and the whole stack of layers of a model assembled from this
// package's own parts. The Python parts call the first three one by one (so a model that mixes them
// with parts of its own runs the same code); a model made of package parts only runs the fourth, one
// call for all layers of a step.
// ------------------------------------------------------------------------------------------------

// Options of the dispatch (oi_configure): values are ints.
enum : int {
  OI_OPT_BATCH_INVARIANT = 0,   // 1: every choice depends on the request alone (one product kernel for all shapes)
  OI_OPT_DECODE_GEMM = 1,       // products of up to 32 rows: 0 streaming tcgen05 kernel, 1 mma.sync kernel, 2 library
  OI_OPT_PREFILL_GEMM = 2,      // plain products of more rows: 0 library, 1 the pair kernel of gemm_tcgen05.cu
  OI_OPT_FORCE_SLICES = 3,      // > 0: K slices of the decode products, whatever the shape (measurements)
  OI_OPT_PAIR_MIN_ROWS = 4,     // rows from which the fused gate/up product uses pairs of CTAs
  OI_OPT_FUSE_NORM = 5,         // 1: steps of up to 32 rows run without norm kernels inside the layer stack (oi_forward);
                                // off by default: measured slower, see host_step.cu
  OI_OPT_COUNT = 6,
};
OI_API int oi_configure(int option, int value);
OI_API int oi_option(int option);

// y[M, N] = x[M, K] W[N, K]^T by the kernel that the operand types, the shape and the options select.
OI_API int oi_linear(void* out, int out_dtype, long long ldc, const void* x, int x_dtype, long long ldx, const void* W,
       int w_dtype, long long ldw, int M, int N, int K, void* stream);
// How many K slices the streaming product uses for a shape (what oi_linear passes to oi_gemm_stream).
OI_API int oi_stream_slices(int N, int K);

// down( act(gate x) * (up x) ): out[M, hidden]. w_gate_up [2 inter, hidden] with rows in blocks of `act_block`
// gate rows followed by the up rows of the same indices; w_down [hidden, inter]. Scratch: `act_buf` [M, inter]
// and `gate_up_buf` [M, 2 inter] in x's type (the second is only written when no kernel forms the activation
// inside the product; it may be null if the caller knows that, see oi_gated_mlp_needs_gate_up).
OI_API int oi_gated_mlp(void* out, const void* x, int dtype, int M, int hidden, int inter, const void* w_gate_up,
       int w_gate_up_dtype, const void* w_down, int w_down_dtype, int act, int act_block, void* act_buf,
       void* gate_up_buf, void* stream);
OI_API int oi_gated_mlp_needs_gate_up(int dtype, int w_dtype, int M, int hidden, int inter, int act_block);

// down( act(up x) ) with one up-projection and the xIELU activation: out[M, hidden] in float32. `act_pq`: the
// activation's two raw numbers on the device (read by the stand-alone activation kernel), a_p / a_n: the numbers the
// formula uses, softplus(p) and 1/2 + softplus(q), formed by the host once (given to the products that apply the
// activation in their epilogue: the weight stream up to 32 rows, the tcgen05 tiles beyond). `z_buf` [M, inter] in x's type.
OI_API int oi_dense_mlp(float* out, const void* x, int dtype, int M, int hidden, int inter, const void* w_up, int w_up_dtype,
       const void* w_down, int w_down_dtype, const void* act_pq, int pq_dtype, float a_p, float a_n, void* z_buf, void* stream);

// What one step's attention calls share, per cache group and attention geometry: the step's metadata on the
// device and the work items planned on the host.
typedef struct OiAttnStep {
  const int* slot_mapping;   // [tokens] page * page_size + offset where the row's key and value go, -1: nowhere
  const int* block_table;    // [requests, bt_stride]
  const int* kv_lens;        // [requests]
  const int* cu_seqlens;     // [requests + 1]
  const int* token_req;      // [tokens]
  const int* positions;      // [tokens]
  int bt_stride, tokens, page_size, num_pages;
  long long page_stride;     // elements between pages of a layer's K (and V) tensor
  int tensor_core;           // 0: the general kernel; 1: the tile / decode kernels below
  int use_tcgen05;           // prompt tiles go to the tcgen05 kernel (else mma.sync)
  int fuse_rope;             // the decode kernel normalises, rotates and stores (single-token steps)
  const int* tile_items;     // [num_tile_items, 4]
  const int* decode_items;   // [num_decode_items, 4]
  const int* row_splits;     // [tokens]
  int num_tile_items, num_decode_items, rows_per_cta, tile_split, max_splits, merge_in_kernel;
  float* part_o;             // partial results of key slices that are merged by a second kernel (or null)
  float* part_lse;
} OiAttnStep;

// One layer's (more exactly: one run-order entry's) attention.
typedef struct OiAttnLayer {
  void* qkv;                 // [tokens, q | k | v] raw projections (q only when write_kv is 0 and rope_mode is 0)
  void* out;                 // [tokens, nq * hd]
  void* k_cache;             // this layer's pages [pages, page_size, nkv, hd]
  void* v_cache;
  const void* q_norm_w;      // [hd] or null
  const void* k_norm_w;
  const float* cos_tab;      // [max_pos, rot_half] or null
  const float* sin_tab;
  int q_row_stride, out_row_stride, dtype;
  int nq, nkv, hd, window;   // window 0: every key
  float scale, eps, w_offset;
  int norm_dtype, rot_half, max_pos;
  int interleaved;           // the rotation turns neighbours (2 d, 2 d + 1) instead of (d, d + half)
  int write_kv;              // the call owns its cache: keys and values of the step's rows are stored
  int rope_mode;             // 0: q is ready and the cache is written; 1: norm + rotation + cache write first (in its own
                             // kernel, or inside the decode kernel when the step says fuse_rope)
  OiScoreMods mods;          // sink, distance slopes, cap and query temperature (all off for a plain softmax)
} OiAttnLayer;

OI_API int oi_attention_layer(const OiAttnStep* step, const OiAttnLayer* layer, void* stream);

// One entry of a model's run order, assembled from this package's parts: pre-norm block of attention and a
// gated feed-forward, each residual add carried out by the norm that follows.
typedef struct OiLayerDesc {
  const void* input_norm_w;
  const void* post_norm_w;
  const void* w_qkv;         // [qkv_rows, hidden]
  const void* w_o;           // [hidden, nq * hd]
  const void* w_gate_up;     // [2 inter, hidden]
  const void* w_down;        // [hidden, inter]
  OiAttnLayer attn;          // qkv / out are filled in per step
  int input_norm_dtype, post_norm_dtype, w_qkv_dtype, w_o_dtype, w_gate_up_dtype, w_down_dtype;
  float input_eps, input_offset, post_eps, post_offset;
  int qkv_rows;              // (nq + 2 nkv) * hd, or nq * hd when the entry reads another entry's cache
  int attn_step;             // which OiAttnStep of the step this entry uses
  int inter, act, act_block;
} OiLayerDesc;

typedef struct OiModelDesc {
  const OiLayerDesc* layers;  // host pointer, num_layers entries in run order
  const void* embedding;      // [vocab, hidden]
  const void* final_norm_w;
  const void* head;           // [vocab, hidden]
  int num_layers, hidden, vocab, dtype;
  int embedding_dtype, final_norm_dtype, head_dtype;
  float embedding_scale, final_eps, final_offset, logit_soft_cap;
  int max_qkv_rows, max_q_dim, max_inter;   // widths of the step's scratch rows
} OiModelDesc;

typedef struct OiStepDesc {
  const int* token_ids;       // [tokens]
  const OiAttnStep* attn_steps;   // host pointer
  const int* want_rows;       // [num_want] rows whose logits are wanted (or null)
  void* h;                    // [tokens, hidden]  the residual stream
  void* x;                    // [tokens, hidden]  normed rows
  void* qkv;                  // [tokens, max_qkv_rows]
  void* attn;                 // [tokens, max_q_dim]
  void* branch_a;             // [tokens, hidden]  output of the mixer
  void* branch_m;             // [tokens, hidden]  output of the feed-forward
  void* act;                  // [tokens, max_inter]
  void* gate_up;              // [tokens, 2 max_inter] or null (see oi_gated_mlp_needs_gate_up)
  void* wanted;               // [num_want, hidden] normed wanted rows
  float* logits;              // [num_want, vocab]
  void* xs;                   // [tokens, hidden] rows times the next norm's weight (steps of up to 32 rows; or null)
  float* ssq;                 // [32, ssq_stride] partial sums of squares (with xs); ssq_stride >= 8 * ceil(hidden / 128)
  int ssq_stride;
  int tokens, num_attn_steps, num_want;
} OiStepDesc;

// Embedding, every layer, final norm of the wanted rows, head: all kernels of one step, launched from native code.
OI_API int oi_forward(const OiModelDesc* model, const OiStepDesc* step, void* stream);

// ------------------------------------------------------------------------------------------------
// The same for models whose every layer is a "branchnorm" block over a float32 stream (branch_ops.cu): an
// optional short convolution in front of the mixer, attention over a cached latent (up-projections multiplied
// into the weights), the norm on each branch's output fused with the residual sum, an optional dense
// feed-forward, an optional weighted average over the results of all layers so far.
// ------------------------------------------------------------------------------------------------
typedef struct OiBranchLayerDesc {
  const void* conv_w;         // [hidden, taps] or null: the mixer then reads the stream as it is
  float* conv_state;          // [slots, 2, taps - 1, hidden] or null (one tap)
  const void* w_in;           // [in_cols, hidden]: queries | latent | gate | zero rows
  const void* w_out;          // [hidden, heads * row]
  const void* latent_norm_w;  // [rank] or null (the layer reads another layer's latent)
  void* pages;                // the latent's pages [pages, page_size, 1, row]
  const void* mixer_norm_w;   // [hidden]
  const void* ff_norm_w;      // [hidden] or null
  const void* w_up;           // [inter, hidden] or null (no feed-forward)
  const void* w_down;         // [hidden, inter]
  const void* act_pq;         // the activation's two numbers as stored; act_a_p / act_a_n: as the formula uses them
  const void* depth_coef;     // [depth_terms] or null
  long long conv_state_stride;
  int conv_w_dtype, taps, add_input;
  int w_in_dtype, w_out_dtype, latent_norm_dtype, mixer_norm_dtype, ff_norm_dtype, w_up_dtype, w_down_dtype, pq_dtype, depth_dtype;
  int in_cols, heads, row, rank, window, latent_off, gate_off, has_gate;
  int attn_step, inter, depth_terms;
  float scale, latent_eps, latent_offset, mixer_eps, mixer_offset, ff_eps, ff_offset, act_a_p, act_a_n;
} OiBranchLayerDesc;

typedef struct OiBranchModelDesc {
  const OiBranchLayerDesc* layers;   // host pointer, num_layers entries in run order
  const void* embedding;
  const void* final_norm_w;
  const void* head;
  int num_layers, hidden, vocab, dtype;
  int embedding_dtype, final_norm_dtype, head_dtype;
  float embedding_scale, final_eps, final_offset, logit_soft_cap, logit_scale;
} OiBranchModelDesc;

typedef struct OiBranchStepDesc {
  const int* token_ids;
  const OiAttnStep* attn_steps;      // host pointer
  const int* want_rows;
  const int* cu_seqlens;
  const int* token_req;
  const int* state_slots;
  const int* state_phase;     // [requests] which copy of a two-phase state the step reads
  float* h;                   // [tokens, hidden] the stream
  float* hist;                // [num_layers + 1, tokens, hidden] or null (no layer averages)
  void* u;                    // [tokens, hidden] what the mixer reads, in the model's type
  void* low;                  // [tokens, hidden] the stream rounded to the model's type (bfloat16 models; else null)
  void* proj;                 // [tokens, max in_cols]
  void* mixed;                // [tokens, max heads * row]
  float* branch;              // [tokens, hidden]
  void* z;                    // [tokens, max inter]
  void* wanted;               // [num_want, hidden]
  float* logits;              // [num_want, vocab]
  int tokens, requests, num_attn_steps, num_want;
} OiBranchStepDesc;

OI_API int oi_forward_branch(const OiBranchModelDesc* model, const OiBranchStepDesc* step, void* stream);
