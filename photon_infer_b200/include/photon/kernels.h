/* photon/kernels.h: the C interface of the sm_100a kernels of photon_infer_b200.
 *
 * Every kernel source under csrc/ becomes one shared library; the functions below are what those libraries
 * export (C linkage, default visibility).  The Python side (photon_infer_b200/kernels/ops.py) calls them through
 * ctypes; a C or C++ program can link the libraries and call them the same way.  csrc/common.cuh includes this
 * header, so a definition that drifts from its declaration does not compile.
 *
 * lumia431/photon_infer's library surface is C++ classes (include/photon/arch/llama_model.hpp:61-240,
 * include/photon/scheduler/continuous_batch_engine.hpp:48-315).  Here the host side (configuration, weights,
 * cache manager, step function, scheduler) is Python; this header is the part of the library that is native.
 *
 * Conventions
 *   - All pointers are device pointers unless a comment says "host".  Kernels run on `stream`.
 *   - Return value: 0 = launched; > 0 = a cudaError_t; PHOTON_ERR_UNSUPPORTED (-2) = this size or alignment is
 *     refused (nothing ran); PHOTON_ERR_ARGUMENT (-3) = invalid argument.  Never a wrong result.
 *   - dtype codes: PHOTON_F32 0, PHOTON_BF16 1.
 *   - `err`: int[4] on the device (may be null).  A kernel that meets a bad index (token id, cache slot, page)
 *     skips the access and records {code, detail0, detail1, detail2} once (PHOTON_DEV_* below); a bounded wait
 *     that ran out records PHOTON_DEV_WAIT_TIMEOUT.
 *   - The paged cache of one layer: K and V each [num_pages][n_kv][page_size][head_dim], contiguous.
 *     block_table [S][max_pages] int: pages of request s in order, -1 where none is held.
 *     slot_mapping [T] int: page * page_size + offset of each token of the step; -1 = do not store.
 *   - A step holds T tokens of S requests; cu_tokens [S + 1] gives each request's first token;
 *     positions [T] each token's position in its request; a token at position p sees keys max(0, p - window + 1)..p
 *     (window 0: all keys up to p).
 *   - Matrix products compute out[M, N] = x[M, K] * W[N, K]^T (W row-major [out, in], no bias), leading
 *     dimensions in elements.
 */
#ifndef PHOTON_KERNELS_H
#define PHOTON_KERNELS_H

#include <cuda_runtime.h>

#if defined(__GNUC__)
#define PHOTON_EXPORT __attribute__((visibility("default")))
#else
#define PHOTON_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define PHOTON_F32 0
#define PHOTON_BF16 1
#define PHOTON_ERR_UNSUPPORTED (-2)
#define PHOTON_ERR_ARGUMENT (-3)
#define PHOTON_DEV_BAD_TOKEN 1
#define PHOTON_DEV_BAD_SLOT 2
#define PHOTON_DEV_BAD_PAGE 3
#define PHOTON_DEV_WAIT_TIMEOUT 4
/* activations of the gated feed-forward kernels: silu, and the tanh form of gelu */
#define PHOTON_ACT_SILU 0
#define PHOTON_ACT_GELU_TANH 1
#define PHOTON_ACT_GELU 2            /* the exact form, 0.5 z (1 + erf(z / sqrt 2)) */
#define PHOTON_ACT_RELU 3
#define PHOTON_ACT_NONE (-1)

/* ------------------------------------------------------------------ elementwise.cu */
/* out[t, :] = table[ids[t], :] as float; ids outside [0, V) give a zero row and PHOTON_DEV_BAD_TOKEN. */
PHOTON_EXPORT int photon_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int V, int* err,
                     cudaStream_t stream);
/* residual (float [*, H], in place) += delta (+ delta2); out = w * residual / sqrt(mean(residual^2) + eps).  delta and
 * delta2 (same type; the two outputs of a parallel block) may be null.
 * rows (may be null): only these rows are read, nothing is written back, out has one row per entry. */
PHOTON_EXPORT int photon_add_rmsnorm(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                       int w_dtype, void* out, int out_dtype, const int* rows, int n, int H, float eps, cudaStream_t stream);
/* The same with delta multiplied channel by channel by delta_scale (float [H], may be null) before the sums. */
PHOTON_EXPORT int photon_add_rmsnorm_scaled(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                       int w_dtype, void* out, int out_dtype, const int* rows, int n, int H, float eps,
                       const float* delta_scale, cudaStream_t stream);
PHOTON_EXPORT int photon_add_layernorm_scaled(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                         int w_dtype, const void* b, int b_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                         float eps, const float* delta_scale, cudaStream_t stream);
/* The same with a layer norm: out = (x - mean(x)) / sqrt(var(x) + eps) * w + b, x = residual + delta (+ delta2); b may be null. */
PHOTON_EXPORT int photon_add_layernorm(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                         int w_dtype, const void* b, int b_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                         float eps, cudaStream_t stream);
/* out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]; gate_up [T, 2I], out [T, I] of one dtype; act: PHOTON_ACT_*.
 * photon_swiglu is photon_glu with silu. */
PHOTON_EXPORT int photon_glu(const void* gate_up, void* out, int dtype, int T, int I, int act, cudaStream_t stream);
PHOTON_EXPORT int photon_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream);
/* out [T, 2H] = [residual + delta + delta2 ; other] rounded once to out_dtype (delta, delta2 may be null). */
PHOTON_EXPORT int photon_stream_concat(const float* residual, const void* delta, const void* delta2, int delta_dtype,
                         const float* other, void* out, int out_dtype, int T, int H, cudaStream_t stream);
/* x [T, H] (float, in place) = x * scale + bias; bias [H] of bias_dtype, may be null. */
PHOTON_EXPORT int photon_scale_bias_rows(float* x, float scale, const void* bias, int bias_dtype, int T, int H, cudaStream_t stream);
/* out[i] = act(x[i]) over total elements of one dtype (x may be out); act: PHOTON_ACT_SILU, _GELU_TANH or _GELU. */
PHOTON_EXPORT int photon_activation(const void* x, void* out, int dtype, long total, int act, cudaStream_t stream);
/* x [T, W] (row stride ldx, in place) *= sigmoid(g [T, W]) (row stride ldg, its own dtype), in 32-bit, rounded once. */
PHOTON_EXPORT int photon_gate_mul(void* x, long ldx, int x_dtype, const void* g, long ldg, int g_dtype, int T, int W, cudaStream_t stream);
/* residual [T, H] (float, in place) += (delta + delta2) + other + bias; delta, delta2 [T, H] of delta_dtype, other [T, H]
 * float, bias [H] of bias_dtype; each may be null. */
PHOTON_EXPORT int photon_stream_add(float* residual, const void* delta, const void* delta2, int delta_dtype, const float* other,
                      const void* bias, int bias_dtype, int T, int H, cudaStream_t stream);

/* ------------------------------------------------------------------ rope_kv.cu */
/* Rotates q [T, n_q * d] and k [T, n_kv * d] in place (rotate != 0; pairs (2j, 2j+1) when interleaved, else
 * (j, j + d/2); angle positions[t] * inv_freq[j] in 32-bit) and stores k, v at slot_mapping in the cache
 * (write_kv != 0).  q, k, v may be views with any row stride (elements). */
PHOTON_EXPORT int photon_rope_kv_write(void* q, long q_stride, void* k, long k_stride, const void* v, long v_stride, int dtype,
                         const int* positions, const float* inv_freq, int interleaved, const int* slot_mapping,
                         void* k_cache, void* v_cache, int T, int n_q, int n_kv, int d, int page_size, long num_slots,
                         int rotate, int write_kv, int* err, cudaStream_t stream);
/* out [count][half][2] float: (cos, sin) of position * inv_freq[j]. */
PHOTON_EXPORT int photon_rope_table(const float* inv_freq, int half, int count, void* out, cudaStream_t stream);

/* ------------------------------------------------------------------ qk_norm.cu */
/* Per head: y = x / sqrt(mean(x^2) + eps) [* w], then the first rot_dims numbers rotated in halves (number j with number
 * j + rot_dims / 2) by position * inv_freq[j] (double [rot_dims / 2]; null: no rotation); queries to q_out (out_dtype),
 * keys and values (dv wide) into their caches at slot_mapping (slot -1: nothing stored; both caches null: only queries).
 * in_dtype may be PHOTON_F32 while out_dtype is PHOTON_BF16. */
PHOTON_EXPORT int photon_qk_norm_rope_write(const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
                              int in_dtype, void* q_out, long qo_stride, int out_dtype, const void* q_w, const void* k_w,
                              int w_dtype, float eps, const int* positions, const double* inv_freq, int rot_dims,
                              const int* slot_mapping, void* k_cache, void* v_cache, int T, int n_q, int n_kv, int d, int dv,
                              int page_size, long num_slots, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention.cu (float32 and any even head size) */
/* Values are dv wide: v_cache [num_pages][n_kv][page_size][dv], out [T][n_q * dv]; v_cache == k_cache (dv <= d): the value
 * of a key is the head of its own row (attention over a cached latent).  splits > 1: every token's key tiles are shared out
 * over that many blocks and merged by a second kernel; part: float [T * n_q * splits * (dv + 2)]. */
PHOTON_EXPORT int photon_paged_attention(const void* q, long q_stride, void* out, long out_stride, int dtype, const void* k_cache,
                           const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                           const int* positions, int T_, int n_q, int n_kv, int d, int dv, int page_size, int num_pages,
                           int window, float scale, int splits, float* part, int* err, cudaStream_t stream);
/* The same with kept first keys (keys < keep_first stay visible behind the window), a sink (one more key with score 0 and
 * no value in the softmax's denominator) and bounded scores (s <- softcap * tanh(s / softcap); 0: off).  gate (may be
 * null; here and in the two tensor-core kernels below): [T, n_q * dv] of the type of q, row stride gate_stride; every
 * output is multiplied by sigmoid(gate) before it is rounded. */
PHOTON_EXPORT int photon_paged_attention_ex(const void* q, long q_stride, void* out, long out_stride, int dtype, const void* k_cache,
                              const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                              const int* positions, int T_, int n_q, int n_kv, int d, int dv, int page_size, int num_pages,
                              int window, float scale, int splits, float* part, int* err, int keep_first, int sink,
                              float softcap, const void* gate, long gate_stride, cudaStream_t stream);

/* ------------------------------------------------------------------ latent.cu: attention over a cached latent */
/* One pass over a token's fused down-projection row down[t] = [query latent (q_rank) | key/value latent (kv_rank) |
 * shared key part (rot)]: cq[t] = rmsnorm(query latent) * q_norm_w; the cache row at slot_mapping[t] becomes
 * [rmsnorm(key/value latent) * kv_norm_w | key part with its first rot_dims numbers rotated (i paired with
 * i + rot_dims / 2, angle positions[t] * inv_freq[i])].  cache: [num_slots][kv_rank + rot]. */
PHOTON_EXPORT int photon_latent_prep(const void* down, long down_stride, int dtype, int q_rank, int kv_rank, int rot, int rot_dims,
                       const void* q_norm_w, int q_norm_dtype, const void* kv_norm_w, int kv_norm_dtype, float eps,
                       const int* positions, const float* inv_freq, const int* slot_mapping, void* cq, long cq_stride,
                       void* cache, long num_slots, int T_, int* err, cudaStream_t stream);
/* out[t, h, out_off .. out_off + rot) = the last rot numbers of head h of q [T][heads][dim + rot], rotated as above. */
PHOTON_EXPORT int photon_latent_q_rope(const void* q, long q_stride, int dtype, int heads, int dim, int rot, int rot_dims,
                         const int* positions, const float* inv_freq, void* out, long out_stride, int out_head,
                         int out_off, int T_, cudaStream_t stream);
/* out[t, h, :] = W[h] x[t, h, :] for every head: x [M][heads][K], out [M][heads][N] (row and head strides in elements),
 * W [heads][N][K]. */
PHOTON_EXPORT int photon_head_linear(const void* x, long x_row, long x_head, const void* W, void* out, long o_row, long o_head,
                       int dtype, int M, int heads, int N, int K, cudaStream_t stream);

/* out[p, :] = the cache row of position p < count of the request whose pages are table (cache [num_pages * page_size][width]). */
PHOTON_EXPORT int photon_gather_rows(const void* cache, int dtype, const int* table, int page_size, int num_pages, int width,
                       int count, void* out, int* err, cudaStream_t stream);
/* probs [rows][ldp] = softmax(scale * scores [rows][ld]) over the keys 0 .. first_pos + r / heads of row r, zero beyond,
 * up to column cols. */
PHOTON_EXPORT int photon_causal_softmax_rows(const float* scores, long ld, void* probs, long ldp, int dtype, int rows, int heads,
                               int first_pos, int cols, float scale, cudaStream_t stream);

/* Decoded tokens on the tensor cores (bfloat16; width and dv multiples of 16): token t sees the rows 0 .. positions[t] of
 * request token_seq[t]; a row's value is its first dv numbers.  splits >= ceil((largest position + 1) / 64); part: float
 * [T * heads * splits * (dv + 2)]. */
PHOTON_EXPORT int photon_latent_decode_attention(const void* q, long q_stride, const void* cache, const int* block_table,
                                   int max_pages, const int* token_seq, const int* positions, int T_, int heads, int width,
                                   int dv, int page_size, int num_pages, float scale, int splits, float* part, void* out,
                                   long out_stride, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ delta.cu: gated delta rule (recurrent state, short convolutions) */
/* The state row of a request: S float [H][dim][vdim], then at conv_offset the last taps - 1 projected rows [taps - 1][C],
 * C = 2 Gq dim + H vdim (Gq query/key heads, H value heads); a state slot of -1 starts from zeros and stores nothing.
 * photon_delta_conv: x [T][>= C] of x_dtype (q, k, v projected, side by side); y float [T][C] = silu(causal convolution per
 * channel, taps_w float [C][taps], last column the current token), q and k heads made unit vectors, q times dim^(-1/2);
 * then the state's rows are brought up to date. */
PHOTON_EXPORT int photon_delta_conv(const void* x, long x_stride, int x_dtype, const float* taps_w, int taps, const int* token_seq,
                      const int* cu_tokens, const int* state_slots, float* state, long state_stride, long conv_offset,
                      int num_slots, float* y, int T, int S, int Gq, int H, int dim, int vdim, int* err, cudaStream_t stream);
/* Per (request, head): g = exp(-exp(a_log) softplus(a + dt_bias)), beta = sigmoid(b); S <- g S; u = beta (v - S^T k);
 * S <- S + k u^T; o = S^T q.  ab [T][>= 2 H] of ab_dtype: the a of the H heads, then the b; o float [T][H * vdim]. */
PHOTON_EXPORT int photon_delta_recurrent(const float* y, const void* ab, long ab_stride, int ab_dtype, const float* a_log,
                           const float* dt_bias, const int* cu_tokens, const int* state_slots, float* state,
                           long state_stride, int num_slots, float* o, int S, int Gq, int H, int dim, int vdim, int* err,
                           cudaStream_t stream);
/* out = o / sqrt(mean(o^2) + eps) * norm_w * silu(z) per head over vdim; z [T][H * vdim] of z_dtype, norm_w float [vdim]. */
PHOTON_EXPORT int photon_delta_out(const float* o, const void* z, long z_stride, int z_dtype, const float* norm_w, float eps,
                     void* out, long out_stride, int out_dtype, int T, int H, int vdim, cudaStream_t stream);

/* ------------------------------------------------------------------ row_norms.cu: norms over parts of a row, PolyNorm, bounded values */
/* The row x [T][H] (x_dtype, row stride x_stride) is cut into `groups` equal consecutive parts, each divided by its own
 * sqrt(mean(part^2) + eps), the whole times w [H].  gate (float [T][H], row stride gate_stride): gate_mode 1 multiplies the
 * row by silu(gate) before the norm, gate_mode 2 the normed row by sigmoid(gate); 0: no gate (null).  residual (float
 * [T][H], may be null): the result is added to it in place and `out` (may then be null) receives the new rows of the
 * stream; x null: `out` receives the stream's rows as they are.  Without a residual `out` receives the result. */
PHOTON_EXPORT int photon_group_rmsnorm(const void* x, long x_stride, int x_dtype, const float* gate, long gate_stride, int gate_mode,
                     float* residual, const void* w, int w_dtype, void* out, long out_stride, int out_dtype, int T, int H,
                     int groups, float eps, const void* x_bias, int xb_dtype, cudaStream_t stream);
/* out = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u / sqrt(mean(u^2) + eps) over the row; coef [4] = (a, b, c, e). */
PHOTON_EXPORT int photon_polynorm(const void* z, long z_stride, int z_dtype, const void* coef, int coef_dtype, void* out,
                     long out_stride, int out_dtype, int T, int F, float eps, cudaStream_t stream);
/* x <- cap * tanh(x / cap) in place, `total` floats. */
PHOTON_EXPORT int photon_softcap(float* x, long total, float cap, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_diff.cu: two score maps per head over the same values */
/* q [T][H * 2 * d], k [T][G * 2 * d] (head by head: map 1, map 2), v [T][G * dv] of in_dtype.  Biases (b_dtype, may be null) are
 * added; every (head, map) of q and k is divided by its root mean square (eps inside the root) and multiplied by q_w / k_w [d]
 * (w_dtype, may be null); its first rot_dims numbers are rotated (number j with j + rot_dims / 2, angle positions[t] *
 * inv_freq[j]).  q_out [T][H * 2 * d] of out_dtype; keys go to k_cache [pages][G][page_size][2 d], values to v_cache
 * [pages][G][page_size][dv] at slot_mapping[t] (-1: nothing).  Null caches: queries only. */
PHOTON_EXPORT int photon_diff_prep(const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
                     int in_dtype, void* q_out, long qo_stride, int out_dtype, const void* q_b, const void* k_b, const void* v_b,
                     int b_dtype, const void* q_w, const void* k_w, int w_dtype, float eps, const int* positions,
                     const double* inv_freq, int rot_dims, const int* slot_mapping, void* k_cache, void* v_cache, int T, int H,
                     int G, int d, int dv, int page_size, long num_slots, int* err, cudaStream_t stream);
/* Per head: a_m = softmax_j((q_m . k_m) * scale) v over the keys the token sees, m = 1, 2; o = a_1 - lambda a_2;
 * out = o / sqrt(mean(o^2) + eps) * out_scale.  out [T][n_q * dv]. */
PHOTON_EXPORT int photon_diff_attention(const void* q, long q_stride, void* out, long out_stride, int dtype, const void* k_cache,
                     const void* v_cache, const int* block_table, int max_pages, const int* token_seq, const int* positions,
                     int T_, int n_q, int n_kv, int d, int dv, int page_size, int num_pages, int window, float scale,
                     float lambda, float out_scale, float eps, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_diff_mma.cu (-DDIFF_D=d -DDIFF_DV=dv, multiples of 16; bfloat16) */
PHOTON_EXPORT int photon_diff_mma_dims(void);                    /* d * 65536 + dv of this build */
/* photon_diff_attention on the tensor cores.  cu_tokens [S + 1]: the first token of every request of the step (a request's
 * tokens have consecutive positions); tiles: sum over the requests of ceil(tokens / (64 / (n_q / n_kv))).  splits > 1: the key
 * tiles of every block are shared out over that many blocks and put together by a second kernel; part: float scratch of
 * num_tokens * n_q * 2 * splits * (dv + 2). */
PHOTON_EXPORT int photon_diff_mma(const void* q, long q_stride, void* out, long out_stride, const void* k_cache, const void* v_cache,
                     const int* block_table, int max_pages, const int* cu_tokens, const int* positions, int num_seqs, int tiles,
                     int n_q, int n_kv, int page_size, int num_pages, int window, float scale, float lambda, float out_scale,
                     float eps, int splits, float* part, int num_tokens, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ linrec.cu: recurrences with one decay per head and token */
/* y float [T][C] = silu(bias + causal convolution over `taps` tokens per channel) of x [T][>= C] (x_dtype); taps_w float
 * [C][taps], the last column weighs the current token; the taps before a request's first token of the step come from its
 * state rows [taps - 1][C] at conv_offset of state [num_slots][state_stride] (slot -1: zeros). */
PHOTON_EXPORT int photon_conv_silu(const void* x, long x_stride, int x_dtype, const float* taps_w, const float* bias, int taps,
                     const int* token_seq, const int* cu_tokens, const int* state_slots, const float* state, long state_stride,
                     long conv_offset, int num_slots, float* y, int T, int C, int* err, cudaStream_t stream);
/* The last taps - 1 input rows of every request of the step become its state rows (slot -1: nothing is stored). */
PHOTON_EXPORT int photon_conv_state(const void* x, long x_stride, int x_dtype, int taps, const int* cu_tokens,
                     const int* state_slots, float* state, long state_stride, long conv_offset, int num_slots, int S, int C,
                     cudaStream_t stream);
/* S_t = keep_t S_(t-1) + take_t k_t v_t^T, o_t = S_t^T q_t per head (S [N][dv] in the request's state row).  mode 0: a
 * state-space layer (keep = exp(-exp(A_log) dt), take = dt = softplus(ga + dt_bias), out = o + D v; p0, p1, p2 = A_log,
 * dt_bias, D).  mode 1: a matrix memory with capped log gates and a running maximum (ga, gb the raw input and forget
 * gates, p0, p1 their biases; out = o / (max(|n . q|, exp(-m)) + 1e-6); n [H][N] and m [H] follow S in the state row). */
PHOTON_EXPORT int photon_linrec(int mode, const float* q, long q_stride, const float* k, long k_stride, const float* v,
                     long v_stride, const float* ga, const float* gb, long g_stride, const float* p0, const float* p1,
                     const float* p2, float cap, float q_scale, const int* cu_tokens, const int* state_slots, float* state,
                     long state_stride, int num_slots, float* out, long out_stride, int S, int H, int qk_heads, int N, int dv,
                     int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_talk.cu: attention whose heads' scores are mixed */
/* Bias (float, may be null) on q [T][H * d] and k [T][G * d] of in_dtype, rotation of the first rot_dims numbers of a head
 * (number j with j + rot_dims / 2, angle positions[t] * inv_freq[j]); q_out of out_dtype; the rotated key goes to k_cache, the
 * value to v_cache (may be null): v [T][G * d] or, with v null, the key before its rotation; both caches
 * [pages][G][page_size][d], written at slot_mapping[t] (-1: nothing). */
PHOTON_EXPORT int photon_talk_prep(const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
                     int in_dtype, const float* q_bias,
                     const float* k_bias, void* q_out, long qo_stride, int out_dtype, const int* positions,
                     const double* inv_freq, int rot_dims, const int* slot_mapping, void* k_cache, void* v_cache, int T, int H,
                     int G, int d, int page_size, long num_slots, int* err, cudaStream_t stream);
/* raw_g = (q_g . k) qmul[g]; s_h = sum_g talk[h][g] raw_g; softmax over the keys max(0, p - window + 1) .. p with exp(sink[h])
 * in the denominator; out_h = sigmoid(gate_h) sum_j p_h(j) v(j).  talk [H][H], sink [H], gate (float rows of H, stride
 * gate_stride) may be null; window 0: none; splits > 1: part float [T * splits * H * (d + 2)]. */
PHOTON_EXPORT int photon_talk_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                          const void* v_cache, int dtype, const int* block_table, int max_pages, const int* token_seq,
                          const int* positions, int T, int H, int G, int d, int page_size, int num_pages, int window,
                          const float* qmul, const float* talk, const float* sink, const float* gate, long gate_stride,
                          int splits, float* part, int* err, cudaStream_t stream);

/* Merges the shares that a token's splits left in part [T][splits][H][d + 2] (maximum as a natural logarithm, sum, d
 * weighted sums) in split order; then sink, gate and the division.  out [T][H * d] of dtype. */
PHOTON_EXPORT int photon_talk_merge(const float* part, int splits, void* out, long out_stride, int dtype, int T, int H, int d,
                      const float* sink, const float* gate, long gate_stride, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_talk_mma.cu: the same attention on the tensor cores */
/* bfloat16; the module is compiled for one (H, G, d) with -DTALK_H, -DTALK_G, -DHEAD_DIM and refuses others.  One block
 * per 16 neighbouring tokens of a request (cu_tokens [S + 1], at most max_tokens tokens a request) with all heads; splits >
 * 1: every split leaves its share in part [T * splits * H * (d + 2)] for photon_talk_merge and out is not written. */
PHOTON_EXPORT int photon_talk_mma(const void* q, long q_stride, void* out, long out_stride, const void* k_cache, const void* v_cache,
                    const int* block_table, int max_pages, const int* cu_tokens, const int* positions, int S, int max_tokens,
                    int H, int G, int d, int page_size, int num_pages, int window, const float* qmul, const float* talk,
                    const float* sink, const float* gate, long gate_stride, int splits, float* part, int* err,
                    cudaStream_t stream);

/* ------------------------------------------------------------------ gla.cu: gated linear attention (recurrent state) */
/* Per (request, head): S = diag(a_t) S + k_t v_t^T with a_t = sigmoid(z_t)^(1/tau), z_t = w_a2 low_t + b_a2, o_t = S^T (q_t *
 * qscale); out = o_t / rms(o_t) * norm_w * silu(g_t).  q, k [T][heads * dim], v, g [T][heads * vdim] and low [T][rank] share
 * one row stride; w_a2 [heads * dim][rank]; state [num_slots][heads][dim][vdim] float, read from and written to
 * state_slots[s] (negative: starts at zero, stores nothing). */
PHOTON_EXPORT int photon_gla_recurrent(const void* q, const void* k, const void* v, const void* g, const void* low, long in_stride,
                         int dtype, int rank, const void* w_a2, const void* b_a2, int b_a2_dtype, const void* norm_w,
                         int norm_w_dtype, float eps, float tau, float qscale, const int* cu_tokens, const int* state_slots,
                         float* state, int num_slots, void* out, long out_stride, int S, int heads, int dim, int vdim,
                         int skip_from, int* err, cudaStream_t stream);
/* One long prompt portion (tokens first .. first + count - 1 of the step, state slot `slot`, negative: from zero, nothing
 * stored) in chunks of `chunk` tokens that run side by side.  scratch: float [count * heads * (vdim + dim) + 4 +
 * ceil(count / chunk) * heads * dim * vdim], 16-byte aligned.  photon_gla_recurrent leaves requests of skip_from tokens or more
 * (skip_from > 0) to this path. */
PHOTON_EXPORT int photon_gla_chunked(const void* q, const void* k, const void* v, const void* g, const void* low, long in_stride,
                       int dtype, int rank, const void* w_a2, const void* b_a2, int b_a2_dtype, const void* norm_w,
                       int norm_w_dtype, float eps, float tau, float qscale, int first, int count, int chunk, int slot,
                       float* state, int num_slots, float* scratch, void* out, long out_stride, int heads, int dim, int vdim,
                       int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ moe.cu: routed experts */
/* Router: logits = Wr h + bias in 32-bit; ids/weights [T][top]: the top experts and the softmax over their logits;
 * counts [E]: pairs per expert. */
PHOTON_EXPORT int photon_moe_route(const void* h, long h_stride, int dtype, const void* Wr, const void* bias, int bias_dtype, int T_,
                     int H, int E, int top, int* ids, float* weights, int* counts, cudaStream_t stream);
/* mode 1: softmax over all experts, groups of neighbours of which only the keep_groups best (by their largest score) may
 * be chosen from, weights = chosen scores / (their sum + 1e-20) * route_scale.  mode 2: scores are sigmoid(logit), a group's
 * score is the sum of its two largest, weights = chosen scores * route_scale.  Wsg [H] (may be null): shared_gate [T] =
 * sigmoid(Wsg . h). */
PHOTON_EXPORT int photon_moe_route_ex(const void* h, long h_stride, int dtype, const void* Wr, const void* bias, int bias_dtype, int T_,
                        int H, int E, int top, int* ids, float* weights, int* counts, int mode, int n_groups, int keep_groups,
                        float route_scale, const void* Wsg, float* shared_gate, cudaStream_t stream);
/* Stable sort of the n = T * top pairs by expert: offsets [E + 1], sorted [n], place [n], tiles [3 * max_tiles] of
 * photon_moe_tile_rows() rows at most (expert, first row, rows), num_tiles [1]. */
PHOTON_EXPORT int photon_moe_align(const int* ids, const int* counts, int n, int E, int* offsets, int* sorted, int* place,
                     int* tiles, int* num_tiles, cudaStream_t stream);
PHOTON_EXPORT int photon_moe_tile_rows(void);
/* Grouped product over the sorted rows with W [E][N][K]; gather (may be null): sorted row r reads A row
 * gather[r] / gather_div; glu != 0: W = [gate rows; up rows], out [n][N / 2] = act(gate) * up. */
PHOTON_EXPORT int photon_moe_gemm(const void* A, long lda, int dtype, const int* gather, int gather_div, const void* W, void* out,
                    long ldo, int out_dtype, int N, int K, const int* tiles, const int* num_tiles, int max_tiles, int glu,
                    int act, cudaStream_t stream);
/* out[t] = sum_j weights[t, j] * y[place[t, j]] (+ shared_out[t]); y [n][H] float or bfloat16; place null: row t * top + j. */
PHOTON_EXPORT int photon_moe_combine(const void* y, long ldy, int y_dtype, const int* place, const float* weights, int top,
                       const void* shared_out, void* out, int out_dtype, int T_, int H, cudaStream_t stream);
/* shared_gate [T] (may be null) multiplies the shared expert's rows. */
PHOTON_EXPORT int photon_moe_combine_ex(const void* y, long ldy, int y_dtype, const int* place, const float* weights, int top,
                          const void* shared_out, const float* shared_gate, void* out, int out_dtype, int T_, int H,
                          cudaStream_t stream);
/* out[r, :] = x[sorted[r] / div, :]: the pairs' input rows in sorted order. */
PHOTON_EXPORT int photon_moe_gather(const void* x, long ldx, int dtype, const int* sorted, int div, void* out, int n, int H,
                      cudaStream_t stream);
/* Few pairs (decode steps), bfloat16: out[p] = W[ids[p]] x[p / x_div], one matrix-vector product per pair, unsorted;
 * glu as photon_moe_gemm. */
PHOTON_EXPORT int photon_moe_gemv(const void* x, long ldx, int x_div, const int* ids, int n, const void* W, void* out, long ldo,
                    int out_dtype, int N, int K, int glu, int act, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_flash.cu (-DHEAD_DIM=d, d % 16 == 0, <= 128; bfloat16) */
PHOTON_EXPORT int photon_flash_attention_head_dim(void);
PHOTON_EXPORT int photon_flash_attention_max_groups(void);
/* mode bit 0: requests with more than 16 rows (tokens x heads per key/value head); bit 1: the others, their keys
 * split over num_splits blocks (part_acc/part_ml: float scratch of T * n_q * num_splits * (d + 2); tickets: int
 * [S * n_kv], zero between launches) and over nsub groups of warps per block.  context_lens may be null. */
PHOTON_EXPORT int photon_flash_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                           const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                           const int* positions, const int* context_lens, float* part_acc, float* part_ml, int* tickets,
                           int S, int max_tokens_per_seq, int n_q, int n_kv, int d, int page_size, int num_pages,
                           int window, float scale, int num_splits, int nsub, int mode, int* err, cudaStream_t stream);
/* The same with kept first keys (with a window, keys < keep_first stay visible), a sink (one more key with score 0 and no
 * value) and bounded scores (softcap * tanh(score * scale / softcap); 0: off). */
PHOTON_EXPORT int photon_flash_attention_ex(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                              const int* positions, const int* context_lens, float* part_acc, float* part_ml, int* tickets,
                              int S, int max_tokens_per_seq, int n_q, int n_kv, int d, int page_size, int num_pages,
                              int window, float scale, int num_splits, int nsub, int mode, int* err, int keep_first,
                              int sink, float softcap, const void* gate, long gate_stride, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_tc.cu (-DHEAD_DIM=64|128; bfloat16; tcgen05) */
PHOTON_EXPORT int photon_attention_tc_head_dim(void);
/* Requests with more than 16 rows only; the others are left untouched. */
PHOTON_EXPORT int photon_attention_tc(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                        const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                        const int* positions, int S, int max_tokens_per_seq, int T, int n_q, int n_kv, int d,
                        int page_size, int num_pages, int window, float scale, int* err, cudaStream_t stream);
PHOTON_EXPORT int photon_attention_tc_ex(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                           const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                           const int* positions, int S, int max_tokens_per_seq, int T, int n_q, int n_kv, int d,
                           int page_size, int num_pages, int window, float scale, int* err, int keep_first, int sink,
                           float softcap, const void* gate, long gate_stride, cudaStream_t stream);

/* ------------------------------------------------------------------ attention_decode.cu (-DHEAD_DIM=64|128; bfloat16; TMA) */
PHOTON_EXPORT int photon_attention_decode_head_dim(void);
PHOTON_EXPORT int photon_attention_decode_slots(void);           /* blocks the current device holds at once (the kernel's grid) */
/* Requests with at most 16 rows only (S <= 512).  context_lens [S]: tokens of each request after this step.
 * chunk_tiles: tiles of 64 keys per work item (1..64); max_chunks_per_seq <= 120.  part_acc: float
 * [scratch_chunks * n_kv * 16 * d], part_ml: float [scratch_chunks * n_kv * 32]; scratch_chunks >= the chunks of
 * all requests together.  tickets: int [S * n_kv + 2], zero between launches.  max_items: bound of the work
 * items (sizes the grid; 0: as many blocks as fit). */
PHOTON_EXPORT int photon_attention_decode(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                            const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                            const int* context_lens, float* part_acc, float* part_ml, long scratch_chunks, int* tickets,
                            int S, int T, int n_q, int n_kv, int d, int page_size, int num_pages, int window,
                            float scale, int chunk_tiles, int max_chunks_per_seq, long max_items, int* err,
                            cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_f32.cu: true 32-bit product (FMA chain in ascending k) */
PHOTON_EXPORT int photon_sgemm_nt(const float* A, long lda, const float* W, long ldw, float* C, long ldc, int M, int N, int K,
                    cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny.cu: bfloat16, M <= 64 (32 with SwiGLU) */
/* epilogue 0: bfloat16 out; 1: float out; 2: SwiGLU (W = [gate rows; up rows], out [M, N / 2]).  K % 8 == 0,
 * 16-byte aligned rows.  scratch (float) and tickets (int, zero between launches) serve the split of K; launches
 * that share them must not overlap on the device. */
PHOTON_EXPORT int photon_skinny_gemm(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                       int epilogue, float* scratch, long scratch_floats, int* tickets, int num_tickets,
                       cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny_fused.cu: M <= 8 */
/* x = res_in + delta (res_out gets the sum when delta is given); out = epilogue(rmsnorm(x; norm_w, eps) W^T).
 * epilogue 0: bfloat16; 2: SwiGLU; 3: q/k/v with rotation (partners must be neighbouring rows of W) and cache write. */
PHOTON_EXPORT int photon_skinny_fused(const float* res_in, float* res_out, const void* delta, const void* norm_w, int norm_w_dtype,
                        float eps, const void* W, long ldw, void* out, long ldo, int M, int N, int K, int epilogue,
                        const int* positions, const float* inv_freq, const int* slot_mapping, void* k_cache,
                        void* v_cache, int n_q, int n_kv, int d, int page_size, long num_slots, int* err,
                        cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_skinny_static.cu: see gemm_skinny_static.h */
PHOTON_EXPORT const char* photon_static_error_string(int code);
PHOTON_EXPORT int photon_skinny_gemm_static(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                              int epilogue, cudaStream_t stream);

/* ------------------------------------------------------------------ gemm_tc.cu, gemm_tc2.cu: bfloat16 on tcgen05 (TMA, tensor memory) */
/* epilogue as photon_skinny_gemm.  gemm_tc: tiles of 128 x 256 on one SM; gemm_tc2: 256 x 256 on pairs of SMs. */
PHOTON_EXPORT int photon_gemm_tc(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                   int epilogue, int* err, cudaStream_t stream);
PHOTON_EXPORT int photon_gemm_tc2(const void* x, long ldx, const void* W, long ldw, void* out, long ldo, int M, int N, int K,
                    int epilogue, int* err, cudaStream_t stream);
/* x W^T with W = [q; k; v] rows (rotation partners as neighbours): rotated q to q_out [M, n_q * d], rotated k and v
 * to slot_mapping of the cache.  table (may be null): photon_rope_table output of table_positions positions. */
PHOTON_EXPORT int photon_gemm_tc2_qkv(const void* x, long ldx, const void* W, long ldw, void* q_out, long ldo, int M, int K,
                        const int* positions, const int* slot_mapping, const float* inv_freq, const void* table,
                        int table_positions, void* k_cache, void* v_cache, int n_q, int n_kv, int d, int page_size,
                        long num_slots, int* err, cudaStream_t stream);

/* ------------------------------------------------------------------ sampling.cu */
/* Per row: first maximum where temperature is null or <= 0, else the first index whose running sum of
 * softmax(logits / temperature) reaches u.  scratch: float [rows * 128] for V > 16384, else may be null. */
PHOTON_EXPORT int photon_sample(const float* logits, long ld, const float* temperature, const float* u, int* out, int rows, int V,
                  float* scratch, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PHOTON_KERNELS_H */
