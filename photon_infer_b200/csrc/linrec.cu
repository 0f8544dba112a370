// Recurrent mixers whose state is one matrix per head, S [N][dv] in 32-bit, that decays by ONE number per head and
// token and takes a rank-one update:
//
//   S_t = keep_t S_(t-1) + take_t k_t v_t^T,      o_t = S_t^T q_t                        (per head)
//
// Two mixers are this recurrence with different gates.
//
//   state-space (mode 0):  k = B_t, q = C_t (of the head's group), v = x_t;  dt = softplus(dt_raw + dt_bias[h]);
//                          keep = exp(-exp(A_log[h]) dt), take = dt;  y_t = o_t + D[h] x_t.
//   matrix memory (mode 1): log gates i = cap tanh((i_raw + b_i[h]) / cap), f = logsigmoid(cap tanh((f_raw + b_f[h]) / cap));
//                          a running maximum m (from 0): m_t = max(f + m_(t-1), i); keep = exp(f + m_(t-1) - m_t),
//                          take = exp(i - m_t); a vector n_t = keep n_(t-1) + take k_t rides along as one more
//                          column of S (with v = 1);  y_t = o_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6).
//
//   photon_conv_silu        y = silu(bias + causal convolution over `taps` tokens per channel); the taps before the
//                           step's first token of a request come from the request's state.
//   photon_conv_state       the last taps - 1 input rows of every request of the step go into its state.
//   photon_linrec           the recurrence over the tokens of a step, for all requests and heads.
//
// A request's state is one float row per layer; S [H][N][dv] comes first, then (mode 1) n [H][N] and m [H]; the
// convolution's rows live at an offset the caller gives.  A state slot of -1 starts from zeros and stores nothing.
// Every token's arithmetic is the same chain whatever the step brought before it, and the cut of a head's columns
// into blocks changes no column's arithmetic, so a request's numbers depend neither on how it was cut into steps nor
// on the batch.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------- short causal convolution
template <typename TI>
__global__ void __launch_bounds__(128)
conv_silu_kernel(const TI* __restrict__ x, long x_stride, const float* __restrict__ taps_w, const float* __restrict__ bias,
                 int taps, const int* __restrict__ token_seq, const int* __restrict__ cu_tokens,
                 const int* __restrict__ state_slots, const float* __restrict__ state, long state_stride, long conv_offset,
                 int num_slots, float* __restrict__ y, int C, int* err) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  const int s = token_seq[t];
  const int p = t - cu_tokens[s];                     // index of the token among the request's tokens of this step
  int slot = state_slots[s];
  if (slot >= num_slots) {
    if (c == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, slot, num_slots);
    slot = -1;
  }
  const float* old = slot >= 0 ? state + (size_t)slot * state_stride + conv_offset : nullptr;   // [taps - 1][C], oldest first
  float a = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;                    // tap j weighs the token `back` places before this one
    float xv;
    if (back <= p) xv = to_f32(x[(size_t)(t - back) * x_stride + c]);
    else xv = old ? old[(size_t)(taps - 1 - (back - p)) * C + c] : 0.f;
    a = fmaf(taps_w[(size_t)c * taps + j], xv, a);
  }
  y[(size_t)t * C + c] = a / (1.0f + expf(-a));
}

// x [T][>= C] of x_dtype (row stride x_stride), taps_w float [C][taps] (the last column weighs the current token), bias
// float [C] or null, y float [T][C].  state float [num_slots][state_stride]; the request's last taps - 1 input rows lie at
// conv_offset, oldest first.
PHOTON_API int photon_conv_silu(const void* x, long x_stride, int x_dtype, const float* taps_w, const float* bias, int taps,
                                const int* token_seq, const int* cu_tokens, const int* state_slots, const float* state,
                                long state_stride, long conv_offset, int num_slots, float* y, int T, int C, int* err,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || taps < 1 || x == nullptr || y == nullptr) return PHOTON_ERR_ARGUMENT;
  if (T > 65535) return PHOTON_ERR_UNSUPPORTED;
  dim3 grid((C + 127) / 128, T);
  if (x_dtype == PHOTON_BF16)
    conv_silu_kernel<bf16><<<grid, 128, 0, stream>>>((const bf16*)x, x_stride, taps_w, bias, taps, token_seq, cu_tokens, state_slots,
                                                     state, state_stride, conv_offset, num_slots, y, C, err);
  else
    conv_silu_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, x_stride, taps_w, bias, taps, token_seq, cu_tokens, state_slots,
                                                      state, state_stride, conv_offset, num_slots, y, C, err);
  return launch_status();
}

// The new rows of a request: the last taps - 1 of (its old rows, then the step's input rows).  A thread owns one channel
// of one request and reads all it needs before it writes, so the rows may move in place.
template <typename TI>
__global__ void __launch_bounds__(128)
conv_state_kernel(const TI* __restrict__ x, long x_stride, int taps, const int* __restrict__ cu_tokens,
                  const int* __restrict__ state_slots, float* __restrict__ state, long state_stride, long conv_offset,
                  int num_slots, int C) {
  const int s = blockIdx.y;
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  const int slot = state_slots[s];
  if (slot < 0 || slot >= num_slots) return;
  const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
  const int keep = taps - 1;
  float* rows = state + (size_t)slot * state_stride + conv_offset;
  constexpr int MAXK = 16;
  float tmp[MAXK];
  for (int r = 0; r < keep; ++r) {
    const int src = r + n;                            // index in (old rows, new rows)
    tmp[r] = src < keep ? rows[(size_t)src * C + c] : to_f32(x[(size_t)(t0 + src - keep) * x_stride + c]);
  }
  for (int r = 0; r < keep; ++r) rows[(size_t)r * C + c] = tmp[r];
}

PHOTON_API int photon_conv_state(const void* x, long x_stride, int x_dtype, int taps, const int* cu_tokens,
                                 const int* state_slots, float* state, long state_stride, long conv_offset, int num_slots,
                                 int S, int C, cudaStream_t stream) {
  if (S <= 0 || taps <= 1) return 0;
  if (taps - 1 > 16) return PHOTON_ERR_UNSUPPORTED;
  if (C <= 0 || S > 65535) return PHOTON_ERR_ARGUMENT;
  dim3 grid((C + 127) / 128, S);
  if (x_dtype == PHOTON_BF16)
    conv_state_kernel<bf16><<<grid, 128, 0, stream>>>((const bf16*)x, x_stride, taps, cu_tokens, state_slots, state, state_stride,
                                                      conv_offset, num_slots, C);
  else
    conv_state_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, x_stride, taps, cu_tokens, state_slots, state, state_stride,
                                                       conv_offset, num_slots, C);
  return launch_status();
}

// ---------------------------------------------------------------- the recurrence
// A block owns LR_COLS neighbouring columns of one (request, head): 8 lanes share a column, lane i of them holding rows
// i, i + 8, ... of it in registers (RPL rows a lane, N <= 8 RPL).  The step's tokens of the request come in chunks of
// LR_CHUNK: their keys, queries, the block's share of their values and their gates are staged in shared memory (one warp
// turns the raw gate inputs into keep and take, the running maximum in token order), then the walk over the chunk
// needs no barrier: per token RPL multiply-adds for the update, RPL for the read-out and three shuffles.  In mode 1
// the block's last column is the vector n (its value is 1), so every block knows n . q for its own columns.
#define LR_CHUNK 16
#define LR_COLS 16
#define LR_THREADS 128

__device__ __forceinline__ float lr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float lr_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <int MODE, int RPL>
__global__ void __launch_bounds__(LR_THREADS)
linrec_kernel(const float* __restrict__ q, long q_stride, const float* __restrict__ k, long k_stride,
              const float* __restrict__ v, long v_stride, const float* __restrict__ ga, const float* __restrict__ gb,
              long g_stride, const float* __restrict__ p0, const float* __restrict__ p1, const float* __restrict__ p2,
              float cap, float q_scale, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
              float* __restrict__ state, long state_stride, int num_slots, float* __restrict__ out, long out_stride,
              int H, int qk_heads, int N, int dv, int* err) {
  constexpr int NP = 8 * RPL;                          // rows with padding
  constexpr int REAL = MODE == 1 ? LR_COLS - 1 : LR_COLS;   // columns of S per block
  __shared__ float ks[LR_CHUNK][NP], qs[LR_CHUNK][NP], vs[LR_CHUNK][LR_COLS], os[LR_CHUNK][LR_COLS];
  __shared__ float keep_s[LR_CHUNK], take_s[LR_CHUNK], floor_s[LR_CHUNK], raw_a[LR_CHUNK], raw_b[LR_CHUNK];
  __shared__ float m_run;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane & 7;                            // this lane's place among the 8 lanes of its column
  const int col = warp * 4 + (lane >> 3);              // column within the block
  const int h = blockIdx.y, s = blockIdx.z;
  const int c0 = blockIdx.x * REAL;
  const bool is_n = MODE == 1 && col == LR_COLS - 1;   // the column that carries n
  const int c = c0 + col;                              // column of S
  const bool live = is_n || (col < REAL && c < dv);
  const int hq = h / (H / qk_heads);
  int slot = state_slots[s];
  if (slot >= num_slots) {
    if (tid == 0 && blockIdx.x == 0 && h == 0) report_error(err, PHOTON_DEV_BAD_SLOT, s, slot, num_slots);
    slot = -1;
  }
  float* st = slot >= 0 ? state + (size_t)slot * state_stride : nullptr;
  float* S_h = st ? st + (size_t)h * N * dv : nullptr;
  float* n_h = (st && MODE == 1) ? st + (size_t)H * N * dv + (size_t)h * N : nullptr;
  float* m_h = (st && MODE == 1) ? st + (size_t)H * N * dv + (size_t)H * N + h : nullptr;

  float S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = sub + 8 * i;
    float x = 0.f;
    if (st && live && r < N) x = is_n ? n_h[r] : S_h[(size_t)r * dv + c];
    S[i] = x;
  }
  if (tid == 0) m_run = (MODE == 1 && m_h) ? *m_h : 0.f;
  const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
  const float a_h = MODE == 0 ? expf(p0[h]) : 0.f;     // the head's decay rate
  for (int base = t0; base < t1; base += LR_CHUNK) {
    const int cnt = min(LR_CHUNK, t1 - base);
    __syncthreads();                                   // the chunk before is written out; m_run is set
    for (int i = tid; i < LR_CHUNK * NP; i += LR_THREADS) {
      const int tt = i / NP, r = i - tt * NP;
      float kv = 0.f, qv = 0.f;
      if (tt < cnt && r < N) {
        kv = k[(size_t)(base + tt) * k_stride + (size_t)hq * N + r];
        qv = q[(size_t)(base + tt) * q_stride + (size_t)hq * N + r] * q_scale;
      }
      ks[tt][r] = kv;
      qs[tt][r] = qv;
    }
    for (int i = tid; i < LR_CHUNK * LR_COLS; i += LR_THREADS) {
      const int tt = i / LR_COLS, cc = i - tt * LR_COLS;
      float x = 0.f;
      if (MODE == 1 && cc == LR_COLS - 1) x = 1.f;
      else if (tt < cnt && cc < REAL && c0 + cc < dv) x = v[(size_t)(base + tt) * v_stride + (size_t)h * dv + c0 + cc];
      vs[tt][cc] = x;
    }
    if (tid < LR_CHUNK) {
      float a = 0.f, b = 0.f;
      if (tid < cnt) {
        a = ga[(size_t)(base + tid) * g_stride + h];
        if (MODE == 1) b = gb[(size_t)(base + tid) * g_stride + h];
      }
      if (MODE == 0) {
        const float dt = lr_softplus(a + p1[h]);
        keep_s[tid] = expf(-a_h * dt);
        take_s[tid] = dt;
      } else {
        raw_a[tid] = cap * tanhf((a + p0[h]) / cap);                       // log input gate
        raw_b[tid] = lr_logsigmoid(cap * tanhf((b + p1[h]) / cap));        // log forget gate
      }
    }
    if (MODE == 1) {
      __syncthreads();
      if (tid == 0) {
        float m = m_run;
        for (int tt = 0; tt < cnt; ++tt) {
          const float fm = raw_b[tt] + m;
          const float mn = fmaxf(fm, raw_a[tt]);
          keep_s[tt] = expf(fm - mn);
          take_s[tt] = expf(raw_a[tt] - mn);
          floor_s[tt] = expf(-mn);
          m = mn;
        }
        m_run = m;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float keep = keep_s[tt];
      const float w = take_s[tt] * vs[tt][col];
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        const int r = sub + 8 * i;
        S[i] = fmaf(ks[tt][r], w, keep * S[i]);
        if (i & 1) a1 = fmaf(S[i], qs[tt][r], a1); else a0 = fmaf(S[i], qs[tt][r], a0);
      }
      float a = a0 + a1;
      a += __shfl_xor_sync(0xffffffffu, a, 1);
      a += __shfl_xor_sync(0xffffffffu, a, 2);
      a += __shfl_xor_sync(0xffffffffu, a, 4);
      if (sub == 0) os[tt][col] = a;
    }
    __syncthreads();
    for (int i = tid; i < cnt * REAL; i += LR_THREADS) {
      const int tt = i / REAL, cc = i - tt * REAL;
      if (c0 + cc >= dv) continue;
      float y = os[tt][cc];
      if (MODE == 0) y = fmaf(p2[h], vs[tt][cc], y);
      else y = y / (fmaxf(fabsf(os[tt][LR_COLS - 1]), floor_s[tt]) + 1e-6f);
      out[(size_t)(base + tt) * out_stride + (size_t)h * dv + c0 + cc] = y;
    }
  }
  if (st && live) {
    if (!is_n) {
#pragma unroll
      for (int i = 0; i < RPL; ++i) { const int r = sub + 8 * i; if (r < N) S_h[(size_t)r * dv + c] = S[i]; }
    } else if (blockIdx.x == 0) {
#pragma unroll
      for (int i = 0; i < RPL; ++i) { const int r = sub + 8 * i; if (r < N) n_h[r] = S[i]; }
    }
  }
  __syncthreads();
  if (MODE == 1 && m_h && tid == 0 && blockIdx.x == 0) *m_h = m_run;
}

template <int MODE>
static int linrec_launch(int rpl, dim3 grid, cudaStream_t stream, const float* q, long q_stride, const float* k, long k_stride,
                         const float* v, long v_stride, const float* ga, const float* gb, long g_stride, const float* p0,
                         const float* p1, const float* p2, float cap, float q_scale, const int* cu_tokens,
                         const int* state_slots, float* state, long state_stride, int num_slots, float* out, long out_stride,
                         int H, int qk_heads, int N, int dv, int* err) {
#define LR_GO(R) linrec_kernel<MODE, R><<<grid, LR_THREADS, 0, stream>>>(q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, \
      p2, cap, q_scale, cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, err)
  if (rpl <= 2) LR_GO(2);
  else if (rpl <= 4) LR_GO(4);
  else if (rpl <= 6) LR_GO(6);
  else if (rpl <= 8) LR_GO(8);
  else if (rpl <= 12) LR_GO(12);
  else if (rpl <= 16) LR_GO(16);
  else if (rpl <= 24) LR_GO(24);
  else if (rpl <= 32) LR_GO(32);
  else return PHOTON_ERR_UNSUPPORTED;
  return launch_status();
}

// q, k: float [T][qk_heads * N] views (row strides in elements); v float [T][H * dv]; ga, gb: float [T][H] views with row
// stride g_stride, the raw gate inputs (mode 0: ga = dt_raw, gb unused; mode 1: ga = i_raw, gb = f_raw).  p0, p1, p2: float
// [H] (mode 0: A_log, dt_bias, D; mode 1: the input gate's bias, the forget gate's bias, unused).  cap: the gates' bound
// (mode 1).  q_scale multiplies the queries.  out float [T][H * dv] (row stride out_stride).  Head h reads query/key head
// h / (H / qk_heads).  state: float [num_slots][state_stride], see the top of the file.
PHOTON_API int photon_linrec(int mode, const float* q, long q_stride, const float* k, long k_stride, const float* v,
                             long v_stride, const float* ga, const float* gb, long g_stride, const float* p0, const float* p1,
                             const float* p2, float cap, float q_scale, const int* cu_tokens, const int* state_slots,
                             float* state, long state_stride, int num_slots, float* out, long out_stride, int S, int H,
                             int qk_heads, int N, int dv, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (mode != 0 && mode != 1) return PHOTON_ERR_ARGUMENT;
  if (H <= 0 || qk_heads <= 0 || H % qk_heads || N <= 0 || dv <= 0) return PHOTON_ERR_ARGUMENT;
  if (mode == 1 && !(cap > 0.f)) return PHOTON_ERR_ARGUMENT;
  if (N > 256 || H > 65535 || S > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int rpl = (N + 7) / 8;
  const int real = mode == 1 ? LR_COLS - 1 : LR_COLS;
  dim3 grid((dv + real - 1) / real, H, S);
  if (mode == 0)
    return linrec_launch<0>(rpl, grid, stream, q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap, q_scale,
                            cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, err);
  return linrec_launch<1>(rpl, grid, stream, q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap, q_scale,
                          cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, err);
}
