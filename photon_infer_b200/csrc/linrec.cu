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
// i RPL .. i RPL + RPL - 1 of it in registers (RPL a multiple of 4, N <= 8 RPL).  The step's tokens of the request come in
// chunks of LR_CHUNK: their keys, queries, the block's share of their values and their raw gates arrive by cp.async in
// one of two stages of shared memory while the chunk before is walked; one warp turns the raw gates into keep and take
// (the running maximum in token order); then the walk over the chunk needs no barrier and no shuffle: per token RPL
// multiply-adds for the update and RPL for the read-out (operands fetched 16 bytes at a time); the eight lanes' shares of
// a column's read-out meet when the chunk is written out.  In mode 1 the block's last column is the vector n (its value
// is 1), so every block knows n . q for its own columns.
#define LR_CHUNK 16
#define LR_COLS 16
#define LR_THREADS 128

__device__ __forceinline__ float lr_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float lr_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ void lr_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void lr_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void lr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K> __device__ __forceinline__ void lr_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }

// Eight shares of one sum, added in a fixed order.
__device__ __forceinline__ float lr_sum8(const float* p) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  return ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
}

template <int MODE, int RPL>
__global__ void __launch_bounds__(LR_THREADS)
linrec_kernel(const float* __restrict__ q, long q_stride, const float* __restrict__ k, long k_stride,
              const float* __restrict__ v, long v_stride, const float* __restrict__ ga, const float* __restrict__ gb,
              long g_stride, const float* __restrict__ p0, const float* __restrict__ p1, const float* __restrict__ p2,
              float cap, float q_scale, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
              float* __restrict__ state, long state_stride, int num_slots, float* __restrict__ out, long out_stride,
              int H, int qk_heads, int N, int dv, int vec, int* err) {
  constexpr int NPS = 8 * (RPL + 4);                   // a staged row: 8 lanes' rows, each lane's share 16 bytes further on
  constexpr int REAL = MODE == 1 ? LR_COLS - 1 : LR_COLS;   // columns of S per block
  extern __shared__ __align__(16) float lr_smem[];
  float* ks = lr_smem;                                 // [2][CHUNK][NPS]
  float* qs = ks + 2 * LR_CHUNK * NPS;                 // [2][CHUNK][NPS]
  float* vs = qs + 2 * LR_CHUNK * NPS;                 // [2][CHUNK][COLS]
  float* raw = vs + 2 * LR_CHUNK * LR_COLS;            // [2][2][CHUNK]: the raw gates
  __shared__ __align__(16) float os[LR_CHUNK][LR_COLS][8];
  __shared__ float keep_s[LR_CHUNK], take_s[LR_CHUNK], floor_s[LR_CHUNK];
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
    const int r = sub * RPL + i;
    float x = 0.f;
    if (st && live && r < N) x = is_n ? n_h[r] : S_h[(size_t)r * dv + c];
    S[i] = x;
  }
  if (tid == 0) m_run = (MODE == 1 && m_h) ? *m_h : 0.f;
  // what no copy writes stays as it is set here: rows beyond N, columns beyond the head, the value 1 of the n column
  for (int i = tid; i < 2 * LR_CHUNK * NPS; i += LR_THREADS) { ks[i] = 0.f; qs[i] = 0.f; }
  for (int i = tid; i < 2 * LR_CHUNK * LR_COLS; i += LR_THREADS) vs[i] = (MODE == 1 && (i % LR_COLS) == LR_COLS - 1) ? 1.f : 0.f;
  for (int i = tid; i < 4 * LR_CHUNK; i += LR_THREADS) raw[i] = 0.f;
  __syncthreads();
  const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
  const float a_h = MODE == 0 ? expf(p0[h]) : 0.f;     // the head's decay rate

  auto issue = [&](int base, int stage) {
    const int cnt = min(LR_CHUNK, t1 - base);
    float* kd = ks + (size_t)stage * LR_CHUNK * NPS;
    float* qd = qs + (size_t)stage * LR_CHUNK * NPS;
    if (vec) {
      const int per = N / 4;                           // 16-byte pieces of a row; a piece never straddles two lanes' shares
      for (int i = tid; i < cnt * per; i += LR_THREADS) {
        const int tt = i / per, r = (i - tt * per) * 4;
        const int at = tt * NPS + r + (r / RPL) * 4;
        lr_cp16(kd + at, k + (size_t)(base + tt) * k_stride + (size_t)hq * N + r);
        lr_cp16(qd + at, q + (size_t)(base + tt) * q_stride + (size_t)hq * N + r);
      }
    } else {
      for (int i = tid; i < cnt * N; i += LR_THREADS) {
        const int tt = i / N, r = i - tt * N;
        const int at = tt * NPS + r + (r / RPL) * 4;
        lr_cp4(kd + at, k + (size_t)(base + tt) * k_stride + (size_t)hq * N + r);
        lr_cp4(qd + at, q + (size_t)(base + tt) * q_stride + (size_t)hq * N + r);
      }
    }
    const int ncol = min(REAL, dv - c0);
    float* vd = vs + (size_t)stage * LR_CHUNK * LR_COLS;
    for (int i = tid; i < cnt * ncol; i += LR_THREADS) {
      const int tt = i / ncol, cc = i - tt * ncol;
      lr_cp4(vd + tt * LR_COLS + cc, v + (size_t)(base + tt) * v_stride + (size_t)h * dv + c0 + cc);
    }
    float* rd = raw + (size_t)stage * 2 * LR_CHUNK;
    if (tid < cnt) lr_cp4(rd + tid, ga + (size_t)(base + tid) * g_stride + h);
    else if (MODE == 1 && tid >= 32 && tid < 32 + cnt) lr_cp4(rd + LR_CHUNK + tid - 32, gb + (size_t)(base + tid - 32) * g_stride + h);
    lr_commit();
  };

  if (t0 < t1) issue(t0, 0);
  int stage = 0;
  for (int base = t0; base < t1; base += LR_CHUNK, stage ^= 1) {
    const int cnt = min(LR_CHUNK, t1 - base);
    __syncthreads();                                   // the chunk before is written out: the other stage is free
    if (base + LR_CHUNK < t1) { issue(base + LR_CHUNK, stage ^ 1); lr_wait<1>(); } else lr_wait<0>();
    __syncthreads();                                   // this chunk has landed for every thread
    const float* kd = ks + (size_t)stage * LR_CHUNK * NPS;
    const float* qd = qs + (size_t)stage * LR_CHUNK * NPS;
    const float* vd = vs + (size_t)stage * LR_CHUNK * LR_COLS;
    const float* rd = raw + (size_t)stage * 2 * LR_CHUNK;
    if (MODE == 0) {
      if (tid < cnt) {
        const float dt = lr_softplus(rd[tid] + p1[h]);
        keep_s[tid] = expf(-a_h * dt);
        take_s[tid] = dt;
      }
    } else if (warp == 0) {
      float gi = 0.f, gf = 0.f;
      if (lane < cnt) {
        gi = cap * tanhf((rd[lane] + p0[h]) / cap);                          // log input gate
        gf = lr_logsigmoid(cap * tanhf((rd[LR_CHUNK + lane] + p1[h]) / cap));  // log forget gate
      }
      float m = m_run, fm_mine = 0.f, mn_mine = 0.f;
      for (int tt = 0; tt < cnt; ++tt) {               // the running maximum, in token order (every lane walks it)
        const float fi = __shfl_sync(0xffffffffu, gi, tt), ff = __shfl_sync(0xffffffffu, gf, tt);
        const float fm = ff + m;
        const float mn = fmaxf(fm, fi);
        if (lane == tt) { fm_mine = fm; mn_mine = mn; }
        m = mn;
      }
      if (lane < cnt) { keep_s[lane] = expf(fm_mine - mn_mine); take_s[lane] = expf(gi - mn_mine); floor_s[lane] = expf(-mn_mine); }
      if (lane == 0) m_run = m;
    }
    __syncthreads();
    const float* kl = kd + sub * (RPL + 4);
    const float* ql = qd + sub * (RPL + 4);
#pragma unroll 4
    for (int tt = 0; tt < cnt; ++tt) {
      const float keep = keep_s[tt];
      const float w = take_s[tt] * vd[tt * LR_COLS + col];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int j = 0; j < RPL / 4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(kl + tt * NPS + 4 * j);
        const float4 q4 = *reinterpret_cast<const float4*>(ql + tt * NPS + 4 * j);
        S[4 * j + 0] = fmaf(k4.x, w, keep * S[4 * j + 0]);
        S[4 * j + 1] = fmaf(k4.y, w, keep * S[4 * j + 1]);
        S[4 * j + 2] = fmaf(k4.z, w, keep * S[4 * j + 2]);
        S[4 * j + 3] = fmaf(k4.w, w, keep * S[4 * j + 3]);
        a0 = fmaf(S[4 * j + 0], q4.x, a0);
        a1 = fmaf(S[4 * j + 1], q4.y, a1);
        a2 = fmaf(S[4 * j + 2], q4.z, a2);
        a3 = fmaf(S[4 * j + 3], q4.w, a3);
      }
      os[tt][col][sub] = (a0 + a1) + (a2 + a3);         // the eight lanes' shares of a column meet after the walk
    }
    __syncthreads();
    for (int i = tid; i < cnt * REAL; i += LR_THREADS) {
      const int tt = i / REAL, cc = i - tt * REAL;
      if (c0 + cc >= dv) continue;
      float y = lr_sum8(os[tt][cc]) * q_scale;         // the queries' factor, taken out of the sums
      if (MODE == 0) y = fmaf(p2[h], vd[tt * LR_COLS + cc], y);
      else y = y / (fmaxf(fabsf(lr_sum8(os[tt][LR_COLS - 1]) * q_scale), floor_s[tt]) + 1e-6f);
      out[(size_t)(base + tt) * out_stride + (size_t)h * dv + c0 + cc] = y;
    }
  }
  if (st && live) {
    if (!is_n) {
#pragma unroll
      for (int i = 0; i < RPL; ++i) { const int r = sub * RPL + i; if (r < N) S_h[(size_t)r * dv + c] = S[i]; }
    } else if (blockIdx.x == 0) {
#pragma unroll
      for (int i = 0; i < RPL; ++i) { const int r = sub * RPL + i; if (r < N) n_h[r] = S[i]; }
    }
  }
  __syncthreads();
  if (MODE == 1 && m_h && tid == 0 && blockIdx.x == 0) *m_h = m_run;
}

template <int MODE, int RPL>
static int linrec_go(dim3 grid, cudaStream_t stream, const float* q, long q_stride, const float* k, long k_stride, const float* v,
                     long v_stride, const float* ga, const float* gb, long g_stride, const float* p0, const float* p1,
                     const float* p2, float cap, float q_scale, const int* cu_tokens, const int* state_slots, float* state,
                     long state_stride, int num_slots, float* out, long out_stride, int H, int qk_heads, int N, int dv, int vec,
                     int* err) {
  const size_t smem = ((size_t)4 * LR_CHUNK * 8 * (RPL + 4) + 2 * LR_CHUNK * LR_COLS + 4 * LR_CHUNK) * sizeof(float);
  if (smem > 36 * 1024) {                              // with the 9 KB of static arrays this passes the default limit
    cudaError_t e = cudaFuncSetAttribute(linrec_kernel<MODE, RPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  linrec_kernel<MODE, RPL><<<grid, LR_THREADS, smem, stream>>>(q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap,
      q_scale, cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, vec, err);
  return launch_status();
}

template <int MODE>
static int linrec_launch(int rpl, dim3 grid, cudaStream_t stream, const float* q, long q_stride, const float* k, long k_stride,
                         const float* v, long v_stride, const float* ga, const float* gb, long g_stride, const float* p0,
                         const float* p1, const float* p2, float cap, float q_scale, const int* cu_tokens,
                         const int* state_slots, float* state, long state_stride, int num_slots, float* out, long out_stride,
                         int H, int qk_heads, int N, int dv, int* err) {
  // 16-byte copies of keys and queries when every row piece is aligned
  const int vec = (N % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0) ? 1 : 0;
#define LR_GO(R) return linrec_go<MODE, R>(grid, stream, q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap, q_scale, \
      cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, vec, err)
  if (rpl <= 4) LR_GO(4);
  if (rpl <= 8) LR_GO(8);
  if (rpl <= 12) LR_GO(12);
  if (rpl <= 16) LR_GO(16);
  if (rpl <= 24) LR_GO(24);
  if (rpl <= 32) LR_GO(32);
  if (rpl <= 48) LR_GO(48);
  if (rpl <= 64) LR_GO(64);
  return PHOTON_ERR_UNSUPPORTED;
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
  if (N > 512 || H > 65535 || S > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int rpl = (N + 7) / 8;
  const int real = mode == 1 ? LR_COLS - 1 : LR_COLS;
  dim3 grid((dv + real - 1) / real, H, S);
  if (mode == 0)
    return linrec_launch<0>(rpl, grid, stream, q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap, q_scale,
                            cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, err);
  return linrec_launch<1>(rpl, grid, stream, q, q_stride, k, k_stride, v, v_stride, ga, gb, g_stride, p0, p1, p2, cap, q_scale,
                          cu_tokens, state_slots, state, state_stride, num_slots, out, out_stride, H, qk_heads, N, dv, err);
}
