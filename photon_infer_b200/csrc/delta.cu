// Gated delta rule: a recurrent mixer whose state is one matrix per head, S [dim][vdim] in 32-bit, with short
// causal convolutions in front of it.
//
//   x = [W_q h ; W_k h ; W_v h]                         the projected row of a token, C = 2 Gq dim + H vdim channels
//   y_c(t) = silu(sum_i w[c][i] x_c(t - taps + 1 + i))  per channel, zeros before the start of the sequence
//   q, k: per query/key head, y / sqrt(sum(y^2) + 1e-6); q also times dim^(-1/2); v = y
//   beta = sigmoid(b), g = exp(-exp(A_log[h]) * softplus(a + dt_bias[h]))            one of each per head and token
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                       (head h uses q/k head h / (H / Gq))
//   out = o / sqrt(mean(o^2) + eps) * norm_w * silu(z)                                   per head over vdim
//
// The state of a request is one float row per layer: S [H][dim][vdim], then the last taps - 1 projected rows
// [taps - 1][C] (oldest first).  A state slot of -1 starts from zeros and stores nothing.  Everything after the
// projections is 32-bit; a request's result does not depend on how it was cut into steps, because every token's
// arithmetic is the same chain whatever the step brought before it.
//
// The recurrence is evaluated in the equivalent form
//   P1 = S^T k, P2 = S^T q (old state), u = beta (v - g P1), o = g P2 + u (k . q), S <- g S + k u^T,
// which needs one pass over the state for the two products and one for the update.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------- convolution, silu, unit vectors
// One warp per (token, segment); a segment is one q head, one k head (dim channels, made a unit vector) or one v head
// (vdim channels).  The taps before the step's first token of the request come from the state.  A lane keeps up to
// HOLD results until the head's norm is known (heads up to 32 * HOLD wide; wider ones are scaled in a second pass).
template <typename TI>
__global__ void __launch_bounds__(128)
delta_conv_kernel(const TI* __restrict__ x, long x_stride, const float* __restrict__ taps_w, int taps,
                  const int* __restrict__ token_seq, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
                  const float* __restrict__ state, long state_stride, long conv_offset, int num_slots,
                  float* __restrict__ y, int Gq, int H, int dim, int vdim, int* err) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.y, seg = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (seg >= 2 * Gq + H) return;
  const int C = 2 * Gq * dim + H * vdim;
  const bool unit = seg < 2 * Gq;
  const int width = unit ? dim : vdim;
  const int c0 = unit ? seg * dim : 2 * Gq * dim + (seg - 2 * Gq) * vdim;
  const int s = token_seq[t];
  const int p = t - cu_tokens[s];                     // index of the token among the request's tokens of this step
  int slot = state_slots[s];
  if (slot >= num_slots) {
    if (lane == 0 && seg == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, slot, num_slots);
    slot = -1;
  }
  const float* old = slot >= 0 ? state + (size_t)slot * state_stride + conv_offset : nullptr;
  float ss = 0.f;
  constexpr int HOLD = 8;
  const bool hold = unit && width <= HOLD * 32;
  float kept[HOLD];
#pragma unroll
  for (int n = 0; n < HOLD; ++n) {
    const int i = lane + n * 32;
    if (i >= width) break;
    const int c = c0 + i;
    float a = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                  // tap j weighs the token `back` places before this one
      float xv;
      if (back <= p) xv = to_f32(x[(size_t)(t - back) * x_stride + c]);
      else xv = old ? old[(size_t)(taps - 1 - (back - p)) * C + c] : 0.f;
      a = fmaf(taps_w[(size_t)c * taps + j], xv, a);
    }
    a = a / (1.0f + expf(-a));
    kept[n] = a;
    if (!hold) y[(size_t)t * C + c] = a;
    ss += a * a;
  }
  for (int i = lane + HOLD * 32; i < width; i += 32) {  // the rest of a very wide segment
    const int c = c0 + i;
    float a = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      float xv;
      if (back <= p) xv = to_f32(x[(size_t)(t - back) * x_stride + c]);
      else xv = old ? old[(size_t)(taps - 1 - (back - p)) * C + c] : 0.f;
      a = fmaf(taps_w[(size_t)c * taps + j], xv, a);
    }
    a = a / (1.0f + expf(-a));
    y[(size_t)t * C + c] = a;
    ss += a * a;
  }
  if (!unit) return;
  ss = warp_sum(ss);
  const float inv = (seg < Gq ? rsqrtf((float)dim) : 1.0f) / sqrtf(ss + 1e-6f);
  if (hold) {
#pragma unroll
    for (int n = 0; n < HOLD; ++n) {
      const int i = lane + n * 32;
      if (i < width) y[(size_t)t * C + c0 + i] = kept[n] * inv;
    }
    return;
  }
  __syncwarp();
  for (int i = lane; i < width; i += 32) y[(size_t)t * C + c0 + i] *= inv;
}

// The last taps - 1 projected rows of every request, after this step: thread per (request, channel).
template <typename TI>
__global__ void delta_conv_state_kernel(const TI* __restrict__ x, long x_stride, int taps, const int* __restrict__ cu_tokens,
                                        const int* __restrict__ state_slots, float* __restrict__ state, long state_stride,
                                        long conv_offset, int num_slots, int C) {
  pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = state_slots[s];
  if (c >= C || slot < 0 || slot >= num_slots) return;
  const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
  if (n <= 0) return;
  float* cs = state + (size_t)slot * state_stride + conv_offset;
  const int keep = taps - 1;
  // new row r (oldest first) is place n - keep + r of the step when that is >= 0, else old row r + n
  for (int r = 0; r < keep; ++r) {               // ascending r reads old rows r + n > r: nothing read after it is overwritten
    const int at = n - keep + r;
    cs[(size_t)r * C + c] = at >= 0 ? to_f32(x[(size_t)(t0 + at) * x_stride + c]) : cs[(size_t)(r + n) * C + c];
  }
}

// ---------------------------------------------------------------- the recurrence
// The columns of a head's state never meet: column j needs k, q, the two per-head numbers and v_j alone.  So one block
// owns `vcols` neighbouring columns of one (request, head), and the launcher cuts a head into as many groups of columns
// as fill the GPU.  Thread jl * RP + r holds the rows (i * RP + r) * 4 .. + 3, i < RPT / 4, of its column in registers
// (neighbouring lanes read neighbouring quads of k and q: no bank conflicts); the RP partial sums of a column
// lie in neighbouring lanes and meet by shuffles, in an order that depends on (RPT, RP) alone, which the launcher
// picks from dim alone: a column's arithmetic is the same chain however the head was cut and whatever else the
// step holds.  The inputs of CH tokens are staged in shared memory (the next chunk's are fetched into registers while
// the current one is computed), so the walk meets one barrier per chunk.
#define DELTA_CH 16

// a token in shared memory: q [dimp], k [dimp], v [vcols, padded to 4], then g, beta and two spare numbers
static inline int delta_tok_floats(int dimp, int vcols) { return 2 * dimp + ((vcols + 3) & ~3) + 4; }   // rows stay 16-byte aligned

__device__ __forceinline__ void delta_cp4(float* dst, const float* src, bool valid) {
  const int n = valid ? 4 : 0;                            // 0: the four bytes become zero, nothing is read
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n) : "memory");
}

template <int RPT, int RP>
__global__ void __launch_bounds__(320)
delta_recurrent_kernel(const float* __restrict__ y, const float* x_ab, long ab_stride, int ab_dtype_bf16,
                       const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                       const int* __restrict__ cu_tokens, const int* __restrict__ state_slots, float* __restrict__ state,
                       long state_stride, int num_slots, float* __restrict__ o_out, int Gq, int H, int dim, int vdim, int vcols,
                       int* err) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, cg = blockIdx.z;
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
  if (t1 <= t0) return;
  const int slot = state_slots[s];
  if (slot >= num_slots) {
    if (tid == 0 && cg == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t0, slot, num_slots);
    return;
  }
  const int C = 2 * Gq * dim + H * vdim;
  constexpr int dimp = RPT * RP;                          // rows padded to whole groups; the padding stays zero
  const int jl = tid / RP, r = tid % RP;
  const int j = cg * vcols + jl;                          // the thread's column of the head
  const bool active = jl < vcols && j < vdim;
  const int hq = h / (H / Gq);
  auto row_of = [&](int i) { return ((i >> 2) * RP + r) * 4 + (i & 3); };      // the state row in register i
  float* S = slot >= 0 ? state + (size_t)slot * state_stride + (size_t)h * dim * vdim : nullptr;
  float2 st[RPT / 2];                                     // pairs of neighbouring rows: the arithmetic below is packed
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const float v = (S != nullptr && active && row_of(i) < dim) ? S[(size_t)row_of(i) * vdim + j] : 0.f;
    if (i & 1) st[i >> 1].y = v; else st[i >> 1].x = v;
  }
  const int vpad = (vcols + 3) & ~3;
  const int per_tok = 2 * dimp + vpad + 4;
  const int buf_floats = DELTA_CH * per_tok;
  float* kqs = sm + 2 * buf_floats + warp * DELTA_CH;     // k . q of the chunk's tokens, a copy per warp
  float* obuf = sm + 2 * buf_floats + (nthreads >> 5) * DELTA_CH;     // the chunk's read-outs [CH][vpad], written out a chunk at a time
  for (int i = tid; i < 2 * buf_floats; i += nthreads) sm[i] = 0.f;
  const float decay_rate = expf(a_log[h]), bias = dt_bias[h];
  // The warps behind the ones that own columns do nothing but fetch: every token's q | k | the block's columns of v.
  const int nwork = (vcols * RP + 31) / 32;               // warps that walk
  const int ftid = tid - nwork * 32, nfetch = nthreads - nwork * 32;
  const int rowlen = 2 * dim + vcols;
  float pre_ab = 0.f;                                     // fetch threads 0 .. 2 CH - 1: a token's raw decay or step-size input
  bool ab_live = false;
  // the chunk that starts at token c0 travels into buffer `buf` (cp.async); the two per-head numbers come raw into a
  // register and are turned into g and beta when they are stored, so that no thread waits for a load before the walk
  auto fetch = [&](int c0, int buf) {
    if (ftid < 0) return;
    float* b = sm + buf * buf_floats;
    for (int w = ftid; w < rowlen; w += nfetch) {
      int src_col, dst_at;
      if (w < dim) { src_col = hq * dim + w; dst_at = w; }
      else if (w < 2 * dim) { src_col = (Gq + hq) * dim + (w - dim); dst_at = dimp + (w - dim); }
      else if (cg * vcols + (w - 2 * dim) < vdim) { src_col = 2 * Gq * dim + h * vdim + cg * vcols + (w - 2 * dim); dst_at = 2 * dimp + (w - 2 * dim); }
      else continue;
      const float* src = y + (size_t)c0 * C + src_col;
      float* dst = b + dst_at;
#pragma unroll
      for (int tt = 0; tt < DELTA_CH; ++tt) delta_cp4(dst + tt * per_tok, src + (size_t)tt * C, c0 + tt < t1);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (ftid < 2 * DELTA_CH) {
      const int t = c0 + (ftid >> 1);
      pre_ab = 0.f; ab_live = t < t1;
      if (ab_live) {
        const size_t at = (size_t)t * ab_stride + ((ftid & 1) == 0 ? h : H + h);
        pre_ab = ab_dtype_bf16 ? __bfloat162float(((const bf16*)x_ab)[at]) : x_ab[at];
      }
    }
  };
  auto stash_ab = [&](int buf) {
    if (ftid >= 0 && ftid < 2 * DELTA_CH) {
      float v = 0.f;
      if (ab_live) {
        if ((ftid & 1) == 0) {
          const float z = pre_ab + bias;
          const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));       // softplus
          v = expf(-decay_rate * sp);
        } else {
          v = 1.0f / (1.0f + expf(-pre_ab));
        }
      }
      sm[buf * buf_floats + (ftid >> 1) * per_tok + 2 * dimp + vpad + (ftid & 1)] = v;
    }
  };
  __syncthreads();
  fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += DELTA_CH, buf ^= 1) {
    stash_ab(buf);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                      // the chunk is in place, and the other buffer is read no more
    if (c0 + DELTA_CH < t1) fetch(c0 + DELTA_CH, buf ^ 1);
    const float* b = sm + buf * buf_floats;
    const int n = min(DELTA_CH, t1 - c0);
    if (warp >= nwork) continue;                          // a fetching warp
    // k . q of every token of the chunk, once per warp: RP lanes a token, 32 / RP tokens a pass
#pragma unroll
    for (int tt0 = 0; tt0 < DELTA_CH; tt0 += 32 / RP) {
      const float* tok = b + (tt0 + lane / RP) * per_tok;
      const float4* q4 = reinterpret_cast<const float4*>(tok) + (lane % RP);
      const float4* k4 = reinterpret_cast<const float4*>(tok + dimp) + (lane % RP);
      float kq = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 kk = k4[i * RP], qq = q4[i * RP];
        kq = fmaf(kk.x, qq.x, kq); kq = fmaf(kk.y, qq.y, kq); kq = fmaf(kk.z, qq.z, kq); kq = fmaf(kk.w, qq.w, kq);
      }
#pragma unroll
      for (int o = RP / 2; o > 0; o >>= 1) kq += __shfl_xor_sync(0xffffffffu, kq, o);
      if (lane % RP == 0) kqs[tt0 + lane / RP] = kq;
    }
    __syncwarp();
    for (int tt = 0; tt < n; ++tt) {
      const float* tok = b + tt * per_tok;
      const float4* q4 = reinterpret_cast<const float4*>(tok) + r;
      const float4* k4 = reinterpret_cast<const float4*>(tok + dimp) + r;
      const float vj = active ? tok[2 * dimp + jl] : 0.f;
      const float2 gb = *reinterpret_cast<const float2*>(tok + 2 * dimp + vpad);
      const float g = gb.x, beta = gb.y, kq = kqs[tt];
      float4 kr[RPT / 4];
      // packed sums over (even rows, odd rows), in up to four chains each so that a long column does not wait for itself
      constexpr int NCH = RPT >= 32 ? 4 : (RPT >= 16 ? 2 : 1);
      float2 p1[NCH], p2[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) { p1[c] = make_float2(0.f, 0.f); p2[c] = make_float2(0.f, 0.f); }
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 kk = k4[i * RP], qq = q4[i * RP];
        kr[i] = kk;
        p1[(2 * i) % NCH] = __ffma2_rn(st[2 * i], make_float2(kk.x, kk.y), p1[(2 * i) % NCH]);
        p2[(2 * i) % NCH] = __ffma2_rn(st[2 * i], make_float2(qq.x, qq.y), p2[(2 * i) % NCH]);
        p1[(2 * i + 1) % NCH] = __ffma2_rn(st[2 * i + 1], make_float2(kk.z, kk.w), p1[(2 * i + 1) % NCH]);
        p2[(2 * i + 1) % NCH] = __ffma2_rn(st[2 * i + 1], make_float2(qq.z, qq.w), p2[(2 * i + 1) % NCH]);
      }
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int c = 0; c < NCH; ++c) { s1 += p1[c].x + p1[c].y; s2 += p2[c].x + p2[c].y; }
#pragma unroll
      for (int o = RP / 2; o > 0; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
      }
      const float u = beta * (vj - g * s1);
      const float2 uu = make_float2(u, u), gg = make_float2(g, g);
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        st[2 * i] = __ffma2_rn(gg, st[2 * i], __fmul2_rn(make_float2(kr[i].x, kr[i].y), uu));
        st[2 * i + 1] = __ffma2_rn(gg, st[2 * i + 1], __fmul2_rn(make_float2(kr[i].z, kr[i].w), uu));
      }
      if (r == 0 && jl < vcols) obuf[tt * vpad + jl] = fmaf(g, s2, u * kq);
    }
    __syncwarp();
    {
      // the warp's columns of the chunk's read-outs go out together: 32 / RP neighbouring floats a token
      constexpr int CPW = 32 / RP;
      const int col0 = warp * CPW;
      for (int idx = lane; idx < n * CPW; idx += 32) {
        const int tt = idx / CPW, c = col0 + idx % CPW;
        if (c < vcols && cg * vcols + c < vdim)
          o_out[(size_t)(c0 + tt) * H * vdim + (size_t)h * vdim + cg * vcols + c] = obuf[tt * vpad + c];
      }
    }
    __syncwarp();                                         // kqs is rewritten for the next chunk
  }
  if (S != nullptr && active) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (row_of(i) < dim) S[(size_t)row_of(i) * vdim + j] = (i & 1) ? st[i >> 1].y : st[i >> 1].x;
  }
}

// out = o / sqrt(mean(o^2) + eps) * norm_w * silu(z): one warp per (token, head).
template <typename TZ, typename TO>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float* __restrict__ o, const TZ* z, long z_stride, const float* __restrict__ norm_w, float eps,
                 TO* __restrict__ out, long out_stride, int T, int H, int vdim) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * 4 + warp;
  if (item >= (long)T * H) return;
  const int t = (int)(item / H), h = (int)(item - (long)t * H);
  const float* row = o + ((size_t)t * H + h) * vdim;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) ss += row[i] * row[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    const float zz = to_f32(z[(size_t)t * z_stride + (size_t)h * vdim + i]);
    out[(size_t)t * out_stride + (size_t)h * vdim + i] = from_f32<TO>(row[i] * inv * norm_w[i] * (zz / (1.0f + expf(-zz))));
  }
}

// x [T][>= C] of x_dtype (row stride x_stride): the projected q, k, v side by side; taps_w float [C][taps];
// state float [num_slots][state_stride], a request's convolution rows at conv_offset; y float [T][C]: q, k (unit
// vectors, q scaled) and v after the convolution.  Then the state's rows are brought up to date.
PHOTON_API int photon_delta_conv(const void* x, long x_stride, int x_dtype, const float* taps_w, int taps, const int* token_seq,
                                 const int* cu_tokens, const int* state_slots, float* state, long state_stride,
                                 long conv_offset, int num_slots, float* y, int T, int S, int Gq, int H, int dim, int vdim,
                                 int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps < 1 || Gq <= 0 || H <= 0 || H % Gq || dim <= 0 || vdim <= 0) return PHOTON_ERR_ARGUMENT;
  if (T > 65535 || S > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int C = 2 * Gq * dim + H * vdim;
  dim3 grid((2 * Gq + H + 3) / 4, T);
  int st;
  if (x_dtype == PHOTON_F32)
    st = launch_pdl(delta_conv_kernel<float>, grid, dim3(128), 0, stream, (const float*)x, x_stride, taps_w, taps, token_seq, cu_tokens,
                    state_slots, (const float*)state, state_stride, conv_offset, num_slots, y, Gq, H, dim, vdim, err);
  else if (x_dtype == PHOTON_BF16)
    st = launch_pdl(delta_conv_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)x, x_stride, taps_w, taps, token_seq, cu_tokens,
                    state_slots, (const float*)state, state_stride, conv_offset, num_slots, y, Gq, H, dim, vdim, err);
  else
    return PHOTON_ERR_ARGUMENT;
  if (st != 0 || taps == 1) return st;
  dim3 g2((C + 127) / 128, S);
  if (x_dtype == PHOTON_F32)
    return launch_pdl(delta_conv_state_kernel<float>, g2, dim3(128), 0, stream, (const float*)x, x_stride, taps, cu_tokens, state_slots,
                      state, state_stride, conv_offset, num_slots, C);
  return launch_pdl(delta_conv_state_kernel<bf16>, g2, dim3(128), 0, stream, (const bf16*)x, x_stride, taps, cu_tokens, state_slots,
                    state, state_stride, conv_offset, num_slots, C);
}

template <int RPT, int RP>
static int delta_recurrent_launch(const float* y, const void* ab, long ab_stride, int ab_bf16, const float* a_log,
                                  const float* dt_bias, const int* cu_tokens, const int* state_slots, float* state,
                                  long state_stride, int num_slots, float* o, int S, int Gq, int H, int dim, int vdim, int* err,
                                  cudaStream_t stream) {
  // Columns a block owns: at most 256 / RP, and few enough that the step has about one block an SM: the warps of a
  // block go to different schedulers of the SM, while the first warps of two blocks on one SM would share one, and a
  // warp that walks tokens wants a scheduler to itself.  A multiple of 8 where the head has that many.  The cut
  // changes no column's arithmetic.
  const int most = 256 / RP;
  const long heads = (long)S * H;
  int groups = (int)((photon_sm_count() + heads - 1) / heads);
  if (groups < 1) groups = 1;
  int vcols = (vdim + groups - 1) / groups;
  vcols = ((vcols + 7) / 8) * 8;
  if (vcols < 32 / RP) vcols = 32 / RP;                   // a full warp of columns
  if (vcols > most) vcols = most;
  if (vcols > vdim) vcols = vdim;
  groups = (vdim + vcols - 1) / vcols;
  // the warps that own the columns, and two more that fetch
  const int threads = ((vcols * RP + 31) / 32) * 32 + 64;
  if (threads > 320 || groups > 65535) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)2 * DELTA_CH * delta_tok_floats(RPT * RP, vcols) + (size_t)(threads / 32) * DELTA_CH +
                       (size_t)DELTA_CH * ((vcols + 3) & ~3)) * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(delta_recurrent_kernel<RPT, RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(delta_recurrent_kernel<RPT, RP>, dim3(S, H, groups), dim3(threads), smem, stream, y, (const float*)ab, ab_stride,
                    ab_bf16, a_log, dt_bias, cu_tokens, state_slots, state, state_stride, num_slots, o, Gq, H, dim, vdim, vcols, err);
}

// y float [T][C] from photon_delta_conv; ab [T][>= 2 H] of ab_dtype (row stride ab_stride): the raw decay inputs of the
// H heads, then the raw beta inputs; a_log, dt_bias float [H]; state as above with S [H][dim][vdim] at its start;
// o float [T][H * vdim]: the read-outs before the norm.  dim up to 256.
PHOTON_API int photon_delta_recurrent(const float* y, const void* ab, long ab_stride, int ab_dtype, const float* a_log,
                                      const float* dt_bias, const int* cu_tokens, const int* state_slots, float* state,
                                      long state_stride, int num_slots, float* o, int S, int Gq, int H, int dim, int vdim,
                                      int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (Gq <= 0 || H <= 0 || H % Gq || dim <= 0 || vdim <= 0) return PHOTON_ERR_ARGUMENT;
  if (ab_dtype != PHOTON_F32 && ab_dtype != PHOTON_BF16) return PHOTON_ERR_ARGUMENT;
  if (S > 2147483647 / 2 || H > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int bf = ab_dtype == PHOTON_BF16;
  // lanes per column (RP) and rows per lane (RPT, a multiple of 4) follow from dim alone: few lanes a column, because
  // every level of shuffles lengthens the chain from one token to the next
#define DELTA_TRY(RPT, RP) if (dim <= RPT * RP) \
    return delta_recurrent_launch<RPT, RP>(y, ab, ab_stride, bf, a_log, dt_bias, cu_tokens, state_slots, state, state_stride, num_slots, \
                                           o, S, Gq, H, dim, vdim, err, stream)
  DELTA_TRY(4, 2); DELTA_TRY(4, 4); DELTA_TRY(8, 4); DELTA_TRY(16, 4); DELTA_TRY(32, 4); DELTA_TRY(64, 4);
  return PHOTON_ERR_UNSUPPORTED;
}

// o float [T][H * vdim]; z [T][H * vdim] of z_dtype (row stride z_stride); norm_w float [vdim]; out [T][H * vdim] of out_dtype.
PHOTON_API int photon_delta_out(const float* o, const void* z, long z_stride, int z_dtype, const float* norm_w, float eps,
                                void* out, long out_stride, int out_dtype, int T, int H, int vdim, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long items = (long)T * H;
  dim3 grid((unsigned)((items + 3) / 4));
#define DOUT_GO(TZ, TO) return launch_pdl(delta_out_kernel<TZ, TO>, grid, dim3(128), 0, stream, o, (const TZ*)z, z_stride, norm_w, eps, \
                                          (TO*)out, out_stride, T, H, vdim)
  if (z_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) DOUT_GO(float, float);
  if (z_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) DOUT_GO(float, bf16);
  if (z_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) DOUT_GO(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}
