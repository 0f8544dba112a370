// Routed experts: a router picks `top` of E small gated feed-forward layers for every token.
//
//   photon_moe_route     logits z = W_r h + b in 32-bit, the `top` largest (the lower index wins a tie), weights =
//                        softmax over the chosen logits only; counts the tokens of every expert;
//   photon_moe_align     sorts the (token, choice) pairs by expert, stably, without the host: offsets of every
//                        expert in the sorted order, the sorted list, every pair's place in it, and the list
//                        of row tiles (expert, first row, rows) that the grouped products walk;
//   photon_moe_gemm      grouped product over the sorted rows: each row tile multiplies with its expert's
//                        matrix; rows of A are gathered through the sorted list (first product) or lie in
//                        sorted order already (second product); optional gated activation in the epilogue;
//   photon_moe_combine   out[t] = sum_j weight[t, j] * y[place(t, j)] (+ the shared expert's output), the sum in
//                        32-bit in the order of j.
//
// Every output of a product is one chain of K fused multiply-adds in ascending k, accumulated in 32-bit, so a
// token's result depends neither on the other tokens of the step nor on its place in the sorted order.
#include "common.cuh"
#include <math.h>

#define MOE_BM 32          // rows of a tile of the grouped products

// ---------------------------------------------------------------- router
// A block owns `tok` consecutive tokens (at most its number of warps, at most 8): a warp takes every nwarp-th row of
// the router and forms that row's logit for all of the block's tokens at once, so the row is read once per block.
// Then warp i chooses for token i.  A logit's sum has the same order whatever `tok` is.  Measured on B200 with 2,048
// tokens, 16 experts, rows of 2,048 (the call with its memset): one token per block 57 us, two 47, four 41, eight 59
// (256 blocks, each walking its rows in sequence, are too few); 8 tokens: one per block 22 us, eight in one block 61.
#define MOE_ROUTE_TOK 8
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, long h_stride, const T* __restrict__ Wr,
                                 const void* __restrict__ bias, int bias_bf16, int H, int E, int top,
                                 int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ counts, int T_,
                                 int mode, int n_groups, int keep_groups, float route_scale,
                                 const T* __restrict__ Wsg, float* __restrict__ shared_gate, int tok) {
  extern __shared__ float logits[];                     // per token: E (+ 1: the shared expert's gate) + n_groups flags
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const int t0 = blockIdx.x * tok;
  const int ntok = min(tok, T_ - t0);
  const int LS = E + 1 + n_groups;
  constexpr int V = 16 / sizeof(T);                      // elements of a 16-byte load
  const bool vec = (H % V == 0) && ((uintptr_t)h % 16 == 0) && (h_stride % V == 0) && ((uintptr_t)Wr % 16 == 0) &&
                   ((uintptr_t)Wsg % 16 == 0);
  for (int e = warp; e < E + (Wsg ? 1 : 0); e += nwarp) {
    const T* w = e < E ? Wr + (size_t)e * H : Wsg;
    float acc[MOE_ROUTE_TOK];
#pragma unroll
    for (int i = 0; i < MOE_ROUTE_TOK; ++i) acc[i] = 0.f;
    if (vec) {
      for (int k = lane * V; k < H; k += 32 * V) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
        const T* wp = reinterpret_cast<const T*>(&wv);
#pragma unroll
        for (int i = 0; i < MOE_ROUTE_TOK; ++i) {
          if (i < ntok) {
            const uint4 xv = *reinterpret_cast<const uint4*>(h + (size_t)(t0 + i) * h_stride + k);
            const T* xp = reinterpret_cast<const T*>(&xv);
#pragma unroll
            for (int u = 0; u < V; ++u) acc[i] = fmaf(to_f32(xp[u]), to_f32(wp[u]), acc[i]);
          }
        }
      }
    } else {
      for (int k = lane; k < H; k += 32) {
        const float wk = to_f32(w[k]);
#pragma unroll
        for (int i = 0; i < MOE_ROUTE_TOK; ++i)
          if (i < ntok) acc[i] = fmaf(to_f32(h[(size_t)(t0 + i) * h_stride + k]), wk, acc[i]);
      }
    }
    const float add = (bias && e < E) ? load_w(bias, bias_bf16, e) : 0.f;
#pragma unroll
    for (int i = 0; i < MOE_ROUTE_TOK; ++i) {
      if (i < ntok) {
        const float v = warp_sum(acc[i]);
        if (lane == 0) logits[i * LS + e] = v + add;
      }
    }
  }
  __syncthreads();
  if (warp >= ntok) return;
  const int t = t0 + warp;                               // this warp's token
  float* lg = logits + warp * LS;
  const bool first = lane == 0;
  if (first && Wsg) shared_gate[t] = 1.0f / (1.0f + expf(-lg[E]));
  if (mode == 1 && E <= 32) {
    // The same rules as the serial form below with one lane per expert: maxima and sums by shuffles, a choice is the
    // lowest lane that holds the maximum (so ties go to the lower index).  top <= E <= 32.
    const unsigned full = 0xffffffffu;
    const bool live = lane < E;
    const float z = live ? lg[lane] : -INFINITY;
    const float mx = warp_max(z);
    const float p = live ? expf(z - mx) : 0.f;
    const float score = p / warp_sum(p);
    float cand = live ? score : -1.f;
    if (n_groups > 1 && keep_groups < n_groups) {
      const int per = E / n_groups;
      float gs = -1.f;                                   // lane g < n_groups: the best score of group g
      for (int g = 0; g < n_groups; ++g) {
        const float m = warp_max((live && lane / per == g) ? score : -1.f);
        if (lane == g) gs = m;
      }
      unsigned kept = 0u;                                // n_groups <= 32 here, because E <= 32
      for (int r = 0; r < keep_groups; ++r) {
        const float m = warp_max(gs);
        const int g = __ffs(__ballot_sync(full, gs == m && lane < n_groups)) - 1;
        kept |= 1u << g;
        if (lane == g) gs = -2.f;
      }
      if (live && !((kept >> (lane / per)) & 1u)) cand = -1.f;
    }
    float sum = 0.f, mine = 0.f;
    for (int j = 0; j < top; ++j) {
      const float m = warp_max(cand);
      const int best = __ffs(__ballot_sync(full, cand == m && live)) - 1;
      if (lane == j) mine = m;
      if (lane == best) cand = -2.f;
      sum += m;
      if (lane == 0) { ids[(size_t)t * top + j] = best; atomicAdd(&counts[best], 1); }
    }
    if (lane < top) weights[(size_t)t * top + lane] = mine / (sum + 1e-20f) * route_scale;
  } else if (first && (mode == 1 || mode == 2)) {
    // mode 1: scores are the softmax over ALL experts; a group's score is its largest score; the weights are the chosen
    // scores over their sum, times route_scale.  mode 2: scores are sigmoid(logit), each expert by itself; a group's
    // score is the sum of its two largest scores; the weights are the chosen scores as they are, times route_scale.
    // Groups of E / n_groups neighbours; only experts of the keep_groups best groups can be chosen.  Ties go to the
    // lower index everywhere.
    if (mode == 1) {
      float mx = -INFINITY;
      for (int e = 0; e < E; ++e) mx = fmaxf(mx, lg[e]);
      float den = 0.f;
      for (int e = 0; e < E; ++e) { const float p = expf(lg[e] - mx); lg[e] = p; den += p; }
      for (int e = 0; e < E; ++e) lg[e] /= den;
    } else {
      for (int e = 0; e < E; ++e) lg[e] = 1.0f / (1.0f + expf(-lg[e]));
    }
    if (n_groups > 1 && keep_groups < n_groups) {
      const int per = E / n_groups;
      float* kept = lg + E + 1;                          // n_groups flags behind the logits
      for (int g = 0; g < n_groups; ++g) kept[g] = 0.f;
      for (int r = 0; r < keep_groups; ++r) {
        int bg = -1;
        float bs = -1.f;
        for (int g = 0; g < n_groups; ++g) {
          if (kept[g] != 0.f) continue;
          float gs = -1.f, second = -1.f;
          for (int i = 0; i < per; ++i) {
            const float v = lg[g * per + i];
            if (v > gs) { second = gs; gs = v; } else if (v > second) second = v;
          }
          if (mode == 2 && per > 1) gs += second;
          if (gs > bs) { bs = gs; bg = g; }
        }
        kept[bg] = 1.f;
      }
      // a score of an expert outside the kept groups is hidden behind a negative number; it is not used again
      for (int g = 0; g < n_groups; ++g)
        if (kept[g] == 0.f)
          for (int i = 0; i < per; ++i) lg[g * per + i] = -1.f;
    }
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float v = lg[e];
        if (v > bv) { bv = v; best = e; }
      }
      ids[(size_t)t * top + j] = best;
      weights[(size_t)t * top + j] = bv;
      sum += bv;
      lg[best] = -2.f;
      atomicAdd(&counts[best], 1);
    }
    for (int j = 0; j < top; ++j) {
      const float wj = weights[(size_t)t * top + j];
      weights[(size_t)t * top + j] = mode == 1 ? wj / (sum + 1e-20f) * route_scale : wj * route_scale;
    }
  }
  if (first && mode == 0) {
    float chosen_max = -INFINITY;
    for (int j = 0; j < top; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float v = lg[e];
        if (best < 0 || v > bv) { bv = v; best = e; }
      }
      ids[(size_t)t * top + j] = best;
      weights[(size_t)t * top + j] = bv;
      if (j == 0) chosen_max = bv;
      lg[best] = -INFINITY;
      atomicAdd(&counts[best], 1);
    }
    float sum = 0.f;
    for (int j = 0; j < top; ++j) {
      const float p = expf(weights[(size_t)t * top + j] - chosen_max);
      weights[(size_t)t * top + j] = p;
      sum += p;
    }
    for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] /= sum;
  }
}

// h [T][H] (row stride in elements), Wr [E][H] of the same type, bias [E] (may be null).  ids, weights [T][top];
// counts [E] is cleared first and then holds the number of (token, choice) pairs of every expert.
PHOTON_API int photon_moe_route(const void* h, long h_stride, int dtype, const void* Wr, const void* bias, int bias_dtype,
                                int T_, int H, int E, int top, int* ids, float* weights, int* counts,
                                cudaStream_t stream) {
  return photon_moe_route_ex(h, h_stride, dtype, Wr, bias, bias_dtype, T_, H, E, top, ids, weights, counts, 0, 1, 1, 1.0f,
                             nullptr, nullptr, stream);
}

// mode 0: as above.  mode 1: scores are the softmax over all experts; with n_groups > 1 the experts form that many
// equal groups of neighbours and only experts of the keep_groups groups with the largest best score can be chosen; the
// weights are the chosen scores divided by their sum (+ 1e-20) times route_scale.  mode 2: scores are sigmoid(logit); a
// group's score is the sum of its two largest scores; the weights are the chosen scores times route_scale, not divided
// by their sum.  Wsg (may be null): one more row
// [H] of the router's type; shared_gate [T] then gets sigmoid(Wsg . h), the gate of a shared expert.
PHOTON_API int photon_moe_route_ex(const void* h, long h_stride, int dtype, const void* Wr, const void* bias, int bias_dtype,
                                   int T_, int H, int E, int top, int* ids, float* weights, int* counts, int mode,
                                   int n_groups, int keep_groups, float route_scale, const void* Wsg, float* shared_gate,
                                   cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || H <= 0) return PHOTON_ERR_ARGUMENT;
  if (mode < 0 || mode > 2) return PHOTON_ERR_ARGUMENT;
  if (n_groups < 1 || keep_groups < 1 || keep_groups > n_groups || E % n_groups) return PHOTON_ERR_ARGUMENT;
  if (mode != 0 && n_groups > 1 && (long)keep_groups * (E / n_groups) < top) return PHOTON_ERR_ARGUMENT;
  if ((Wsg == nullptr) != (shared_gate == nullptr)) return PHOTON_ERR_ARGUMENT;
  const int warps = E >= 8 ? 8 : (E >= 4 ? 4 : 2);
  // few tokens (a decode step): one per block, so that every token's logits form on an SM of their own
  const int tok = T_ >= 64 ? (warps < 4 ? warps : 4) : 1;
  const size_t smem = (size_t)tok * (E + 1 + n_groups) * sizeof(float);
  if (smem > 48 * 1024) return PHOTON_ERR_UNSUPPORTED;
  cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  const int blocks = (T_ + tok - 1) / tok;
  if (dtype == PHOTON_BF16)
    moe_route_kernel<bf16><<<blocks, warps * 32, smem, stream>>>((const bf16*)h, h_stride, (const bf16*)Wr, bias,
                                                                bias_dtype == PHOTON_BF16, H, E, top, ids, weights, counts, T_,
                                                                mode, n_groups, keep_groups, route_scale, (const bf16*)Wsg, shared_gate, tok);
  else
    moe_route_kernel<float><<<blocks, warps * 32, smem, stream>>>((const float*)h, h_stride, (const float*)Wr, bias,
                                                                 bias_dtype == PHOTON_BF16, H, E, top, ids, weights, counts, T_,
                                                                 mode, n_groups, keep_groups, route_scale, (const float*)Wsg, shared_gate, tok);
  return launch_status();
}

// ---------------------------------------------------------------- sort by expert
// One block per expert e: its first row in the sorted order is the number of pairs of the experts before it, and
// its pairs take the following places in the order in which they stand in `ids`.
__global__ void moe_align_kernel(const int* __restrict__ ids, const int* __restrict__ counts, int n, int E,
                                 int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ place,
                                 int* __restrict__ tiles, int* __restrict__ num_tiles) {
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (threadIdx.x == 0) {
    int off = 0, tl = 0;
    for (int i = 0; i < e; ++i) { off += counts[i]; tl += (counts[i] + MOE_BM - 1) / MOE_BM; }
    base_s = off;
    offsets[e] = off;
    const int own = counts[e];
    for (int i = 0; i * MOE_BM < own; ++i) {
      tiles[3 * (tl + i)] = e;
      tiles[3 * (tl + i) + 1] = off + i * MOE_BM;
      tiles[3 * (tl + i) + 2] = min(MOE_BM, own - i * MOE_BM);
    }
    if (e == E - 1) { offsets[E] = off + own; *num_tiles = tl + (own + MOE_BM - 1) / MOE_BM; }
  }
  __syncthreads();
  int running = base_s;
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool mine = i < n && ids[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    const int before = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(ballot);
    __syncthreads();
    int wbase = 0, total = 0;
    for (int w = 0; w < nwarp; ++w) { if (w < warp) wbase += warp_tot[w]; total += warp_tot[w]; }
    if (mine) { const int p = running + wbase + before; sorted[p] = i; place[i] = p; }
    running += total;
    __syncthreads();
  }
}

// ids [n] (n = T * top), counts [E] -> offsets [E + 1], sorted [n] (pair index at each sorted row), place [n]
// (sorted row of each pair), tiles [3 * max_tiles] (expert, first row, rows), num_tiles [1].
// max_tiles >= n / MOE_BM + E always suffices.
PHOTON_API int photon_moe_align(const int* ids, const int* counts, int n, int E, int* offsets, int* sorted, int* place,
                                int* tiles, int* num_tiles, cudaStream_t stream) {
  if (n <= 0 || E <= 0) return 0;
  moe_align_kernel<<<E, 256, 0, stream>>>(ids, counts, n, E, offsets, sorted, place, tiles, num_tiles);
  return launch_status();
}

PHOTON_API int photon_moe_tile_rows(void) { return MOE_BM; }

// ---------------------------------------------------------------- grouped product
#define MOE_BN 64
#define MOE_BK 16

__device__ __forceinline__ float moe_act(float g, int act) {
  if (act == PHOTON_ACT_NONE) return g;
  if (act == PHOTON_ACT_GELU) return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));
  if (act == PHOTON_ACT_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.0f + expf(-g));
}

// GLU: W holds [gate rows; up rows] per expert (N = 2 * cols); the block computes the gate and the up column of
// each of its output columns and stores act(gate) * up.
template <typename T, typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const T* __restrict__ A, long lda, const int* __restrict__ gather, int gather_div,
                const T* __restrict__ W, TO* __restrict__ out, long ldo, int N, int K,
                const int* __restrict__ tiles, const int* __restrict__ num_tiles, int act) {
  __shared__ float As[MOE_BK][MOE_BM + 4];
  __shared__ float Ws[GLU ? 2 : 1][MOE_BK][MOE_BN + 4];
  __shared__ int arow[MOE_BM];
  const int tile = blockIdx.y;
  if (tile >= *num_tiles) return;
  const int e = tiles[3 * tile], r0 = tiles[3 * tile + 1], rows = tiles[3 * tile + 2];
  const int cols = GLU ? N / 2 : N;
  const int n0 = blockIdx.x * MOE_BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;       // 16 x 16 threads: 2 rows x 4 columns each
  const T* We = W + (size_t)e * N * K;
  if (tid < MOE_BM) arow[tid] = tid < rows ? (gather ? gather[r0 + tid] / gather_div : r0 + tid) : -1;
  __syncthreads();
  float acc[GLU ? 2 : 1][2][4];
#pragma unroll
  for (int p = 0; p < (GLU ? 2 : 1); ++p)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[p][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int idx = tid + r * 256;                     // 32 rows x 16 k
      const int row = idx >> 4, kk = idx & 15;
      const int ar = arow[row], gk = k0 + kk;
      As[kk][row] = (ar >= 0 && gk < K) ? to_f32(A[(size_t)ar * lda + gk]) : 0.f;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = tid + r * 256;                     // 64 columns x 16 k
      const int col = idx >> 4, kk = idx & 15;
      const int gn = n0 + col, gk = k0 + kk;
      const bool ok = gn < cols && gk < K;
      Ws[0][kk][col] = ok ? to_f32(We[(size_t)gn * K + gk]) : 0.f;
      if (GLU) Ws[GLU ? 1 : 0][kk][col] = ok ? to_f32(We[(size_t)(gn + cols) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_BK; ++kk) {
      float a[2], b[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = As[kk][ty * 2 + i];
#pragma unroll
      for (int p = 0; p < (GLU ? 2 : 1); ++p) {
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[p][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[p][i][j] = fmaf(a[i], b[j], acc[p][i][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = ty * 2 + i;
    if (row >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= cols) continue;
      float v = acc[0][i][j];
      v = GLU ? moe_act(v, act) * acc[GLU ? 1 : 0][i][j] : moe_act(v, act);
      out[(size_t)(r0 + row) * ldo + gn] = from_f32<TO>(v);
    }
  }
}

// A [*][K] (row stride lda).  gather (may be null): row r of the sorted order reads A row gather[r] / gather_div;
// null: row r itself.  W [E][N][K] contiguous.  out [n][N] (or [n][N / 2] with glu != 0), rows in sorted order.
// act: PHOTON_ACT_*; with glu != 0 it is applied to the gate, otherwise to every output (PHOTON_ACT_NONE: plain product).
// out_dtype: PHOTON_F32 or the input type.  max_tiles: bound of the tile list (the grid's height).
PHOTON_API int photon_moe_gemm(const void* A, long lda, int dtype, const int* gather, int gather_div, const void* W,
                               void* out, long ldo, int out_dtype, int N, int K, const int* tiles, const int* num_tiles,
                               int max_tiles, int glu, int act, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  if (K <= 0 || gather_div <= 0 || (glu && (N & 1))) return PHOTON_ERR_ARGUMENT;
  if (max_tiles > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int cols = glu ? N / 2 : N;
  dim3 grid((cols + MOE_BN - 1) / MOE_BN, max_tiles);
#define MOE_GEMM(T, TO, GLU) moe_gemm_kernel<T, TO, GLU><<<grid, 256, 0, stream>>>((const T*)A, lda, gather, gather_div, \
      (const T*)W, (TO*)out, ldo, N, K, tiles, num_tiles, act)
  if (dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) { if (glu) MOE_GEMM(bf16, bf16, true); else MOE_GEMM(bf16, bf16, false); }
  else if (dtype == PHOTON_BF16 && out_dtype == PHOTON_F32) { if (glu) MOE_GEMM(bf16, float, true); else MOE_GEMM(bf16, float, false); }
  else if (dtype == PHOTON_F32 && out_dtype == PHOTON_F32) { if (glu) MOE_GEMM(float, float, true); else MOE_GEMM(float, float, false); }
  else return PHOTON_ERR_ARGUMENT;
  return launch_status();
}

// ---------------------------------------------------------------- weighted sum of the chosen experts
template <typename TY, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, long ldy, const int* __restrict__ place,
                                   const float* __restrict__ weights, int top, const TO* __restrict__ shared_out,
                                   TO* __restrict__ out, int H, const float* __restrict__ shared_gate) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc = fmaf(weights[(size_t)t * top + j],
                 to_f32(y[(size_t)(place ? place[(size_t)t * top + j] : t * top + j) * ldy + i]), acc);
    if (shared_out) acc += shared_gate ? shared_gate[t] * to_f32(shared_out[(size_t)t * H + i]) : to_f32(shared_out[(size_t)t * H + i]);
    out[(size_t)t * H + i] = from_f32<TO>(acc);
  }
}

// y [n][H] (float or bfloat16): row place[t, j] is the output of token t's j-th expert (place null: row t * top + j);
// weights [T][top]; shared_out [T][H] (may be null) and out [T][H] of out_dtype.
PHOTON_API int photon_moe_combine(const void* y, long ldy, int y_dtype, const int* place, const float* weights, int top,
                                  const void* shared_out, void* out, int out_dtype, int T_, int H, cudaStream_t stream) {
  return photon_moe_combine_ex(y, ldy, y_dtype, place, weights, top, shared_out, nullptr, out, out_dtype, T_, H, stream);
}

// The same; shared_gate [T] (may be null): the shared expert's output of token t is multiplied by shared_gate[t].
PHOTON_API int photon_moe_combine_ex(const void* y, long ldy, int y_dtype, const int* place, const float* weights, int top,
                                     const void* shared_out, const float* shared_gate, void* out, int out_dtype, int T_,
                                     int H, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (out_dtype == PHOTON_BF16 && y_dtype == PHOTON_F32)
    moe_combine_kernel<float, bf16><<<T_, threads, 0, stream>>>((const float*)y, ldy, place, weights, top, (const bf16*)shared_out, (bf16*)out, H, shared_gate);
  else if (out_dtype == PHOTON_BF16 && y_dtype == PHOTON_BF16)
    moe_combine_kernel<bf16, bf16><<<T_, threads, 0, stream>>>((const bf16*)y, ldy, place, weights, top, (const bf16*)shared_out, (bf16*)out, H, shared_gate);
  else if (out_dtype == PHOTON_F32 && y_dtype == PHOTON_F32)
    moe_combine_kernel<float, float><<<T_, threads, 0, stream>>>((const float*)y, ldy, place, weights, top, (const float*)shared_out, (float*)out, H, shared_gate);
  else
    return PHOTON_ERR_ARGUMENT;
  return launch_status();
}

// ---------------------------------------------------------------- rows in sorted order
// out[r, :] = x[sorted[r] / div, :]: the input rows of the (token, choice) pairs, expert by expert, as the
// library's grouped product wants them.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, long ldx, const int* __restrict__ sorted, int div,
                                  T* __restrict__ out, int H) {
  const T* src = x + (size_t)(sorted[blockIdx.x] / div) * ldx;
  T* dst = out + (size_t)blockIdx.x * H;
  if (H % (16 / sizeof(T)) == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0) {
    const int n = H / (16 / sizeof(T));
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

PHOTON_API int photon_moe_gather(const void* x, long ldx, int dtype, const int* sorted, int div, void* out, int n, int H,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  if (div <= 0) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16) moe_gather_kernel<bf16><<<n, 128, 0, stream>>>((const bf16*)x, ldx, sorted, div, (bf16*)out, H);
  else moe_gather_kernel<float><<<n, 128, 0, stream>>>((const float*)x, ldx, sorted, div, (float*)out, H);
  return launch_status();
}

// ---------------------------------------------------------------- few rows: one matrix-vector product per pair
// A decode step brings a handful of (token, choice) pairs, each to another expert as a rule: nothing is sorted,
// block (c, p) streams the rows c * 32 .. of pair p's expert matrix once, 16 bytes per lane and load, against the
// pair's input row in shared memory; a warp owns four output features at a time and adds its lanes' sums up.
#define GEMV_COLS 32

template <typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemv_kernel(const bf16* __restrict__ x, long ldx, int x_div, const int* __restrict__ ids, const bf16* __restrict__ W,
                TO* __restrict__ out, long ldo, int N, int K, int act) {
  extern __shared__ __align__(16) bf16 xs[];
  const int p = blockIdx.y;
  const int e = ids[p];
  const int cols = GLU ? N / 2 : N;
  const bf16* xr = x + (size_t)(p / x_div) * ldx;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(xr + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* We = W + (size_t)e * N * K;
#pragma unroll
  for (int c = 0; c < GEMV_COLS / 8; ++c) {
    const int col = blockIdx.x * GEMV_COLS + c * 8 + warp;
    if (col >= cols) continue;                           // the whole warp
    float a0 = 0.f, a1 = 0.f;
    const bf16* w0 = We + (size_t)col * K;
    const bf16* w1 = We + (size_t)(col + cols) * K;
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + k);
      const uint4 wv = *reinterpret_cast<const uint4*>(w0 + k);
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 xf = __bfloat1622float2(xp[i]), wf = __bfloat1622float2(wp[i]);
        a0 = fmaf(xf.x, wf.x, a0); a0 = fmaf(xf.y, wf.y, a0);
      }
      if (GLU) {
        const uint4 uv = *reinterpret_cast<const uint4*>(w1 + k);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __bfloat1622float2(xp[i]), uf = __bfloat1622float2(up[i]);
          a1 = fmaf(xf.x, uf.x, a1); a1 = fmaf(xf.y, uf.y, a1);
        }
      }
    }
    a0 = warp_sum(a0);
    if (GLU) a1 = warp_sum(a1);
    if (lane == 0) out[(size_t)p * ldo + col] = from_f32<TO>(GLU ? moe_act(a0, act) * a1 : moe_act(a0, act));
  }
}

// x [*][K] bfloat16: pair p reads row p / x_div.  ids [n]: the expert of every pair.  W [E][N][K] bfloat16.
// out [n][N] float or bfloat16 (glu: [n][N / 2]), rows in the order of the pairs.  K % 8 == 0, 16-byte aligned rows.
PHOTON_API int photon_moe_gemv(const void* x, long ldx, int x_div, const int* ids, int n, const void* W, void* out, long ldo,
                               int out_dtype, int N, int K, int glu, int act, cudaStream_t stream) {
  if (n <= 0 || N <= 0) return 0;
  if (K <= 0 || x_div <= 0 || (glu && (N & 1))) return PHOTON_ERR_ARGUMENT;
  if (K % 8 || ldx % 8 || (uintptr_t)x % 16 || (uintptr_t)W % 16 || n > 65535 || (size_t)K * 2 > 96 * 1024) return PHOTON_ERR_UNSUPPORTED;
  const int cols = glu ? N / 2 : N;
  dim3 grid((cols + GEMV_COLS - 1) / GEMV_COLS, n);
  const size_t smem = (size_t)K * sizeof(bf16);
#define MOE_GEMV(TO, GLU) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(moe_gemv_kernel<TO, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    moe_gemv_kernel<TO, GLU><<<grid, 256, smem, stream>>>((const bf16*)x, ldx, x_div, ids, (const bf16*)W, (TO*)out, ldo, N, K, act); } while (0)
  if (out_dtype == PHOTON_BF16) { if (glu) MOE_GEMV(bf16, true); else MOE_GEMV(bf16, false); }
  else if (out_dtype == PHOTON_F32) { if (glu) MOE_GEMV(float, true); else MOE_GEMV(float, false); }
  else return PHOTON_ERR_ARGUMENT;
  return launch_status();
}
