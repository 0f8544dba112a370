// Paged causal attention whose heads talk to each other before the softmax, the general kernels: any head size up
// to 256, any number of heads and groups, any page size, float or bfloat16 storage, an optional window.
//
//   raw_g(i, j)  = (q_g(i) . k_{g / (H/G)}(j)) * qmul[g]              qmul[g] = scale * temperature[g]
//   s_h(i, j)    = sum_g talk[h][g] raw_g(i, j)                        all H heads, across the key/value groups
//   p_h(i, j)    = exp(s_h(i, j)) / (exp(sink[h]) + sum_j' exp(s_h(i, j')))      over the keys i sees
//   o_h(i)       = sigmoid(gate_h(i)) * sum_j p_h(i, j) v_{h / (H/G)}(j)
//
// A token at position i sees the keys max(0, i - window + 1) .. i.  talk, sink and gate may each be absent (null).
// Because every head's score needs every other head's, one block owns one token of the step with ALL its heads:
// it walks the keys in tiles of 32 from the cache, forms the raw scores of all heads for the tile, mixes them,
// and keeps a running softmax per head, all in 32-bit.  Prompt portions and single decoded tokens are the same
// case.  The tile grid starts at a multiple of 32 at or below the window's first key, so the order of every sum
// depends on the token's position alone.  The tiles of a token may be shared out over `splits` blocks, whose
// partial results a second kernel merges in split order.
//
// The cache planes are [pages, G, page_size, d]; the value plane may hold anything d numbers wide (this mixer's
// values are its keys before their rotation, which talk_prep writes there).
#include "common.cuh"
#include <math.h>

#define TALK_TILE 32
#define TALK_THREADS 256
#define TALK_MAX_D 256

// ---------------------------------------------------------------- bias, rotation and cache write
// One warp per (token, head) of the projected row.  q and k get their bias (32-bit), the first rot_dims numbers of a
// head are rotated by the token's position (number j with number j + rot_dims/2; angle, sine and cosine in 64-bit),
// and every result is rounded once.  The value plane gets the projected value row v, or, when v is null, the key's row
// BEFORE the rotation (a mixer whose values are its keys).
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
talk_prep_kernel(const TI* q, long q_stride, const TI* k, long k_stride, const TI* v, long v_stride, const float* __restrict__ q_bias,
                 const float* __restrict__ k_bias, TO* q_out, long qo_stride, const int* __restrict__ positions,
                 const double* __restrict__ inv_freq, int rot_dims, const int* __restrict__ slot_mapping,
                 TO* __restrict__ k_cache, TO* __restrict__ v_cache, int H, int G, int d, int page_size, long num_slots,
                 int* err) {
  extern __shared__ __align__(16) float prep_smem[];
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int item = blockIdx.x * 4 + warp;
  const int kv_items = k_cache ? G : 0;
  if (item >= H + kv_items) return;
  const bool is_q = item < H;
  const int h = is_q ? item : item - H;
  float* xs = prep_smem + (size_t)warp * d;
  const TI* row = (is_q ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * d;
  const float* bias = is_q ? q_bias : k_bias;
  for (int i = lane; i < d; i += 32) xs[i] = to_f32(row[i]) + (bias ? bias[(size_t)h * d + i] : 0.f);
  __syncwarp();
  TO* kdst = nullptr;
  if (!is_q) {
    long slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (lane == 0 && h == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
    if (slot < 0) return;                                  // a slot of -1 stores nothing
    const long page = slot / page_size;
    const size_t at = (((size_t)page * G + h) * page_size + (size_t)(slot - page * page_size)) * d;
    kdst = k_cache + at;
    if (v_cache != nullptr) {
      TO* vdst = v_cache + at;
      if (v != nullptr) {                                  // projected values of their own
        const TI* vrow = v + (size_t)t * v_stride + (size_t)h * d;
        for (int i = lane; i < d; i += 32) vdst[i] = from_f32<TO>(to_f32(vrow[i]));
      } else {                                             // the values are the keys before their rotation
        for (int i = lane; i < d; i += 32) vdst[i] = from_f32<TO>(xs[i]);
      }
    }
  }
  if (rot_dims > 0) {
    const int half = rot_dims >> 1;
    const double pos = (double)positions[t];
    for (int j = lane; j < half; j += 32) {
      double sn, cs;
      sincos(pos * inv_freq[j], &sn, &cs);
      const float c = (float)cs, s = (float)sn;
      const float a = xs[j], b = xs[j + half];
      xs[j] = a * c - b * s;
      xs[j + half] = b * c + a * s;
    }
    __syncwarp();
  }
  TO* dst = is_q ? q_out + (size_t)t * qo_stride + (size_t)h * d : kdst;
  for (int i = lane; i < d; i += 32) dst[i] = from_f32<TO>(xs[i]);
}

// q [T, H * d], k [T, G * d] of in_dtype (sections of one fused row; strides in elements); biases float [H * d],
// [G * d] or null; q_out [T, H * d] of out_dtype.  inv_freq: double [rot_dims / 2]; null or rot_dims 0: no rotation.
// k_cache, v_cache [pages, G, page_size, d] of out_dtype: the rotated key and (v_cache not null) the value: v [T, G * d]
// of in_dtype, or with v null the key before its rotation; k_cache null: nothing is stored and k, v are not read.
PHOTON_API int photon_talk_prep(const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
                                int in_dtype, const float* q_bias,
                                const float* k_bias, void* q_out, long qo_stride, int out_dtype, const int* positions,
                                const double* inv_freq, int rot_dims, const int* slot_mapping, void* k_cache, void* v_cache,
                                int T, int H, int G, int d, int page_size, long num_slots, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || H <= 0 || G <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > d) return PHOTON_ERR_ARGUMENT;
  if (k_cache == nullptr && v_cache != nullptr) return PHOTON_ERR_ARGUMENT;
  if (T > 65535 || d > 8192) return PHOTON_ERR_UNSUPPORTED;
  if (inv_freq == nullptr) rot_dims = 0;
  const int items = H + (k_cache ? G : 0);
  dim3 grid((items + 3) / 4, T);
  const size_t smem = (size_t)4 * d * sizeof(float);
#define PREP_GO(TI, TO) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(talk_prep_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    return launch_pdl(talk_prep_kernel<TI, TO>, grid, dim3(128), smem, stream, (const TI*)q, q_stride, (const TI*)k, k_stride, \
        (const TI*)v, v_stride, q_bias, k_bias, (TO*)q_out, qo_stride, positions, inv_freq, rot_dims, slot_mapping, (TO*)k_cache, (TO*)v_cache, H, G, d, \
        page_size, num_slots, err); } while (0)
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) PREP_GO(float, float);
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) PREP_GO(float, bf16);
  if (in_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) PREP_GO(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}

// ---------------------------------------------------------------- attention, one block per token (and split)
// part (splits > 1): float [T][splits][H * (d + 2)]: per head the running maximum, the sum and the d weighted sums.
template <typename T>
__global__ void __launch_bounds__(TALK_THREADS)
talk_attention_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_seq,
                      const int* __restrict__ positions, int H, int G, int d, int page_size, int num_pages, int window,
                      const float* __restrict__ qmul, const float* __restrict__ talk, const float* __restrict__ sink,
                      const float* gate, long gate_stride, int splits, float* __restrict__ part, int* err) {
  extern __shared__ __align__(16) float smem[];
  const int t = blockIdx.x, z = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hpg = H / G;
  float* qs = smem;                          // H * d, times qmul
  float* acc = qs + H * d;                   // H * d
  float* sraw = acc + H * d;                 // H * TILE
  float* pm = sraw + H * TALK_TILE;          // H * TILE
  float* tk = pm + H * TALK_TILE;            // H * H
  float* mrun = tk + H * H;                  // H
  float* lsum = mrun + H;                    // H
  float* corr = lsum + H;                    // H
  long long* rowbase = (long long*)(corr + H);     // TILE; H (H + 3) is even, so this is 8-byte aligned
  pdl_wait();
  const int p = positions[t];
  const int seq = token_seq[t];
  const int kstart = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)seq * max_pages;
  for (int i = tid; i < H * d; i += TALK_THREADS) {
    qs[i] = to_f32(q[(size_t)t * q_stride + i]) * qmul[i / d];
    acc[i] = 0.f;
  }
  if (talk) for (int i = tid; i < H * H; i += TALK_THREADS) tk[i] = talk[i];
  for (int h = tid; h < H; h += TALK_THREADS) { mrun[h] = -INFINITY; lsum[h] = 0.f; corr[h] = 0.f; }
  const int tile_lo = kstart / TALK_TILE, tile_hi = p / TALK_TILE + 1;
  int vt_lo = tile_lo, vt_hi = tile_hi;
  if (splits > 1) {
    const int per = (tile_hi - tile_lo + splits - 1) / splits;
    vt_lo = tile_lo + z * per;
    vt_hi = min(tile_hi, vt_lo + per);
  }
  const size_t head_step = (size_t)page_size * d;
  for (int vt = vt_lo; vt < vt_hi; ++vt) {
    const int tile0 = vt * TALK_TILE;
    __syncthreads();                         // the tile before is consumed; qs and tk are ready on the first pass
    if (tid < TALK_TILE) {
      const int kk = tile0 + tid;
      long long base = -1;
      if (kk <= p && kk >= kstart) {
        const int page = table[kk / page_size];
        if (page < 0 || page >= num_pages) report_error(err, PHOTON_DEV_BAD_PAGE, t, kk, page);
        else base = (((long long)page * G) * page_size + (kk % page_size)) * d;
      }
      rowbase[tid] = base;
    }
    __syncthreads();
    // raw scores: a warp takes a (key, key/value head) pair, holds the key row, and serves the group's query heads
    for (int pp = warp; pp < G * TALK_TILE; pp += TALK_THREADS / 32) {
      const int c = pp / TALK_TILE, jj = pp - c * TALK_TILE;
      const long long base = rowbase[jj];
      if (base < 0) {
        for (int g = lane; g < hpg; g += 32) sraw[(c * hpg + g) * TALK_TILE + jj] = 0.f;
        continue;
      }
      const T* krow = k_cache + base + (size_t)c * head_step;
      float kr[TALK_MAX_D / 32];
#pragma unroll
      for (int n = 0; n < TALK_MAX_D / 32; ++n) { const int dd = lane + 32 * n; kr[n] = dd < d ? to_f32(krow[dd]) : 0.f; }
      for (int g = c * hpg; g < (c + 1) * hpg; ++g) {
        float s = 0.f;
#pragma unroll
        for (int n = 0; n < TALK_MAX_D / 32; ++n) { const int dd = lane + 32 * n; if (dd < d) s = fmaf(qs[g * d + dd], kr[n], s); }
        s = warp_sum(s);
        if (lane == 0) sraw[g * TALK_TILE + jj] = s;
      }
    }
    __syncthreads();
    // the heads' scores are mixed; keys the token does not see leave the softmax
    for (int e = tid; e < H * TALK_TILE; e += TALK_THREADS) {
      const int h = e / TALK_TILE, jj = e - h * TALK_TILE;
      float s = -INFINITY;
      if (rowbase[jj] >= 0) {
        if (talk) {
          s = 0.f;
          for (int g = 0; g < H; ++g) s = fmaf(tk[h * H + g], sraw[g * TALK_TILE + jj], s);
        } else {
          s = sraw[e];
        }
      }
      pm[e] = s;
    }
    __syncthreads();
    for (int h = warp; h < H; h += TALK_THREADS / 32) {
      const float s = pm[h * TALK_TILE + lane];
      const float m_old = mrun[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float pr = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float sum = warp_sum(pr);
      pm[h * TALK_TILE + lane] = pr;
      if (lane == 0) {
        const float cr = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        corr[h] = cr;
        lsum[h] = lsum[h] * cr + sum;
        mrun[h] = m_new;
      }
    }
    __syncthreads();
    for (int idx = tid; idx < H * d; idx += TALK_THREADS) {
      const int h = idx / d, dd = idx - h * d;
      const size_t off = (size_t)(h / hpg) * head_step + dd;
      float a = acc[idx] * corr[h];
      for (int jj = 0; jj < TALK_TILE; ++jj) {
        const long long base = rowbase[jj];
        if (base >= 0) a = fmaf(pm[h * TALK_TILE + jj], to_f32(v_cache[base + off]), a);
      }
      acc[idx] = a;
    }
  }
  __syncthreads();
  pdl_launch_dependents();
  if (splits > 1) {
    float* dst = part + ((size_t)t * splits + z) * H * (d + 2);
    for (int h = tid; h < H; h += TALK_THREADS) { dst[h * (d + 2)] = mrun[h]; dst[h * (d + 2) + 1] = lsum[h]; }
    for (int idx = tid; idx < H * d; idx += TALK_THREADS) dst[(idx / d) * (d + 2) + 2 + idx % d] = acc[idx];
    return;
  }
  for (int idx = tid; idx < H * d; idx += TALK_THREADS) {
    const int h = idx / d;
    float m = mrun[h], l = lsum[h], a = acc[idx];
    if (sink) {
      const float M = fmaxf(m, sink[h]);
      const float c = (m == -INFINITY) ? 0.f : expf(m - M);
      l = l * c + expf(sink[h] - M);
      a *= c;
    }
    float o = l > 0.f ? a / l : 0.f;
    if (gate) o *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
    out[(size_t)t * out_stride + idx] = from_f32<T>(o);
  }
}

// Merges the partial results of a token's splits in split order, then the sink and the gate.
template <typename T>
__global__ void __launch_bounds__(TALK_THREADS)
talk_merge_kernel(const float* __restrict__ part, int splits, T* __restrict__ out, long out_stride, int H, int d,
                  const float* __restrict__ sink, const float* gate, long gate_stride) {
  pdl_wait();
  const int t = blockIdx.x;
  const float* src = part + (size_t)t * splits * H * (d + 2);
  for (int idx = threadIdx.x; idx < H * d; idx += TALK_THREADS) {
    const int h = idx / d, dd = idx - h * d;
    float M = sink ? sink[h] : -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, src[((size_t)z * H + h) * (d + 2)]);
    float l = sink ? expf(sink[h] - M) : 0.f, a = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float* ph = src + ((size_t)z * H + h) * (d + 2);
      const float c = (ph[0] == -INFINITY) ? 0.f : expf(ph[0] - M);
      l = fmaf(ph[1], c, l);
      a = fmaf(ph[2 + dd], c, a);
    }
    float o = l > 0.f ? a / l : 0.f;
    if (gate) o *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + h]));
    out[(size_t)t * out_stride + idx] = from_f32<T>(o);
  }
}

static size_t talk_smem_bytes(int H, int d) {
  size_t floats = (size_t)2 * H * d + (size_t)2 * H * TALK_TILE + (size_t)H * H + 3 * H;
  floats += floats & 1;
  return floats * sizeof(float) + TALK_TILE * sizeof(long long);
}

// q, out [T, H * d] of dtype (row strides in elements); k_cache, v_cache [num_pages, G, page_size, d] of dtype;
// block_table [S, max_pages]; token_seq, positions [T]; qmul float [H]; talk float [H, H], sink float [H], gate float
// (row stride gate_stride, H numbers a row): each may be null.  window 0: none.  splits > 1: part float
// [T * splits * H * (d + 2)].
PHOTON_API int photon_talk_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                     const void* v_cache, int dtype, const int* block_table, int max_pages,
                                     const int* token_seq, const int* positions, int T, int H, int G, int d, int page_size,
                                     int num_pages, int window, const float* qmul, const float* talk, const float* sink,
                                     const float* gate, long gate_stride, int splits, float* part, int* err,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || window < 0 || splits < 1 || qmul == nullptr) return PHOTON_ERR_ARGUMENT;
  if (splits > 1 && part == nullptr) return PHOTON_ERR_ARGUMENT;
  if (d > TALK_MAX_D || T > 2147483647 / 2 || splits > 65535) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = talk_smem_bytes(H, d);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
#define TALK_GO(TT) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(talk_attention_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    int st_ = launch_pdl(talk_attention_kernel<TT>, dim3(T, splits), dim3(TALK_THREADS), smem, stream, (const TT*)q, q_stride, (TT*)out, \
        out_stride, (const TT*)k_cache, (const TT*)v_cache, block_table, max_pages, token_seq, positions, H, G, d, page_size, \
        num_pages, window, qmul, talk, sink, gate, gate_stride, splits, part, err); \
    if (st_ != 0 || splits == 1) return st_; \
    return launch_pdl(talk_merge_kernel<TT>, dim3(T), dim3(TALK_THREADS), 0, stream, (const float*)part, splits, (TT*)out, out_stride, \
        H, d, sink, gate, gate_stride); } while (0)
  if (dtype == PHOTON_F32) TALK_GO(float);
  if (dtype == PHOTON_BF16) TALK_GO(bf16);
  return PHOTON_ERR_ARGUMENT;
}

// The shares of a token's splits, part float [T][splits][H][d + 2] (per head: the running maximum as a natural
// logarithm, the sum, the d weighted sums), merged in split order; then the sink, the gate and the division.
PHOTON_API int photon_talk_merge(const float* part, int splits, void* out, long out_stride, int dtype, int T, int H, int d,
                                 const float* sink, const float* gate, long gate_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (part == nullptr || splits < 1 || H <= 0 || d <= 0) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_F32)
    return launch_pdl(talk_merge_kernel<float>, dim3(T), dim3(TALK_THREADS), 0, stream, part, splits, (float*)out, out_stride, H, d,
                      sink, gate, gate_stride);
  if (dtype == PHOTON_BF16)
    return launch_pdl(talk_merge_kernel<bf16>, dim3(T), dim3(TALK_THREADS), 0, stream, part, splits, (bf16*)out, out_stride, H, d,
                      sink, gate, gate_stride);
  return PHOTON_ERR_ARGUMENT;
}
