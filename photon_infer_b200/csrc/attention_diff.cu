// Differential attention over the paged cache: every query head has TWO score maps over the same values, and its
// output is the difference of the two maps' outputs.
//
//   q [H][2][d], k [G][2][d] per token (head by head, map 1 then map 2), v [G][dv]; query head h uses key/value
//   head h / (H / G).  Per head and map: y = x / sqrt(mean(x^2) + eps) * w (w [d] shared by all heads and maps), then
//   the first rot_dims numbers are rotated by the position (number j with j + rot_dims / 2, angle p * inv_freq[j]).
//   s_m = (q_m . k_m) * scale over the keys max(0, p - window + 1) .. p, softmax per map, a_m = sum_j p_m[j] v[j];
//   o = a_1 - lambda a_2;  o <- o / sqrt(mean(o^2) + eps) * out_scale      (per head over its dv numbers).
//
//   photon_diff_prep        biases, norm, rotation; queries out in the run type; keys and values into the cache.
//                           The key cache holds both maps of a head side by side: [pages][G][page_size][2 d]; the
//                           value cache [pages][G][page_size][dv].  Null caches: queries only (a layer that reads
//                           another layer's keys and values).  A slot of -1 stores nothing.
//   photon_diff_attention   the general kernel: one block per token and key/value head (its query heads in chunks),
//                           tiles of 32 keys from a multiple of 32 at or below the window's first key, running softmax
//                           in 32-bit per (head, map).  The order of every sum depends on the token's position
//                           alone, never on how the request was cut into steps or on the rest of the batch.
//
// Norm, rotation, scores, softmax, the difference and the head norm are 32-bit; the angle and its sine and cosine
// 64-bit; every result is rounded once, to the run type.
#include "common.cuh"
#include <math.h>

#define DP_WARPS 4

template <typename TI, typename TO>
__global__ void __launch_bounds__(DP_WARPS * 32)
diff_prep_kernel(const TI* q, long q_stride, const TI* k, long k_stride, const TI* v, long v_stride, TO* q_out, long qo_stride,
                 const void* __restrict__ q_b, const void* __restrict__ k_b, const void* __restrict__ v_b, int b_bf16,
                 const void* __restrict__ q_w, const void* __restrict__ k_w, int w_bf16, float eps,
                 const int* __restrict__ positions, const double* __restrict__ inv_freq, int rot_dims,
                 const int* __restrict__ slot_mapping, TO* __restrict__ k_cache, TO* __restrict__ v_cache, int H, int G,
                 int d, int dv, int page_size, long num_slots, int* err) {
  extern __shared__ __align__(16) float dp_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int item = blockIdx.x * DP_WARPS + warp;
  const int k_items = k_cache ? 2 * G : 0, v_items = k_cache ? G : 0;
  if (item >= 2 * H + k_items + v_items) return;
  const int which = item < 2 * H ? 0 : (item < 2 * H + k_items ? 1 : 2);
  const int idx = which == 0 ? item : (which == 1 ? item - 2 * H : item - 2 * H - k_items);   // (head, map) or value head
  float* xs = dp_smem + (size_t)warp * d;

  long slot = -1;
  size_t row_at = 0;                                   // (page, head, slot in page) as one row index
  if (which != 0) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (lane == 0 && which == 1 && idx == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
    if (slot < 0) return;
    const long page = slot / page_size;
    const int g = which == 1 ? idx >> 1 : idx;
    row_at = ((size_t)page * G + g) * page_size + (size_t)(slot - page * page_size);
  }
  if (which == 2) {
    const TI* vr = v + (size_t)t * v_stride + (size_t)idx * dv;
    TO* dst = v_cache + row_at * dv;
    for (int i = lane; i < dv; i += 32)
      dst[i] = from_f32<TO>(to_f32(vr[i]) + (v_b ? load_w(v_b, b_bf16, (size_t)idx * dv + i) : 0.f));
    return;
  }
  const TI* row = (which == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)idx * d;
  const void* bias = which == 0 ? q_b : k_b;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float x = to_f32(row[i]) + (bias ? load_w(bias, b_bf16, (size_t)idx * d + i) : 0.f);
    xs[i] = x;
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  const void* w = which == 0 ? q_w : k_w;
  __syncwarp();
  for (int i = lane; i < d; i += 32) xs[i] = w ? xs[i] * inv * load_w(w, w_bf16, i) : xs[i] * inv;
  __syncwarp();
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
  TO* dst = which == 0 ? q_out + (size_t)t * qo_stride + (size_t)idx * d
                       : k_cache + row_at * (2 * (size_t)d) + (size_t)(idx & 1) * d;
  for (int i = lane; i < d; i += 32) dst[i] = from_f32<TO>(xs[i]);
}

// q [T][2 H d], k [T][2 G d], v [T][G dv] of in_dtype, each with its own row stride in elements (sections of one fused
// row as a rule).  Biases of b_dtype (each may be null), norm weights [d] of w_dtype (may be null: no weight).
// q_out [T][2 H d] of out_dtype.  inv_freq: double [rot_dims / 2]; null or rot_dims 0: no rotation.
PHOTON_API int photon_diff_prep(const void* q, long q_stride, const void* k, long k_stride, const void* v, long v_stride,
                                int in_dtype, void* q_out, long qo_stride, int out_dtype, const void* q_b, const void* k_b,
                                const void* v_b, int b_dtype, const void* q_w, const void* k_w, int w_dtype, float eps,
                                const int* positions, const double* inv_freq, int rot_dims, const int* slot_mapping,
                                void* k_cache, void* v_cache, int T, int H, int G, int d, int dv, int page_size,
                                long num_slots, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || dv <= 0 || H <= 0 || G <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > d) return PHOTON_ERR_ARGUMENT;
  if ((k_cache == nullptr) != (v_cache == nullptr)) return PHOTON_ERR_ARGUMENT;
  if (k_cache != nullptr && (k == nullptr || v == nullptr || slot_mapping == nullptr)) return PHOTON_ERR_ARGUMENT;
  if (T > 65535 || d > 8192) return PHOTON_ERR_UNSUPPORTED;
  if (inv_freq == nullptr) rot_dims = 0;
  const int items = 2 * H + (k_cache ? 3 * G : 0);
  dim3 grid((items + DP_WARPS - 1) / DP_WARPS, T);
  const size_t smem = (size_t)DP_WARPS * d * sizeof(float);
#define DP_GO(TI, TO) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(diff_prep_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    diff_prep_kernel<TI, TO><<<grid, DP_WARPS * 32, smem, stream>>>((const TI*)q, q_stride, (const TI*)k, k_stride, (const TI*)v, v_stride, \
        (TO*)q_out, qo_stride, q_b, k_b, v_b, b_dtype == PHOTON_BF16, q_w, k_w, w_dtype == PHOTON_BF16, eps, positions, inv_freq, \
        rot_dims, slot_mapping, (TO*)k_cache, (TO*)v_cache, H, G, d, dv, page_size, num_slots, err); \
    return launch_status(); } while (0)
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) DP_GO(float, float);
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) DP_GO(float, bf16);
  if (in_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) DP_GO(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}

// ---------------------------------------------------------------- attention, the general kernel
#define DA_TILE 32
#define DA_THREADS 128

template <typename T, int PPT>
__global__ void __launch_bounds__(DA_THREADS)
diff_attention_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ block_table,
                      int max_pages, const int* __restrict__ token_seq, const int* __restrict__ positions, int n_q, int n_kv,
                      int d, int dv, int hb, int page_size, int num_pages, int window, float scale, float lambda,
                      float out_scale, float eps, int* err) {
  extern __shared__ __align__(16) float smem[];
  const int per_kv = n_q / n_kv;
  const int chunks = (per_kv + hb - 1) / hb;
  const int t = blockIdx.x, g = blockIdx.y / chunks;
  const int h0 = g * per_kv + (blockIdx.y % chunks) * hb;                  // first query head of this block
  const int NH = min(hb, (g + 1) * per_kv - h0);                           // query heads of this block
  const int R = 2 * NH;                                                    // (head, map) rows
  const int d2 = 2 * d, kld = d2 + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* qs = smem;                          // 2 hb d
  float* ks = qs + 2 * hb * d;               // TILE * (2 d + 1)
  float* vs = ks + DA_TILE * kld;            // TILE * dv
  float* sc = vs + DA_TILE * dv;             // 2 hb * TILE
  float* fin = sc + 2 * hb * DA_TILE;        // 2 hb * dv
  float* mrun = fin + 2 * hb * dv;           // 2 hb
  float* lsum = mrun + 2 * hb;               // 2 hb
  float* corr = lsum + 2 * hb;               // 2 hb
  long long* kbase = (long long*)(corr + 2 * hb);   // TILE (the float count before it is even)

  const int p = positions[t];
  const int seq = token_seq[t];
  const int kstart = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)seq * max_pages;

  {
    const T* qrow = q + (size_t)t * q_stride + (size_t)h0 * d2;
    for (int i = tid; i < R * d; i += DA_THREADS) qs[i] = to_f32(qrow[i]);
  }
  for (int r = tid; r < R; r += DA_THREADS) { mrun[r] = -INFINITY; lsum[r] = 0.f; corr[r] = 0.f; }
  float acc[PPT];
#pragma unroll
  for (int n = 0; n < PPT; ++n) acc[n] = 0.f;

  const int tile_lo = kstart / DA_TILE, tile_hi = p / DA_TILE + 1;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int tile0 = tile * DA_TILE;
    __syncthreads();                          // previous tile fully consumed; qs ready on the first pass
    if (tid < DA_TILE) {
      const int kk = tile0 + tid;
      long long base = -1;
      if (kk <= p && kk >= kstart) {
        const int page = table[kk / page_size];
        if (page < 0 || page >= num_pages) report_error(err, PHOTON_DEV_BAD_PAGE, t, kk, page);
        else base = ((long long)page * n_kv + g) * page_size + (kk % page_size);      // the key's row in the cache
      }
      kbase[tid] = base;
    }
    __syncthreads();
    for (int i = tid; i < DA_TILE * d2; i += DA_THREADS) {
      const int key = i / d2, j = i - key * d2;
      const long long base = kbase[key];
      ks[key * kld + j] = base >= 0 ? to_f32(k_cache[base * d2 + j]) : 0.f;
    }
    for (int i = tid; i < DA_TILE * dv; i += DA_THREADS) {
      const int key = i / dv, j = i - key * dv;
      const long long base = kbase[key];
      vs[i] = base >= 0 ? to_f32(v_cache[base * dv + j]) : 0.f;
    }
    __syncthreads();
    // scores of every (head, map) row against the tile's keys
    for (int i = tid; i < R * DA_TILE; i += DA_THREADS) {
      const int r = i / DA_TILE, key = i - r * DA_TILE;
      float s = -INFINITY;
      if (kbase[key] >= 0) {
        const float* qh = qs + r * d;
        const float* kr = ks + key * kld + (r & 1) * d;
        float dot = 0.f;
        for (int j = 0; j < d; ++j) dot += qh[j] * kr[j];
        s = dot * scale;
      }
      sc[i] = s;
    }
    __syncthreads();
    // running softmax, one warp per row, one lane per key of the tile
    for (int r = warp; r < R; r += DA_THREADS / 32) {
      const float s = sc[r * DA_TILE + lane];
      const float tmax = warp_max(s);
      const float m_old = mrun[r];
      const float m_new = fmaxf(m_old, tmax);
      const float pr = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float psum = warp_sum(pr);
      const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
      __syncwarp();
      sc[r * DA_TILE + lane] = pr;
      if (lane == 0) { mrun[r] = m_new; lsum[r] = lsum[r] * c + psum; corr[r] = c; }
    }
    __syncthreads();
    // weighted values: both maps of a head read the same values
#pragma unroll
    for (int n = 0; n < PPT; ++n) {
      const int i = tid + n * DA_THREADS;
      if (i < R * dv) {
        const int r = i / dv, j = i - r * dv;
        float a = acc[n] * corr[r];
        const float* pr = sc + r * DA_TILE;
#pragma unroll 8
        for (int key = 0; key < DA_TILE; ++key) a += pr[key] * vs[key * dv + j];
        acc[n] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < PPT; ++n) {
    const int i = tid + n * DA_THREADS;
    if (i < R * dv) {
      const float l = lsum[i / dv];
      fin[i] = l > 0.f ? acc[n] / l : 0.f;
    }
  }
  __syncthreads();
  // the difference of the two maps and the head's norm, one warp per head
  for (int h = warp; h < NH; h += DA_THREADS / 32) {
    const float* a1 = fin + (size_t)(2 * h) * dv;
    const float* a2 = a1 + dv;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) { const float o = a1[j] - lambda * a2[j]; ss += o * o; }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)dv + eps);
    T* dst = out + (size_t)t * out_stride + (size_t)(h0 + h) * dv;
    for (int j = lane; j < dv; j += 32) dst[j] = from_f32<T>((a1[j] - lambda * a2[j]) * inv);
  }
}

template <typename T, int PPT>
static int diff_attention_launch(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                 const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                                 const int* positions, int T_, int n_q, int n_kv, int d, int dv, int hb, int page_size,
                                 int num_pages, int window, float scale, float lambda, float out_scale, float eps, int* err,
                                 cudaStream_t stream) {
  const size_t floats = (size_t)2 * hb * d + (size_t)DA_TILE * (2 * d + 1) + (size_t)DA_TILE * dv + (size_t)2 * hb * DA_TILE +
                        (size_t)2 * hb * dv + (size_t)6 * hb;
  const size_t smem = (floats + (floats & 1)) * sizeof(float) + DA_TILE * sizeof(long long);
  if (smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(diff_attention_kernel<T, PPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(T_, n_kv * ((n_q / n_kv + hb - 1) / hb));
  diff_attention_kernel<T, PPT><<<grid, DA_THREADS, smem, stream>>>(
      (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, block_table, max_pages, token_seq,
      positions, n_q, n_kv, d, dv, hb, page_size, num_pages, window, scale, lambda, out_scale, eps, err);
  return launch_status();
}

#define DA_ARGS q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_pages, token_seq, positions, T_, n_q, n_kv, \
                d, dv, hb, page_size, num_pages, window, scale, lambda, out_scale, eps, err, stream
#define DA_DISPATCH(TYPE)                                              \
  if (ppt <= 1) return diff_attention_launch<TYPE, 1>(DA_ARGS);        \
  if (ppt <= 2) return diff_attention_launch<TYPE, 2>(DA_ARGS);        \
  if (ppt <= 4) return diff_attention_launch<TYPE, 4>(DA_ARGS);        \
  if (ppt <= 8) return diff_attention_launch<TYPE, 8>(DA_ARGS);        \
  if (ppt <= 16) return diff_attention_launch<TYPE, 16>(DA_ARGS);      \
  if (ppt <= 32) return diff_attention_launch<TYPE, 32>(DA_ARGS);      \
  if (ppt <= 64) return diff_attention_launch<TYPE, 64>(DA_ARGS);      \
  return PHOTON_ERR_UNSUPPORTED;

// q [T][n_q * 2 d] (row stride q_stride), out [T][n_q * dv]; k_cache [pages][n_kv][page_size][2 d], v_cache
// [pages][n_kv][page_size][dv], all of `dtype`.  window <= 0: all keys.  lambda: the weight of the second map;
// out_scale: the factor behind the head norm.
PHOTON_API int photon_diff_attention(const void* q, long q_stride, void* out, long out_stride, int dtype, const void* k_cache,
                                     const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                                     const int* positions, int T_, int n_q, int n_kv, int d, int dv, int page_size,
                                     int num_pages, int window, float scale, float lambda, float out_scale, float eps,
                                     int* err, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (n_kv <= 0 || n_q <= 0 || n_q % n_kv || d <= 0 || dv <= 0 || page_size <= 0) return PHOTON_ERR_ARGUMENT;
  if (T_ > 65535 * 32 || d > 2048 || dv > 4096) return PHOTON_ERR_UNSUPPORTED;
  const int widest = 2 * d > dv ? 2 * d : dv;
  int hb = 4096 / widest;
  if (hb < 1) hb = 1;
  if (hb > n_q / n_kv) hb = n_q / n_kv;
  if ((long)n_kv * ((n_q / n_kv + hb - 1) / hb) > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int ppt = (2 * hb * dv + DA_THREADS - 1) / DA_THREADS;
  if (dtype == PHOTON_BF16) { DA_DISPATCH(bf16) }
  DA_DISPATCH(float)
}
