// Differential attention on the tensor cores (bfloat16; -DDIFF_D=<size of a map's key>, -DDIFF_DV=<size of a value>, both
// multiples of 16).  The formulas are those of attention_diff.cu.
//
// A block owns 64 rows: the query heads that share ONE key/value head, for up to 64 / (heads per key/value head)
// neighbouring tokens of one request, so a key tile that comes into shared memory serves all of them.  Its eight warps
// are four groups of 16 rows times the two maps: warp (group, map) runs an attention of its own, S = Q_m K_m^T
// (mma.m16n8k16, 32-bit sums), running maximum and sum in 32-bit, weights rounded to bfloat16, O_m += P V, over key
// tiles of 64.  Both maps read the same value tile; a key's row in the cache holds both maps side by side, so one copy
// brings both.  Tiles arrive by cp.async into two stages (16-byte chunks, swizzled by the key's number so that
// ldmatrix meets no bank twice).  At the end the two maps' outputs meet in shared memory: o = a_1 - lambda a_2, the
// head's norm over its DV numbers, one rounding.  The key tiles start at a multiple of 64 at or below the first key
// that the block's first token sees, so a token's sums depend on its place in the block, which is why this kernel
// serves the bfloat16 run only (its float32 run keeps the general kernel, whose sums depend on the position alone).
// Decode steps share a token's key tiles out over several blocks; a second kernel puts the shares together.
#include "common.cuh"
#include <math.h>
#include <mma.h>

#ifndef DIFF_D
#define DIFF_D 128
#endif
#ifndef DIFF_DV
#define DIFF_DV 256
#endif
#define DM_KT 64
#define DM_ROWS 64
#define DM_THREADS 256

static_assert(DIFF_D % 16 == 0 && DIFF_DV % 16 == 0, "sizes must be multiples of 16");

__device__ __forceinline__ uint32_t dm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dm_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dm_smem(dst)), "l"(src));
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void dm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void dm_ldm4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dm_smem(p)));
}
__device__ __forceinline__ void dm_ldm4t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(dm_smem(p)));
}
__device__ __forceinline__ void dm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Rows of `width` bfloat16 (a multiple of 8) in shared memory; the 16-byte chunk c of row r lies at chunk c ^ (r & 7)
// within its group of eight chunks, when a row is whole groups (else the rows lie as they are, at the price of bank
// conflicts).
__device__ __forceinline__ int dm_at(int row, int chunk, int width) {
  return (width % 64 == 0) ? row * width + (((chunk & ~7) | ((chunk ^ row) & 7)) << 3) : row * width + (chunk << 3);
}

__global__ void __launch_bounds__(DM_THREADS, 1)
diff_mma_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const int* __restrict__ block_table,
                int max_pages, const int* __restrict__ cu_tokens, const int* __restrict__ positions, int num_seqs, int n_q,
                int n_kv, int page_size, int num_pages, int window, float scale, float lambda, float out_scale, float eps,
                int tokens_per_block, int splits, float* __restrict__ part, int* err) {
  constexpr int D = DIFF_D, DV = DIFF_DV, D2 = 2 * DIFF_D;
  extern __shared__ __align__(128) unsigned char dm_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(dm_raw);                       // [64][2 D]
  bf16* Ks = Qs + DM_ROWS * D2;                                     // [2][KT][2 D]
  bf16* Vs = Ks + 2 * DM_KT * D2;                                   // [2][KT][DV]
  float* fin = reinterpret_cast<float*>(Ks);                        // [2][64][DV], over the stages when the walk is done
  __shared__ long long krow[2][DM_KT];
  __shared__ int row_pos[DM_ROWS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int GH = n_q / n_kv;
  const int g = blockIdx.y;
  // which request and which of its token tiles this block owns
  // (the last tiles first: with a causal walk they are the longest, and the short ones fill the tail of the grid)
  int s = 0, tile = gridDim.x - 1 - blockIdx.x, t_first = 0, n_tok = 0;
  for (; s < num_seqs; ++s) {
    t_first = cu_tokens[s];
    n_tok = cu_tokens[s + 1] - t_first;
    const int tiles = (n_tok + tokens_per_block - 1) / tokens_per_block;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (s >= num_seqs) return;
  const int tok0 = t_first + tile * tokens_per_block;
  const int ntok = min(tokens_per_block, t_first + n_tok - tok0);
  const int rows = ntok * GH;                                       // rows in use: (token, head of the group)
  const int p_first = positions[tok0], p_last = positions[tok0 + ntok - 1];
  const int kmin = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  int tile_lo = kmin / DM_KT, tile_hi = p_last / DM_KT + 1;
  if (splits > 1) {
    // this block's share of the key tiles; the shares of a row meet in diff_merge_kernel, in the order of the shares
    const int per = (tile_hi - tile_lo + splits - 1) / splits;
    tile_lo += blockIdx.z * per;
    tile_hi = min(tile_hi, tile_lo + per);
  }
  const int* table = block_table + (size_t)s * max_pages;

  for (int r = tid; r < DM_ROWS; r += DM_THREADS) row_pos[r] = r < rows ? positions[tok0 + r / GH] : -1;
  // queries: row r = (token r / GH, head r % GH); both maps of a head side by side
  for (int i = tid; i < DM_ROWS * (D2 / 8); i += DM_THREADS) {
    const int r = i / (D2 / 8), c = i - r * (D2 / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + r / GH) * q_stride + (size_t)(g * GH + r % GH) * D2 + c * 8);
    *reinterpret_cast<uint4*>(Qs + dm_at(r, c, D2)) = v;
  }

  auto load_tile = [&](int kt, int stage) {
    if (tid < DM_KT) {
      const int kk = kt * DM_KT + tid;
      long long base = -1;
      if (kk <= p_last && kk >= kmin) {
        const int page = table[kk / page_size];
        if (page < 0 || page >= num_pages) report_error(err, PHOTON_DEV_BAD_PAGE, tok0, kk, page);
        else base = ((long long)page * n_kv + g) * page_size + (kk % page_size);
      }
      krow[stage][tid] = base;
    }
  };
  auto copy_tile = [&](int stage) {
    bf16* kd = Ks + (size_t)stage * DM_KT * D2;
    bf16* vd = Vs + (size_t)stage * DM_KT * DV;
    for (int i = tid; i < DM_KT * (D2 / 8); i += DM_THREADS) {
      const int key = i / (D2 / 8), c = i - key * (D2 / 8);
      const long long base = krow[stage][key];
      bf16* dst = kd + dm_at(key, c, D2);
      if (base >= 0) dm_cp16(dst, k_cache + base * D2 + c * 8);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < DM_KT * (DV / 8); i += DM_THREADS) {
      const int key = i / (DV / 8), c = i - key * (DV / 8);
      const long long base = krow[stage][key];
      bf16* dst = vd + dm_at(key, c, DV);
      if (base >= 0) dm_cp16(dst, v_cache + base * DV + c * 8);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  };

  const int rg = warp >> 1, mp = warp & 1;                           // this warp's 16 rows and its map
  const int r_lo = rg * 16 + (lane >> 2), r_hi = r_lo + 8;          // the two rows this lane holds parts of
  float o[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  if (tile_lo < tile_hi) load_tile(tile_lo, 0);
  __syncthreads();                                                  // krow, row_pos and Qs are written
  if (tile_lo < tile_hi) { copy_tile(0); dm_commit(); }
  const int p_lo = row_pos[r_lo], p_hi = row_pos[r_hi];
  const float sl2 = scale * 1.4426950408889634f;                    // scores in units of log 2
  for (int kt = tile_lo; kt < tile_hi; ++kt) {
    const int stage = (kt - tile_lo) & 1;
    __syncthreads();                                                // the other stage is consumed by every warp
    if (kt + 1 < tile_hi) load_tile(kt + 1, stage ^ 1);
    __syncthreads();                                                // the next tile's rows are known
    if (kt + 1 < tile_hi) { copy_tile(stage ^ 1); dm_commit(); dm_wait<1>(); } else dm_wait<0>();
    __syncthreads();                                                // this stage has landed for every thread
    const bf16* kd = Ks + (size_t)stage * DM_KT * D2;
    const bf16* vd = Vs + (size_t)stage * DM_KT * DV;
    // S = Q_m K_m^T for 16 rows x 64 keys
    float sc[DM_KT / 8][4];
#pragma unroll
    for (int n = 0; n < DM_KT / 8; ++n) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      {
        const int row = rg * 16 + (lane & 15), chunk = (mp * D + ks * 16) / 8 + (lane >> 4);
        dm_ldm4(a, Qs + dm_at(row, chunk, D2));
      }
#pragma unroll
      for (int np = 0; np < DM_KT / 16; ++np) {
        uint32_t b[4];
        const int key = np * 16 + (lane & 7) + ((lane >> 4) << 3), chunk = (mp * D + ks * 16) / 8 + ((lane >> 3) & 1);
        dm_ldm4(b, kd + dm_at(key, chunk, D2));
        dm_mma(sc[2 * np], a, b[0], b[1]);
        dm_mma(sc[2 * np + 1], a, b[2], b[3]);
      }
    }
    // who sees whom, the running maximum and sum
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < DM_KT / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * DM_KT + n * 8 + (lane & 3) * 2 + (e & 1);
        const int p = (e < 2) ? p_lo : p_hi;
        const bool ok = key <= p && (window <= 0 || p - key < window) && krow[stage][key - kt * DM_KT] >= 0;
        const float v = ok ? sc[n][e] * sl2 : -INFINITY;
        sc[n][e] = v;
        if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
    const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);       // exp2(-inf) = 0 for a row that has seen nothing
    m_lo = mn_lo; m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
    uint32_t pa[DM_KT / 16][4];
#pragma unroll
    for (int n = 0; n < DM_KT / 8; ++n) {
      const float e0 = exp2f(sc[n][0] - ref_lo), e1 = exp2f(sc[n][1] - ref_lo);
      const float e2 = exp2f(sc[n][2] - ref_hi), e3 = exp2f(sc[n][3] - ref_hi);
      ps_lo += e0 + e1; ps_hi += e2 + e3;
      pa[n >> 1][(n & 1) * 2] = dm_pack(e0, e1);
      pa[n >> 1][(n & 1) * 2 + 1] = dm_pack(e2, e3);
    }
    l_lo = l_lo * c_lo + ps_lo;
    l_hi = l_hi * c_hi + ps_hi;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) { o[n][0] *= c_lo; o[n][1] *= c_lo; o[n][2] *= c_hi; o[n][3] *= c_hi; }
    // O_m += P V
#pragma unroll
    for (int kk = 0; kk < DM_KT / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < DV / 16; ++np) {
        uint32_t b[4];
        const int key = kk * 16 + (lane & 15), chunk = np * 2 + (lane >> 4);
        dm_ldm4t(b, vd + dm_at(key, chunk, DV));
        dm_mma(o[2 * np], pa[kk], b[0], b[1]);
        dm_mma(o[2 * np + 1], pa[kk], b[2], b[3]);
      }
    }
  }
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if (splits > 1) {
    // a share of the keys: the sums as they stand, with the running maximum (in units of log 2) and denominator behind them
    const int n_rows[2] = {r_lo, r_hi};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = n_rows[half];
      if (r >= rows) continue;
      float* dst = part + ((((size_t)(tok0 + r / GH) * n_q + (g * GH + r % GH)) * 2 + mp) * splits + blockIdx.z) * (DV + 2);
#pragma unroll
      for (int n = 0; n < DV / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8 + (lane & 3) * 2) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
      if ((lane & 3) == 0) { dst[DV] = half ? m_hi : m_lo; dst[DV + 1] = half ? l_hi : l_lo; }
    }
    return;
  }
  __syncthreads();                                                  // the stages are free: the maps' outputs go there
  {
    const float i_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
    float* f_lo = fin + ((size_t)mp * DM_ROWS + r_lo) * DV;
    float* f_hi = fin + ((size_t)mp * DM_ROWS + r_hi) * DV;
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      const int col = n * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(f_lo + col) = make_float2(o[n][0] * i_lo, o[n][1] * i_lo);
      *reinterpret_cast<float2*>(f_hi + col) = make_float2(o[n][2] * i_hi, o[n][3] * i_hi);
    }
  }
  __syncthreads();
  // the difference of the maps and the head's norm, a warp per row
  for (int r = warp; r < rows; r += DM_THREADS / 32) {
    const float* a1 = fin + (size_t)r * DV;
    const float* a2 = fin + ((size_t)DM_ROWS + r) * DV;
    float ss = 0.f;
    for (int j = lane; j < DV; j += 32) { const float x = a1[j] - lambda * a2[j]; ss += x * x; }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)DV + eps);
    bf16* dst = out + (size_t)(tok0 + r / GH) * out_stride + (size_t)(g * GH + r % GH) * DV;
    for (int j = lane; j < DV; j += 32) dst[j] = __float2bfloat16_rn((a1[j] - lambda * a2[j]) * inv);
  }
}

// The shares of one (token, head) put together, in the order of the shares, for both maps; then the difference of the
// maps and the head's norm.
__global__ void __launch_bounds__(128)
diff_merge_kernel(const float* __restrict__ part, int splits, bf16* __restrict__ out, long out_stride, int n_q, float lambda,
                  float out_scale, float eps) {
  constexpr int DV = DIFF_DV;
  __shared__ float a[2][DIFF_DV];
  __shared__ float red[32];
  const int t = blockIdx.x, h = blockIdx.y;
  for (int mp = 0; mp < 2; ++mp) {
    const float* src = part + (((size_t)t * n_q + h) * 2 + mp) * splits * (DV + 2);
    float m = -INFINITY;
    for (int z = 0; z < splits; ++z) m = fmaxf(m, src[z * (DV + 2) + DV]);
    float l = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = src[z * (DV + 2) + DV];
      if (mz != -INFINITY) l += src[z * (DV + 2) + DV + 1] * exp2f(mz - m);
    }
    for (int j = threadIdx.x; j < DV; j += blockDim.x) {
      float acc = 0.f;
      for (int z = 0; z < splits; ++z) {
        const float mz = src[z * (DV + 2) + DV];
        if (mz != -INFINITY) acc += src[z * (DV + 2) + j] * exp2f(mz - m);
      }
      a[mp][j] = l > 0.f ? acc / l : 0.f;
    }
  }
  __syncthreads();
  float ss = 0.f;
  for (int j = threadIdx.x; j < DV; j += blockDim.x) { const float x = a[0][j] - lambda * a[1][j]; ss += x * x; }
  ss = block_sum(ss, red);
  const float inv = out_scale / sqrtf(ss / (float)DV + eps);
  bf16* dst = out + (size_t)t * out_stride + (size_t)h * DV;
  for (int j = threadIdx.x; j < DV; j += blockDim.x) dst[j] = __float2bfloat16_rn((a[0][j] - lambda * a[1][j]) * inv);
}

PHOTON_API int photon_diff_mma_dims(void) { return DIFF_D * 65536 + DIFF_DV; }

// q [T][n_q * 2 D] bfloat16 (row stride q_stride, 16-byte aligned rows), out [T][n_q * DV]; k_cache [pages][n_kv][page_size][2 D],
// v_cache [pages][n_kv][page_size][DV].  cu_tokens [S + 1]: the first token of every request of the step; a request's
// tokens have consecutive positions.  window <= 0: all keys.  tiles: an upper bound of sum over requests of
// ceil(tokens / tokens_per_block), tokens_per_block = 64 / (n_q / n_kv).  splits > 1 (decode steps, where a block per
// (token tile, key/value head) leaves the GPU empty): every block's key tiles are shared out over that many blocks, which
// leave their shares in part (float [T * n_q * 2 * splits * (DV + 2)], T the step's tokens) for a second kernel to put together.
PHOTON_API int photon_diff_mma(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                               const void* v_cache, const int* block_table, int max_pages, const int* cu_tokens,
                               const int* positions, int num_seqs, int tiles, int n_q, int n_kv, int page_size, int num_pages,
                               int window, float scale, float lambda, float out_scale, float eps, int splits, float* part,
                               int num_tokens, int* err, cudaStream_t stream) {
  if (num_seqs <= 0 || tiles <= 0) return 0;
  if (splits < 1 || splits > 64 || (splits > 1 && (part == nullptr || num_tokens <= 0 || n_q > 65535))) return PHOTON_ERR_ARGUMENT;
  if (n_kv <= 0 || n_q <= 0 || n_q % n_kv || page_size <= 0) return PHOTON_ERR_ARGUMENT;
  const int GH = n_q / n_kv;
  if (GH > DM_ROWS || n_kv > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (q_stride % 8 || out_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return PHOTON_ERR_UNSUPPORTED;
  const size_t stages = (size_t)2 * DM_KT * (2 * DIFF_D + DIFF_DV) * sizeof(bf16);
  const size_t fin = (size_t)2 * DM_ROWS * DIFF_DV * sizeof(float);
  const size_t smem = (size_t)DM_ROWS * 2 * DIFF_D * sizeof(bf16) + (stages > fin ? stages : fin);
  if (smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(diff_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  diff_mma_kernel<<<dim3(tiles, n_kv, splits), DM_THREADS, smem, stream>>>(
      (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages,
      cu_tokens, positions, num_seqs, n_q, n_kv, page_size, num_pages, window, scale, lambda, out_scale, eps, DM_ROWS / GH,
      splits, part, err);
  int st = launch_status();
  if (st != 0 || splits <= 1) return st;
  diff_merge_kernel<<<dim3(num_tokens, n_q), 128, 0, stream>>>(part, splits, (bf16*)out, out_stride, n_q, lambda, out_scale, eps);
  return launch_status();
}
