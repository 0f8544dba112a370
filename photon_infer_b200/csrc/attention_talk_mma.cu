// Paged causal attention whose heads talk to each other before the softmax, on the tensor cores: bfloat16, head
// sizes that are a multiple of 16, compiled per model with -DHEAD_DIM=<d> -DTALK_H=<heads> -DTALK_G=<key/value heads>.
//
//   raw_g(i, j)  = q_g(i) . k_{g / (H/G)}(j)
//   s_h(i, j)    = sum_g talk[h][g] qmul[g] raw_g(i, j)                all H heads, across the key/value groups
//   p_h(i, j)    = exp(s_h(i, j)) / (exp(sink[h]) + sum_j' exp(s_h(i, j')))      over the keys i sees
//   o_h(i)       = sigmoid(gate_h(i)) * sum_j p_h(i, j) v_{h / (H/G)}(j)
//
// Every head's score needs every other head's for the same pair of tokens, so one block owns 16 neighbouring tokens
// of a request with ALL their heads and walks the keys in tiles.  A tile passes three phases:
//   1. raw scores: the warp that owns head g forms the 16 x TILE matrix Q_g K^T (mma.m16n8k16, 32-bit sums) and
//      leaves it in shared memory, [head][row][key];
//   2. mixing: a thread takes two neighbouring pairs (i, j), reads their H raw scores, forms the H mixed ones with
//      32-bit multiply-adds (talk times qmul from shared memory, broadcast) and puts them back in place; pairs that
//      row i does not see are skipped;
//   3. softmax and values: the warp that owns head h reads S_h back in the layout of an mma A operand, keeps a
//      running maximum and sum per row in 32-bit, rounds the weights to bfloat16 and adds P V to its accumulators.
// Keys and values stream from the paged cache by cp.async while phase 2 runs: the tile's values and the next tile's
// keys.  Two block-wide barriers a tile (after phase 1 and after phase 2); phase 3 of a tile and phase 1 of the next
// follow each other inside a warp, which owns the same heads in both.  A token's key tiles may be shared out over `splits` blocks (decode steps): each
// leaves (maximum, sum, weighted sums) per head, merged in split order by photon_talk_merge (attention_talk.cu).
//
// Window: position i sees keys max(0, i - window + 1) .. i.  sink and gate may be null; talk null mixes nothing
// (s_h = qmul[h] raw_h).  Cache planes [pages][G][page_size][d]; the value plane holds whatever talk_prep wrote there.
#include "common.cuh"
#include <math.h>
#include <type_traits>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif
#ifndef TALK_H
#define TALK_H 4
#endif
#ifndef TALK_G
#define TALK_G 1
#endif

static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size");
static_assert(TALK_H % TALK_G == 0, "query heads per key/value head");

constexpr int TM_NW = TALK_H <= 8 ? (TALK_H < 4 ? 4 : TALK_H) : 16;       // warps; a warp owns heads warp, warp + NW, ...
constexpr int TM_HPW = (TALK_H + TM_NW - 1) / TM_NW;                      // heads a warp owns
constexpr int TM_THREADS = TM_NW * 32;
constexpr int TM_LD = HEAD_DIM + 8;                                       // padded rows: conflict-free ldmatrix
constexpr int TM_KD = HEAD_DIM / 16, TM_ND = HEAD_DIM / 8;
constexpr int TM_HP = (TALK_H + 3) & ~3;                                  // a row of the mixing matrix, padded to float4
// the accumulators of a warp's heads must fit its registers (128 a thread with 16 warps, 255 with up to 8)
static_assert(TM_HPW * HEAD_DIM <= (TM_NW > 8 ? 128 : 256), "heads x head size too large for this kernel");

constexpr size_t tm_smem_bytes(int bn) {
  return (size_t)TALK_H * 16 * TM_LD * 2 + (size_t)2 * TALK_G * bn * TM_LD * 2 + (size_t)TALK_H * 16 * (bn + 8) * 4 +
         (size_t)TALK_H * TM_HP * 8 + 32 * 4;
}
constexpr int TM_BN = tm_smem_bytes(64) <= 226 * 1024 ? 64 : 32;          // keys per tile
static_assert(tm_smem_bytes(TM_BN) <= 226 * 1024, "shared memory");
constexpr int TM_SLD = TM_BN + 8;                                         // padded score rows (floats)
constexpr float TM_LOG2E = 1.4426950408889634f, TM_LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t tm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_cp16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;           // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tm_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void tm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tm_ldsm4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(tm_smem(p)));
}
__device__ __forceinline__ void tm_ldsm4t(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(tm_smem(p)));
}
__device__ __forceinline__ void tm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float tm_exp2(float x) {         // 2^x; -inf gives 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t tm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct TalkMmaParams {
  const bf16* q; long q_stride;           // [T, H * d]
  bf16* out; long out_stride;             // [T, H * d]
  const bf16* k_cache; const bf16* v_cache;   // [pages, G, page_size, d]
  const int* block_table; int max_pages;  // [S, max_pages]
  const int* cu_tokens;                   // [S + 1] first token of each request in the step
  const int* positions;                   // [T], ascending by one inside a request
  int page_size, page_shift, num_pages, window, splits, tiles_per_seq;   // page_shift: log2(page_size) or -1
  const float* qmul; const float* talk; const float* sink;
  const float* gate; long gate_stride;    // float rows of H numbers, or null
  float* part;                            // splits > 1: [T][splits][H][d + 2]
  int* err;
};

__global__ void __launch_bounds__(TM_THREADS, 1) talk_mma_kernel(const TalkMmaParams P) {
  extern __shared__ __align__(16) unsigned char tm_dyn[];
  bf16* Qs = reinterpret_cast<bf16*>(tm_dyn);                              // [H][16][LD]
  bf16* Ks = Qs + TALK_H * 16 * TM_LD;                                     // [G][BN][LD]
  bf16* Vs = Ks + TALK_G * TM_BN * TM_LD;                                  // [G][BN][LD]
  float* Sb = reinterpret_cast<float*>(Vs + TALK_G * TM_BN * TM_LD);       // [H][16][SLD]
  float2* Tm = reinterpret_cast<float2*>(Sb + TALK_H * 16 * TM_SLD);       // [H][HP]: talk[h][g] * qmul[g], twice (packed multiply-adds)
  int* pos_s = reinterpret_cast<int*>(Tm + TALK_H * TM_HP);                // [16] position of each row, -1: no row
  int* lo_s = pos_s + 16;                                                  // [16] first key each row sees
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = blockIdx.x / P.tiles_per_seq;
  const int qtile = P.tiles_per_seq - 1 - (blockIdx.x - seq * P.tiles_per_seq);   // tiles with the most keys start first
  const int split = blockIdx.y;
  const int tok0 = P.cu_tokens[seq], ntok = P.cu_tokens[seq + 1] - tok0;
  const int row0 = qtile * 16;
  if (row0 >= ntok) return;
  const int nrows = min(16, ntok - row0);
  const int tfirst = tok0 + row0;
  const int* table = P.block_table + (size_t)seq * P.max_pages;
  constexpr int hpg = TALK_H / TALK_G;
  constexpr int CPR = HEAD_DIM / 8;                                        // 16-byte chunks per row

  if (tid < 16) {
    const int p = tid < nrows ? P.positions[tfirst + tid] : -1;
    pos_s[tid] = p;
    lo_s[tid] = (P.window > 0 && p - P.window + 1 > 0) ? p - P.window + 1 : 0;
  }
  for (int i = tid; i < TALK_H * TM_HP; i += TM_THREADS) {
    const int h = i / TM_HP, g = i - h * TM_HP;
    float w = 0.f;
    if (g < TALK_H) w = (P.talk ? P.talk[h * TALK_H + g] : (h == g ? 1.f : 0.f)) * P.qmul[g];
    Tm[i] = make_float2(w, w);
  }
  const int pos_first = P.positions[tfirst], pos_last = P.positions[tfirst + nrows - 1];
  const int key_lo = (P.window > 0 && pos_first - P.window + 1 > 0) ? pos_first - P.window + 1 : 0;
  int tile_begin = key_lo / TM_BN, tile_end = pos_last / TM_BN + 1;
  if (P.splits > 1) {
    const int per = (tile_end - tile_begin + P.splits - 1) / P.splits;
    tile_begin += split * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  const int ntiles = max(0, tile_end - tile_begin);

  // one plane (keys or values) of a tile: all key/value heads, zeros for keys no row of the block sees
  auto load_plane = [&](const bf16* cache, bf16* dst, int key0) {
    for (int c = tid; c < TALK_G * TM_BN * CPR; c += TM_THREADS) {
      const int row = c / CPR, cc = c - row * CPR;
      const int g = row / TM_BN, r = row - g * TM_BN;
      const int key = key0 + r;
      bool valid = key >= key_lo && key <= pos_last;
      size_t src = 0;
      if (valid) {
        const int pidx = P.page_shift >= 0 ? (key >> P.page_shift) : key / P.page_size;
        const int page = table[pidx];
        if (page < 0 || page >= P.num_pages) {
          if (cc == 0 && g == 0) report_error(P.err, PHOTON_DEV_BAD_PAGE, tfirst, key, page);
          valid = false;
        } else {
          src = (((size_t)page * TALK_G + g) * P.page_size + (key - pidx * P.page_size)) * HEAD_DIM + cc * 8;
        }
      }
      tm_cp16(dst + row * TM_LD + cc * 8, cache + src, valid);
    }
  };
  // the queries of the 16 rows, all heads (zeros beyond the request's rows); they join the first group of copies
  for (int c = tid; c < TALK_H * 16 * CPR; c += TM_THREADS) {
    const int row = c / CPR, cc = c - row * CPR;
    const int h = row >> 4, i = row & 15;
    const bool valid = i < nrows;
    const size_t src = valid ? (size_t)(tfirst + i) * P.q_stride + (size_t)h * HEAD_DIM + cc * 8 : 0;
    tm_cp16(Qs + row * TM_LD + cc * 8, P.q + src, valid);
  }
  if (ntiles > 0) load_plane(P.k_cache, Ks, tile_begin * TM_BN);
  tm_commit();

  float m[TM_HPW][2], l[TM_HPW][2], o[TM_HPW][TM_ND][4];
#pragma unroll
  for (int hh = 0; hh < TM_HPW; ++hh) {
    m[hh][0] = m[hh][1] = -INFINITY; l[hh][0] = l[hh][1] = 0.f;
#pragma unroll
    for (int n = 0; n < TM_ND; ++n) { o[hh][n][0] = o[hh][n][1] = o[hh][n][2] = o[hh][n][3] = 0.f; }
  }
  const int r0 = lane >> 2, c2 = (lane & 3) * 2;

  for (int it = 0; it < ntiles; ++it) {
    const int key_base = (tile_begin + it) * TM_BN;
    if (it == 0) {
      tm_wait<0>();
      __syncthreads();                                 // Q, the first tile's keys, Tm and pos_s are in place
    }
    // ---- 1. raw scores of the warp's heads
#pragma unroll
    for (int hh = 0; hh < TM_HPW; ++hh) {
      const int h = warp + hh * TM_NW;
      if (h >= TALK_H) break;
      const bf16* kg = Ks + (size_t)(h / hpg) * TM_BN * TM_LD;
      float s[TM_BN / 8][4];
#pragma unroll
      for (int j = 0; j < TM_BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
      for (int kd = 0; kd < TM_KD; ++kd) {
        uint32_t a[4];
        tm_ldsm4(a, Qs + (h * 16 + (lane & 15)) * TM_LD + kd * 16 + ((lane >> 4) << 3));
#pragma unroll
        for (int j = 0; j < TM_BN / 8; j += 2) {
          uint32_t b[4];
          tm_ldsm4(b, kg + (j * 8 + (lane & 7) + ((lane >> 4) << 3)) * TM_LD + kd * 16 + (((lane >> 3) & 1) << 3));
          tm_mma(s[j], a, b[0], b[1]);
          tm_mma(s[j + 1], a, b[2], b[3]);
        }
      }
      float* S0 = Sb + (h * 16 + r0) * TM_SLD + c2;
#pragma unroll
      for (int j = 0; j < TM_BN / 8; ++j) {
        *reinterpret_cast<float2*>(S0 + j * 8) = make_float2(s[j][0], s[j][1]);
        *reinterpret_cast<float2*>(S0 + 8 * TM_SLD + j * 8) = make_float2(s[j][2], s[j][3]);
      }
    }
    __syncthreads();                                   // raw scores complete; every warp has left the tile before: the
                                                       // key tile and the value tile are free
    load_plane(P.v_cache, Vs, key_base);
    if (it + 1 < ntiles) load_plane(P.k_cache, Ks, key_base + TM_BN);
    tm_commit();
    // ---- 2. the heads' scores are mixed, two neighbouring keys of one row per thread
    for (int idx = tid; idx < nrows * (TM_BN / 2); idx += TM_THREADS) {
      const int i = idx / (TM_BN / 2), j = (idx - i * (TM_BN / 2)) * 2;
      const int key = key_base + j;
      if (key > pos_s[i] || key + 1 < lo_s[i]) continue;               // neither key is seen by this row
      float* cell = Sb + i * TM_SLD + j;
      float2 raw[TALK_H];
#pragma unroll
      for (int g = 0; g < TALK_H; ++g) raw[g] = *reinterpret_cast<const float2*>(cell + g * 16 * TM_SLD);
#pragma unroll
      for (int h = 0; h < TALK_H; ++h) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int g2 = 0; g2 < TM_HP; g2 += 2) {
          const float4 w = *reinterpret_cast<const float4*>(Tm + h * TM_HP + g2);      // (w_g, w_g, w_g+1, w_g+1)
          if (g2 < TALK_H) acc = __ffma2_rn(make_float2(w.x, w.y), raw[g2], acc);
          if (g2 + 1 < TALK_H) acc = __ffma2_rn(make_float2(w.z, w.w), raw[g2 + 1], acc);
        }
        *reinterpret_cast<float2*>(cell + h * 16 * TM_SLD) = acc;
      }
    }
    tm_wait<0>();
    __syncthreads();                                   // mixed scores complete; this tile's values and the next tile's keys
                                                       // are in place
    // ---- 3. running softmax and P V of the warp's heads
    const int p0 = pos_s[r0], p1 = pos_s[r0 + 8], lo0 = lo_s[r0], lo1 = lo_s[r0 + 8];
    // every row of the block sees every key of the tile: the comparisons are left out
    const bool whole = nrows == 16 && key_base >= lo_s[15] && key_base + TM_BN - 1 <= pos_s[0];
    auto phase3 = [&](auto masked) {
    constexpr bool MASK = decltype(masked)::value;
#pragma unroll
    for (int hh = 0; hh < TM_HPW; ++hh) {
      const int h = warp + hh * TM_NW;
      if (h >= TALK_H) break;
      const bf16* vg = Vs + (size_t)(h / hpg) * TM_BN * TM_LD;
      const float* S0 = Sb + (h * 16 + r0) * TM_SLD + c2;
      const float* S1 = S0 + 8 * TM_SLD;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < TM_BN / 8; ++j) {
        const int key = key_base + j * 8 + c2;
        const float2 a = *reinterpret_cast<const float2*>(S0 + j * 8), b = *reinterpret_cast<const float2*>(S1 + j * 8);
        if (!MASK || (key >= lo0 && key <= p0)) mx0 = fmaxf(mx0, a.x);
        if (!MASK || (key + 1 >= lo0 && key + 1 <= p0)) mx0 = fmaxf(mx0, a.y);
        if (!MASK || (key >= lo1 && key <= p1)) mx1 = fmaxf(mx1, b.x);
        if (!MASK || (key + 1 >= lo1 && key + 1 <= p1)) mx1 = fmaxf(mx1, b.y);
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      // the running maximum is kept in units of log2: weights are 2^(s log2(e) - m)
      const float mn0 = fmaxf(m[hh][0], mx0 * TM_LOG2E), mn1 = fmaxf(m[hh][1], mx1 * TM_LOG2E);
      const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
      const float corr0 = tm_exp2(m[hh][0] - sub0), corr1 = tm_exp2(m[hh][1] - sub1);
      m[hh][0] = mn0; m[hh][1] = mn1;
#pragma unroll
      for (int n = 0; n < TM_ND; ++n) { o[hh][n][0] *= corr0; o[hh][n][1] *= corr0; o[hh][n][2] *= corr1; o[hh][n][3] *= corr1; }
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int kk = 0; kk < TM_BN / 16; ++kk) {
        uint32_t pa[4];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = kk * 2 + jj;
          const int key = key_base + j * 8 + c2;
          const float2 a = *reinterpret_cast<const float2*>(S0 + j * 8), b = *reinterpret_cast<const float2*>(S1 + j * 8);
          const float w00 = (!MASK || (key >= lo0 && key <= p0)) ? tm_exp2(fmaf(a.x, TM_LOG2E, -sub0)) : 0.f;
          const float w01 = (!MASK || (key + 1 >= lo0 && key + 1 <= p0)) ? tm_exp2(fmaf(a.y, TM_LOG2E, -sub0)) : 0.f;
          const float w10 = (!MASK || (key >= lo1 && key <= p1)) ? tm_exp2(fmaf(b.x, TM_LOG2E, -sub1)) : 0.f;
          const float w11 = (!MASK || (key + 1 >= lo1 && key + 1 <= p1)) ? tm_exp2(fmaf(b.y, TM_LOG2E, -sub1)) : 0.f;
          sum0 += w00 + w01; sum1 += w10 + w11;
          pa[jj * 2] = tm_pack(w00, w01);
          pa[jj * 2 + 1] = tm_pack(w10, w11);
        }
#pragma unroll
        for (int n = 0; n < TM_ND; n += 2) {
          uint32_t b[4];
          tm_ldsm4t(b, vg + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * TM_LD + n * 8 + ((lane >> 4) << 3));
          tm_mma(o[hh][n], pa, b[0], b[1]);
          tm_mma(o[hh][n + 1], pa, b[2], b[3]);
        }
      }
      l[hh][0] = l[hh][0] * corr0 + sum0;              // per-lane partial sums; the quad is added up at the end
      l[hh][1] = l[hh][1] * corr1 + sum1;
    }
    };
    if (whole) phase3(std::false_type{}); else phase3(std::true_type{});
    // no barrier here: a warp goes on to the raw scores of the next tile, which it writes into the rows of S that only
    // it has just read; the next tile's first barrier keeps the mixing and the value tile behind the slowest warp
  }
  tm_wait<0>();
  pdl_launch_dependents();

#pragma unroll
  for (int hh = 0; hh < TM_HPW; ++hh) {
    const int h = warp + hh * TM_NW;
    if (h >= TALK_H) break;
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      float ll = l[hh][h2];
      ll += __shfl_xor_sync(0xffffffffu, ll, 1);
      ll += __shfl_xor_sync(0xffffffffu, ll, 2);
      const int row = r0 + h2 * 8;
      if (row >= nrows) continue;
      const int t = tfirst + row;
      const float mm = m[hh][h2];
      if (P.splits > 1) {
        float* dst = P.part + (((size_t)t * P.splits + split) * TALK_H + h) * (HEAD_DIM + 2);
        if ((lane & 3) == 0) { dst[0] = mm * TM_LN2; dst[1] = ll; }      // the merge works with natural logarithms
#pragma unroll
        for (int n = 0; n < TM_ND; ++n)
          *reinterpret_cast<float2*>(dst + 2 + n * 8 + c2) = make_float2(o[hh][n][h2 * 2], o[hh][n][h2 * 2 + 1]);
        continue;
      }
      float keep = 1.f;
      if (P.sink) {
        const float sk = P.sink[h] * TM_LOG2E;
        const float M = fmaxf(mm, sk);
        keep = (mm == -INFINITY) ? 0.f : tm_exp2(mm - M);
        ll = ll * keep + tm_exp2(sk - M);
      }
      float f = ll > 0.f ? keep / ll : 0.f;
      if (P.gate) f *= 1.0f / (1.0f + expf(-P.gate[(size_t)t * P.gate_stride + h]));
      bf16* dst = P.out + (size_t)t * P.out_stride + (size_t)h * HEAD_DIM + c2;
#pragma unroll
      for (int n = 0; n < TM_ND; ++n)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[hh][n][h2 * 2] * f, o[hh][n][h2 * 2 + 1] * f);
    }
  }
}

// q, out [T, H * d] bfloat16 (row strides in elements); k_cache, v_cache [num_pages, G, page_size, d] bfloat16;
// block_table [S, max_pages]; cu_tokens [S + 1]; positions [T]; max_tokens: the most tokens a request brings;
// qmul float [H]; talk float [H, H], sink float [H], gate float rows of H (stride gate_stride): each may be null;
// window 0: none.  H, G and d must be the values the module was compiled for.  splits > 1: part float
// [T * splits * H * (d + 2)] gets every split's share, for photon_talk_merge.
PHOTON_API int photon_talk_mma(const void* q, long q_stride, void* out, long out_stride, const void* k_cache, const void* v_cache,
                               const int* block_table, int max_pages, const int* cu_tokens, const int* positions, int S,
                               int max_tokens, int H, int G, int d, int page_size, int num_pages, int window,
                               const float* qmul, const float* talk, const float* sink, const float* gate, long gate_stride,
                               int splits, float* part, int* err, cudaStream_t stream) {
  if (S <= 0 || max_tokens <= 0) return 0;
  if (H != TALK_H || G != TALK_G || d != HEAD_DIM) return PHOTON_ERR_UNSUPPORTED;
  if (window < 0 || splits < 1 || qmul == nullptr || page_size <= 0 || (splits > 1 && part == nullptr)) return PHOTON_ERR_ARGUMENT;
  if ((q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16) ||
      ((uintptr_t)out % 4) || ((uintptr_t)part % 8))
    return PHOTON_ERR_ARGUMENT;
  TalkMmaParams P;
  P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out; P.out_stride = out_stride;
  P.k_cache = (const bf16*)k_cache; P.v_cache = (const bf16*)v_cache; P.block_table = block_table; P.max_pages = max_pages;
  P.cu_tokens = cu_tokens; P.positions = positions; P.page_size = page_size; P.num_pages = num_pages;
  P.page_shift = -1;
  for (int b = 0; b < 31; ++b) if ((1 << b) == page_size) P.page_shift = b;
  P.window = window;
  P.splits = splits; P.tiles_per_seq = (max_tokens + 15) / 16; P.qmul = qmul; P.talk = talk; P.sink = sink; P.gate = gate;
  P.gate_stride = gate_stride; P.part = part; P.err = err;
  const long blocks = (long)S * P.tiles_per_seq;
  if (blocks > 2147483647L || splits > 65535) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = tm_smem_bytes(TM_BN);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(talk_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  return launch_pdl(talk_mma_kernel, dim3((unsigned)blocks, splits), dim3(TM_THREADS), smem, stream, P);
}
