// Row kernels around norms that work on parts of a row or on its powers.  All arithmetic is 32-bit; storage is
// float or bfloat16.
//
//   photon_group_rmsnorm   the row is cut into `groups` equal consecutive parts; each part is divided by its own
//                          sqrt(mean(part^2) + eps); the whole is multiplied by w.  Optionally the row is multiplied
//                          by silu(gate) before the norm, or by sigmoid(gate) after it.  The result is written out,
//                          or added to a 32-bit stream whose new row is written out in the run type as well
//                          (a layer whose norm sits on the sublayer's output: x <- x + norm(f(x))).
//   photon_polynorm        act(z) = a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(u) = u /
//                          sqrt(mean(u^2) + eps) over the row.
//   photon_softcap         x <- cap * tanh(x / cap), in place.
//
// Every sum runs over one row in an order that depends on the row's width alone, so a token's numbers do not
// depend on what else is in the step.
#include "common.cuh"
#include <math.h>

#define RN_THREADS 256

__device__ __forceinline__ float rn_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// gate_mode 0: no gate; 1: y = x * silu(gate) before the norm; 2: the normed row times sigmoid(gate).
template <typename TX, typename TO>
__global__ void __launch_bounds__(RN_THREADS)
group_rmsnorm_kernel(const TX* x, long x_stride, const float* gate, long gate_stride, int gate_mode, float* residual,
                     const void* __restrict__ w, int w_bf16, TO* out, long out_stride, int H, int groups, float eps,
                     const void* __restrict__ x_bias, int xb_bf16) {
  __shared__ float red[32];
  extern __shared__ __align__(16) float rn_stash[];              // H floats: the row as it enters the norm
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = RN_THREADS / 32;
  float* res = residual ? residual + (size_t)r * H : nullptr;
  TO* o = out ? out + (size_t)r * out_stride : nullptr;
  if (x == nullptr) {                                            // nothing pending: the stream's row in the run type
    if (o) for (int i = tid; i < H; i += RN_THREADS) o[i] = from_f32<TO>(res[i]);
    return;
  }
  const TX* xr = x + (size_t)r * x_stride;
  const float* gr = gate ? gate + (size_t)r * gate_stride : nullptr;
  for (int i = tid; i < H; i += RN_THREADS) {
    float v = to_f32(xr[i]);
    if (x_bias) v += load_w(x_bias, xb_bf16, i);                  // the bias of the product that made x
    if (gate_mode == 1) { const float z = gr[i]; v *= z * rn_sigmoid(z); }
    rn_stash[i] = v;
  }
  __syncthreads();
  const int gs = H / groups;
  if (groups >= nwarp) {
    // a warp per part: no barrier between parts
    for (int g = warp; g < groups; g += nwarp) {
      const float* p = rn_stash + (size_t)g * gs;
      float ss = 0.f;
      for (int i = lane; i < gs; i += 32) ss += p[i] * p[i];
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
      for (int i = lane; i < gs; i += 32) {
        const int c = g * gs + i;
        float y = p[i] * inv * load_w(w, w_bf16, c);
        if (gate_mode == 2) y *= rn_sigmoid(gr[c]);
        if (res) { y += res[c]; res[c] = y; }
        if (o) o[c] = from_f32<TO>(y);
      }
    }
  } else if (nwarp % groups == 0) {
    // several warps per part: every warp sums its slice, the slices of a part meet in shared memory in a fixed order
    const int wpg = nwarp / groups, g = warp / wpg, slice = warp - g * wpg;
    const float* p = rn_stash + (size_t)g * gs;
    float ss = 0.f;
    for (int i = slice * 32 + lane; i < gs; i += wpg * 32) ss += p[i] * p[i];
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int j = 0; j < wpg; ++j) tot += red[g * wpg + j];
    const float inv = 1.0f / sqrtf(tot / (float)gs + eps);
    for (int i = slice * 32 + lane; i < gs; i += wpg * 32) {
      const int c = g * gs + i;
      float y = p[i] * inv * load_w(w, w_bf16, c);
      if (gate_mode == 2) y *= rn_sigmoid(gr[c]);
      if (res) { y += res[c]; res[c] = y; }
      if (o) o[c] = from_f32<TO>(y);
    }
  } else {
    for (int g = 0; g < groups; ++g) {
      const float* p = rn_stash + (size_t)g * gs;
      float ss = 0.f;
      for (int i = tid; i < gs; i += RN_THREADS) ss += p[i] * p[i];
      ss = block_sum(ss, red);
      const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
      for (int i = tid; i < gs; i += RN_THREADS) {
        const int c = g * gs + i;
        float y = p[i] * inv * load_w(w, w_bf16, c);
        if (gate_mode == 2) y *= rn_sigmoid(gr[c]);
        if (res) { y += res[c]; res[c] = y; }
        if (o) o[c] = from_f32<TO>(y);
      }
    }
  }
}

// x [T][H] of x_dtype with row stride x_stride (elements); null with a residual: the stream's rows are only copied out.
// gate: float [T][H] with row stride gate_stride, needed when gate_mode is 1 or 2.  residual: float [T][H] contiguous
// or null.  w [H] of w_dtype.  out [T][H] of out_dtype with row stride out_stride, may be null when a residual is given.
// x_bias [H] of xb_dtype (may be null): added to every row of x first (the bias of the product that made x).
PHOTON_API int photon_group_rmsnorm(const void* x, long x_stride, int x_dtype, const float* gate, long gate_stride,
                                    int gate_mode, float* residual, const void* w, int w_dtype, void* out, long out_stride,
                                    int out_dtype, int T, int H, int groups, float eps, const void* x_bias, int xb_dtype,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || groups <= 0 || H % groups || gate_mode < 0 || gate_mode > 2) return PHOTON_ERR_ARGUMENT;
  if ((gate_mode != 0) != (gate != nullptr)) return PHOTON_ERR_ARGUMENT;
  if (x == nullptr && residual == nullptr) return PHOTON_ERR_ARGUMENT;
  if (out == nullptr && residual == nullptr) return PHOTON_ERR_ARGUMENT;
  if (x != nullptr && w == nullptr) return PHOTON_ERR_ARGUMENT;
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  const int wb = w_dtype == PHOTON_BF16;
#define RN_GO(TX, TO) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(group_rmsnorm_kernel<TX, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    group_rmsnorm_kernel<TX, TO><<<T, RN_THREADS, smem, stream>>>((const TX*)x, x_stride, gate, gate_stride, gate_mode, residual, \
        w, wb, (TO*)out, out_stride, H, groups, eps, x_bias, xb_dtype == PHOTON_BF16); \
    return launch_status(); } while (0)
  if (x_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) RN_GO(float, float);
  if (x_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) RN_GO(float, bf16);
  if (x_dtype == PHOTON_BF16 && out_dtype == PHOTON_F32) RN_GO(bf16, float);
  if (x_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) RN_GO(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}

// ---------------------------------------------------------------- PolyNorm
template <typename TX, typename TO>
__global__ void __launch_bounds__(RN_THREADS)
polynorm_kernel(const TX* __restrict__ z, long z_stride, const void* __restrict__ coef, int coef_bf16, TO* __restrict__ out,
                long out_stride, int F, float eps) {
  __shared__ float red[32];
  const int tid = threadIdx.x;
  const TX* zr = z + (size_t)blockIdx.x * z_stride;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = tid; i < F; i += RN_THREADS) {
    const float v = to_f32(zr[i]), v2 = v * v, v3 = v2 * v;
    s2 += v2; s4 += v2 * v2; s6 += v3 * v3;
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float a = load_w(coef, coef_bf16, 0) / sqrtf(s2 / (float)F + eps);
  const float b = load_w(coef, coef_bf16, 1) / sqrtf(s4 / (float)F + eps);
  const float c = load_w(coef, coef_bf16, 2) / sqrtf(s6 / (float)F + eps);
  const float e = load_w(coef, coef_bf16, 3);
  TO* o = out + (size_t)blockIdx.x * out_stride;
  for (int i = tid; i < F; i += RN_THREADS) {
    const float v = to_f32(zr[i]), v2 = v * v;
    o[i] = from_f32<TO>(a * v + b * v2 + c * (v2 * v) + e);
  }
}

// z [T][F] of z_dtype (row stride z_stride), coef [4] = (a, b, c, e) of coef_dtype, out [T][F] of out_dtype.
PHOTON_API int photon_polynorm(const void* z, long z_stride, int z_dtype, const void* coef, int coef_dtype, void* out,
                               long out_stride, int out_dtype, int T, int F, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0 || z == nullptr || coef == nullptr || out == nullptr) return PHOTON_ERR_ARGUMENT;
  const int cb = coef_dtype == PHOTON_BF16;
#define PN_GO(TX, TO) do { polynorm_kernel<TX, TO><<<T, RN_THREADS, 0, stream>>>((const TX*)z, z_stride, coef, cb, (TO*)out, out_stride, F, eps); \
                           return launch_status(); } while (0)
  if (z_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) PN_GO(float, float);
  if (z_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) PN_GO(float, bf16);
  if (z_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) PN_GO(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}

// ---------------------------------------------------------------- bounded values
__global__ void softcap_kernel(float* __restrict__ x, long total, float cap) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

PHOTON_API int photon_softcap(float* x, long total, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return PHOTON_ERR_ARGUMENT;
  softcap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, total, cap);
  return launch_status();
}
