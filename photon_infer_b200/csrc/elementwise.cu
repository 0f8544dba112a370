// Row-wise kernels of the decoder: embedding lookup, residual add fused with RMSNorm
// (on all rows or on a list of rows), SwiGLU.  All arithmetic is 32-bit; storage is
// float or bfloat16.  Formulas: include/photon/ops/kernels/rmsnorm_kernel.hpp:71-86
// (w * (x * 1/sqrt(mean(x^2)+eps))), include/photon/ops/kernels/swiglu_kernel.hpp:67-76
// (g / (1 + exp(-g)) * u), include/photon/ops/kernels/embedding_kernel.hpp:85-121.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int H, int V, int* err) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) report_error(err, PHOTON_DEV_BAD_TOKEN, t, id, V);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

PHOTON_API int photon_embedding(const int* ids, const void* table, int table_dtype, float* out,
                                int T, int H, int V, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == PHOTON_BF16)
    embedding_kernel<bf16><<<T, threads, 0, stream>>>(ids, (const bf16*)table, out, H, V, err);
  else
    embedding_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, H, V, err);
  return launch_status();
}

// ---------------------------------------------------------------- add + RMSNorm
// residual (float, in place) += delta; out = w * (residual * r).  rows == nullptr: row = blockIdx.x
// of both residual and out.  rows != nullptr: reads row rows[blockIdx.x] and does NOT write the sum
// back (the listed rows are only read; out has one row per list entry).
template <typename T> struct Quad;            // four consecutive elements as one load or store
template <> struct Quad<float> {
  __device__ static void load(const float* p, float* f) { const float4 r = *reinterpret_cast<const float4*>(p); f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Quad<bf16> {
  __device__ static void load(const bf16* p, float* f) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  __device__ static void store(bf16* p, const float* f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&a);
    r.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

// VEC: rows are read and written four elements at a time (H a multiple of 4, aligned pointers).
// CENTER: layer norm, (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b; the row's mean is taken first and the
// squared deviations are summed in a second pass over the row held in shared memory.
template <typename TD, typename TO, bool VEC, bool CENTER = false>
__global__ void add_rmsnorm_kernel(const TD* delta, const TD* delta2, float* residual,   // written by earlier kernels that
                                   const void* __restrict__ w, int w_bf16,    // may still run when this one starts: no
                                   TO* out, const int* rows, int H, float eps,   // read-only path for them
                                   const void* __restrict__ b = nullptr, int b_bf16 = 0,
                                   const float* __restrict__ dscale = nullptr) {   // [H]: delta is multiplied by it first
  __shared__ float red[32];
  extern __shared__ __align__(16) float stash[];               // H floats: the summed row
  pdl_wait();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* res = residual + (size_t)r * H;
  const TD* d = delta ? delta + (size_t)r * H : nullptr;
  const TD* d2 = (delta && delta2) ? delta2 + (size_t)r * H : nullptr;   // a second sublayer's output (parallel blocks)
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4], dv[4];
      Quad<float>::load(res + i, v);
      if (d) {
        Quad<TD>::load(d + i, dv);
        if (dscale) {
          float sc[4];
          Quad<float>::load(dscale + i, sc);
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] *= sc[e];
        }
        if (d2) {
          float dw[4];
          Quad<TD>::load(d2 + i, dw);
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] += dw[e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += dv[e];
      }
      Quad<float>::store(stash + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = res[i];
      if (d) {
        const float d1 = dscale ? to_f32(d[i]) * dscale[i] : to_f32(d[i]);
        v += d2 ? d1 + to_f32(d2[i]) : d1;
      }
      stash[i] = v;
      ss += v * v;
    }
  }
  float mean = 0.f;
  if (CENTER) {
    float sm = 0.f;
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x) sm += stash[i];
    mean = block_sum(sm, red) / (float)H;
    ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { const float c = stash[i] - mean; ss += c * c; }
  }
  ss = block_sum(ss, red);
  pdl_launch_dependents();                         // the next kernel may be scheduled while the row is written
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)blockIdx.x * H;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float v[4], wv[4], y[4];
      Quad<float>::load(stash + i, v);
      if (w_bf16) Quad<bf16>::load((const bf16*)w + i, wv); else Quad<float>::load((const float*)w + i, wv);
      if (d && !rows) Quad<float>::store(res + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = CENTER ? (v[e] - mean) * inv * wv[e] + (b ? load_w(b, b_bf16, i + e) : 0.f) : wv[e] * (v[e] * inv);
      Quad<TO>::store(o + i, y);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = stash[i];
      if (d && !rows) res[i] = v;
      o[i] = from_f32<TO>(CENTER ? (v - mean) * inv * load_w(w, w_bf16, i) + (b ? load_w(b, b_bf16, i) : 0.f)
                                 : load_w(w, w_bf16, i) * (v * inv));
    }
  }
}

template <typename TD, typename TO, bool CENTER = false>
static int add_rmsnorm_launch(const void* delta, const void* delta2, float* residual, const void* w, int w_bf16, void* out,
                              const int* rows, int n, int H, float eps, cudaStream_t stream,
                              const void* b = nullptr, int b_bf16 = 0, const float* dscale = nullptr) {
  const size_t smem = (size_t)H * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  const bool vec = (H % 4 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)delta2 % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                   ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)dscale % 16 == 0);
  if (smem > 48 * 1024) {
    cudaError_t e = vec ? cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, true, CENTER>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false, CENTER>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = 128;
  while (threads < 1024 && threads * 4 < H) threads <<= 1;   // depends on H only
  if (vec)
    return launch_pdl(add_rmsnorm_kernel<TD, TO, true, CENTER>, dim3(n), dim3(threads), smem, stream, (const TD*)delta,
                      (const TD*)delta2, residual, w, w_bf16, (TO*)out, rows, H, eps, b, b_bf16, dscale);
  return launch_pdl(add_rmsnorm_kernel<TD, TO, false, CENTER>, dim3(n), dim3(threads), smem, stream, (const TD*)delta,
                    (const TD*)delta2, residual, w, w_bf16, (TO*)out, rows, H, eps, b, b_bf16, dscale);
}

// delta may be null (plain norm); delta2 (same type as delta, may be null) is added as well: the sum of the two is
// formed first, in 32-bit, and then added to the residual.  delta_dtype / out_dtype: PHOTON_F32 or PHOTON_BF16.
// delta_scale (float [H], may be null): delta is multiplied by it, channel by channel, before the sums.
PHOTON_API int photon_add_rmsnorm_scaled(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                                  int w_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                                  float eps, const float* delta_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int wb = (w_dtype == PHOTON_BF16);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<bf16, bf16>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, nullptr, 0, delta_scale);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<float, float>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, nullptr, 0, delta_scale);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<float, bf16>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, nullptr, 0, delta_scale);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<bf16, float>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, nullptr, 0, delta_scale);
  return PHOTON_ERR_ARGUMENT;
}

PHOTON_API int photon_add_rmsnorm(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                                  int w_dtype, void* out, int out_dtype, const int* rows, int n, int H,
                                  float eps, cudaStream_t stream) {
  return photon_add_rmsnorm_scaled(delta, delta_dtype, delta2, residual, w, w_dtype, out, out_dtype, rows, n, H, eps, nullptr, stream);
}

// The same with a layer norm: out = (x - mean(x)) / sqrt(var(x) + eps) * w + b, x = residual + delta (+ delta2).
// b may be null.
PHOTON_API int photon_add_layernorm_scaled(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                                    int w_dtype, const void* b, int b_dtype, void* out, int out_dtype, const int* rows,
                                    int n, int H, float eps, const float* delta_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int wb = (w_dtype == PHOTON_BF16), bb = (b_dtype == PHOTON_BF16);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<bf16, bf16, true>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, b, bb, delta_scale);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<float, float, true>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, b, bb, delta_scale);
  if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16)
    return add_rmsnorm_launch<float, bf16, true>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, b, bb, delta_scale);
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_F32)
    return add_rmsnorm_launch<bf16, float, true>(delta, delta2, residual, w, wb, out, rows, n, H, eps, stream, b, bb, delta_scale);
  return PHOTON_ERR_ARGUMENT;
}

PHOTON_API int photon_add_layernorm(const void* delta, int delta_dtype, const void* delta2, float* residual, const void* w,
                                    int w_dtype, const void* b, int b_dtype, void* out, int out_dtype, const int* rows,
                                    int n, int H, float eps, cudaStream_t stream) {
  return photon_add_layernorm_scaled(delta, delta_dtype, delta2, residual, w, w_dtype, b, b_dtype, out, out_dtype, rows, n, H, eps,
                                     nullptr, stream);
}

// ---------------------------------------------------------------- gated activation (SwiGLU, GeGLU)
// gate_up [T, 2*I]: columns [0, I) are the gate, [I, 2I) the up projection.  out [T, I] = act(gate) * up.
// act 0: silu, g / (1 + exp(-g)); act 1: the tanh form of gelu, 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).
__device__ __forceinline__ float glu_act(float g, int act) {
  if (act == PHOTON_ACT_RELU) return fmaxf(g, 0.f);
  if (act == PHOTON_ACT_GELU) return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));
  if (act == PHOTON_ACT_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.0f + expf(-g));
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total, int act) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_f32(gate_up[t * 2 * I + i]);
    const float u = to_f32(gate_up[t * 2 * I + I + i]);
    out[idx] = from_f32<T>(glu_act(g, act) * u);
  }
}

// The same, 16 bytes per load: I a multiple of the elements in 16 bytes, aligned pointers.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total_vecs, int act) {
  constexpr int N = 16 / sizeof(T);
  const int per_row = I / N;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vecs; idx += stride) {
    const size_t t = idx / per_row;
    const int i = (int)(idx - t * per_row) * N;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + t * 2 * I + i);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + t * 2 * I + I + i);
    const T* gp = reinterpret_cast<const T*>(&gv);
    const T* up = reinterpret_cast<const T*>(&uv);
    uint4 ov;
    T* op = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float g = to_f32(gp[e]);
      op[e] = from_f32<T>(glu_act(g, act) * to_f32(up[e]));
    }
    *reinterpret_cast<uint4*>(out + t * I + i) = ov;
  }
}

PHOTON_API int photon_glu(const void* gate_up, void* out, int dtype, int T, int I, int act, cudaStream_t stream) {
  if (act != PHOTON_ACT_SILU && act != PHOTON_ACT_GELU_TANH && act != PHOTON_ACT_GELU && act != PHOTON_ACT_RELU) return PHOTON_ERR_ARGUMENT;
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  const int n = dtype == PHOTON_BF16 ? 8 : 4;
  const bool vec = (I % n == 0) && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const size_t work = vec ? total / n : total;
  size_t blocks = (work + threads - 1) / threads;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (dtype == PHOTON_BF16) {
    if (vec) swiglu_vec_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, work, act);
    else swiglu_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, total, act);
  } else {
    if (vec) swiglu_vec_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, work, act);
    else swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total, act);
  }
  return launch_status();
}

PHOTON_API int photon_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
  return photon_glu(gate_up, out, dtype, T, I, PHOTON_ACT_SILU, stream);
}

// ---------------------------------------------------------------- the stream joined with a second one
// out [T, 2H] (TO) = [residual + delta + delta2 ; other]: the input of a product that mixes the running stream
// with another stream of the same width (the embedding output, for a block of layers that is entered again).
// delta and delta2 may be null.  The sum is formed in 32-bit and rounded once.
template <typename TD, typename TO>
__global__ void stream_concat_kernel(const float* residual, const TD* delta, const TD* delta2, const float* other,
                                     TO* out, int H) {
  const size_t r = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = residual[r * H + i];
    if (delta) v += delta2 ? to_f32(delta[r * H + i]) + to_f32(delta2[r * H + i]) : to_f32(delta[r * H + i]);
    out[r * 2 * H + i] = from_f32<TO>(v);
    out[r * 2 * H + H + i] = from_f32<TO>(other[r * H + i]);
  }
}

PHOTON_API int photon_stream_concat(const float* residual, const void* delta, const void* delta2, int delta_dtype,
                                    const float* other, void* out, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (delta_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16)
    stream_concat_kernel<bf16, bf16><<<T, threads, 0, stream>>>(residual, (const bf16*)delta, (const bf16*)delta2, other, (bf16*)out, H);
  else if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_F32)
    stream_concat_kernel<float, float><<<T, threads, 0, stream>>>(residual, (const float*)delta, (const float*)delta2, other, (float*)out, H);
  else if (delta_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16)
    stream_concat_kernel<float, bf16><<<T, threads, 0, stream>>>(residual, (const float*)delta, (const float*)delta2, other, (bf16*)out, H);
  else
    return PHOTON_ERR_ARGUMENT;
  return launch_status();
}

// x [T, H] (float, in place) = x * scale + bias (bias [H] may be null; stored as float or bfloat16).
__global__ void scale_bias_rows_kernel(float* x, float scale, const void* bias, int bias_bf16, int H, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    float v = x[idx] * scale;
    if (bias) v += load_w(bias, bias_bf16, idx % H);
    x[idx] = v;
  }
}

PHOTON_API int photon_scale_bias_rows(float* x, float scale, const void* bias, int bias_dtype, int T, int H,
                                      cudaStream_t stream) {
  const size_t total = (size_t)T * H;
  if (total == 0) return 0;
  size_t blocks = (total + 255) / 256;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  scale_bias_rows_kernel<<<(int)blocks, 256, 0, stream>>>(x, scale, bias, bias_dtype == PHOTON_BF16, H, total);
  return launch_status();
}

// ---------------------------------------------------------------- plain activation, gate, stream sums
// out[i] = act(x[i]) over `total` elements of one dtype (x and out may be the same buffer); 32-bit arithmetic.
template <typename T>
__global__ void activation_kernel(const T* x, T* out, size_t total, int act) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) out[idx] = from_f32<T>(glu_act(to_f32(x[idx]), act));
}

// The same, 16 bytes per load and store: total a multiple of the elements in 16 bytes, aligned pointers.
template <typename T>
__global__ void activation_vec_kernel(const T* x, T* out, size_t total_vecs, int act) {
  constexpr int N = 16 / sizeof(T);
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_vecs; idx += stride) {
    const uint4 v = reinterpret_cast<const uint4*>(x)[idx];
    const T* p = reinterpret_cast<const T*>(&v);
    uint4 o;
    T* q = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < N; ++e) q[e] = from_f32<T>(glu_act(to_f32(p[e]), act));
    reinterpret_cast<uint4*>(out)[idx] = o;
  }
}

PHOTON_API int photon_activation(const void* x, void* out, int dtype, long total, int act, cudaStream_t stream) {
  if (act != PHOTON_ACT_SILU && act != PHOTON_ACT_GELU_TANH && act != PHOTON_ACT_GELU && act != PHOTON_ACT_RELU) return PHOTON_ERR_ARGUMENT;
  if (total <= 0) return 0;
  const int n = dtype == PHOTON_BF16 ? 8 : 4;
  const bool vec = (total % n == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const size_t work = vec ? (size_t)total / n : (size_t)total;
  size_t blocks = (work + 255) / 256;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (vec) {
    if (dtype == PHOTON_BF16) activation_vec_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((const bf16*)x, (bf16*)out, work, act);
    else activation_vec_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (float*)out, work, act);
    return launch_status();
  }
  if (dtype == PHOTON_BF16) activation_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((const bf16*)x, (bf16*)out, (size_t)total, act);
  else activation_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)x, (float*)out, (size_t)total, act);
  return launch_status();
}

// x [T, W] (row stride ldx, in place) *= sigmoid(g [T, W]) (row stride ldg; its own type): the gate of a mixer's
// output.  The sigmoid and the product are 32-bit, the result is rounded once.
template <typename TX, typename TG>
__global__ void gate_mul_kernel(TX* x, long ldx, const TG* g, long ldg, int W, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const size_t t = idx / W;
    const int i = (int)(idx - t * W);
    const float z = to_f32(g[t * ldg + i]);
    x[t * ldx + i] = from_f32<TX>(to_f32(x[t * ldx + i]) / (1.0f + expf(-z)));
  }
}

// Four elements per thread and step: W and both row strides multiples of 4, 16-byte aligned pointers (8-byte for
// bfloat16 rows).
template <typename TX, typename TG>
__global__ void gate_mul_vec_kernel(TX* x, long ldx, const TG* g, long ldg, int W, size_t total_quads) {
  const int per_row = W / 4;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total_quads; idx += stride) {
    const size_t t = idx / per_row;
    const int i = (int)(idx - t * per_row) * 4;
    float xv[4], gv[4];
    Quad<TX>::load(x + t * ldx + i, xv);
    Quad<TG>::load(g + t * ldg + i, gv);
#pragma unroll
    for (int e = 0; e < 4; ++e) xv[e] = xv[e] / (1.0f + expf(-gv[e]));
    Quad<TX>::store(x + t * ldx + i, xv);
  }
}

PHOTON_API int photon_gate_mul(void* x, long ldx, int x_dtype, const void* g, long ldg, int g_dtype, int T, int W,
                               cudaStream_t stream) {
  const size_t total = (size_t)T * W;
  if (total == 0) return 0;
  const bool vec = (W % 4 == 0) && (ldx % 4 == 0) && (ldg % 4 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)g % 16 == 0);
  size_t blocks = ((vec ? total / 4 : total) + 255) / 256;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (vec) {
    if (x_dtype == PHOTON_BF16 && g_dtype == PHOTON_BF16) gate_mul_vec_kernel<bf16, bf16><<<(int)blocks, 256, 0, stream>>>((bf16*)x, ldx, (const bf16*)g, ldg, W, total / 4);
    else if (x_dtype == PHOTON_BF16 && g_dtype == PHOTON_F32) gate_mul_vec_kernel<bf16, float><<<(int)blocks, 256, 0, stream>>>((bf16*)x, ldx, (const float*)g, ldg, W, total / 4);
    else if (x_dtype == PHOTON_F32 && g_dtype == PHOTON_F32) gate_mul_vec_kernel<float, float><<<(int)blocks, 256, 0, stream>>>((float*)x, ldx, (const float*)g, ldg, W, total / 4);
    else return PHOTON_ERR_ARGUMENT;
    return launch_status();
  }
  if (x_dtype == PHOTON_BF16 && g_dtype == PHOTON_BF16) gate_mul_kernel<bf16, bf16><<<(int)blocks, 256, 0, stream>>>((bf16*)x, ldx, (const bf16*)g, ldg, W, total);
  else if (x_dtype == PHOTON_BF16 && g_dtype == PHOTON_F32) gate_mul_kernel<bf16, float><<<(int)blocks, 256, 0, stream>>>((bf16*)x, ldx, (const float*)g, ldg, W, total);
  else if (x_dtype == PHOTON_F32 && g_dtype == PHOTON_F32) gate_mul_kernel<float, float><<<(int)blocks, 256, 0, stream>>>((float*)x, ldx, (const float*)g, ldg, W, total);
  else return PHOTON_ERR_ARGUMENT;
  return launch_status();
}

// residual [T, H] (float, in place) += (delta + delta2) + other + bias: what is pending on the stream, a second
// stream of the same width (may be null) and one vector for all rows (may be null), each term added in 32-bit in
// this order.
template <typename TD>
__global__ void stream_add_kernel(float* residual, const TD* delta, const TD* delta2, const float* other,
                                  const void* bias, int bias_bf16, int H, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    float v = residual[idx];
    if (delta) v += delta2 ? to_f32(delta[idx]) + to_f32(delta2[idx]) : to_f32(delta[idx]);
    if (other) v += other[idx];
    if (bias) v += load_w(bias, bias_bf16, idx % H);
    residual[idx] = v;
  }
}

PHOTON_API int photon_stream_add(float* residual, const void* delta, const void* delta2, int delta_dtype, const float* other,
                                 const void* bias, int bias_dtype, int T, int H, cudaStream_t stream) {
  const size_t total = (size_t)T * H;
  if (total == 0) return 0;
  size_t blocks = (total + 255) / 256;
  const size_t cap = (size_t)photon_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (delta_dtype == PHOTON_BF16)
    stream_add_kernel<bf16><<<(int)blocks, 256, 0, stream>>>(residual, (const bf16*)delta, (const bf16*)delta2, other, bias, bias_dtype == PHOTON_BF16, H, total);
  else
    stream_add_kernel<float><<<(int)blocks, 256, 0, stream>>>(residual, (const float*)delta, (const float*)delta2, other, bias, bias_dtype == PHOTON_BF16, H, total);
  return launch_status();
}
