// Fused residual blocks of transformer layers: dropout + residual add + LayerNorm in one pass (forward and
// backward), and the backward of a stand-alone dropout.
//
//   forward :  s = residual + dropout(h) ;  y = LayerNorm(s) * gamma + beta
//   backward:  ds = LayerNorm'(dy)  (also the residual's gradient) ;  dh = ds * keep / (1 - p)
//
// Stock PyTorch (and the reference, whose eager layer has separate cnnl calls for every one of these) runs
// native_dropout, add, native_layer_norm forward and layer_norm_backward, add, mul, mul backward: seven
// launches and as many passes over a [tokens, hidden] activation.  Here one warp owns one row: the row is read
// once, kept in registers, and every output is written once.  Rows are processed with 8-byte (4 x 16-bit)
// accesses; one Philox call yields the four uniforms of such a vector, keyed by the vector's position, so the
// mask does not depend on the launch configuration.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"
#include "philox.cuh"

namespace {

template <typename T> struct Cv;
template <> struct Cv<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16(v); }
};
template <> struct Cv<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float v) { return __float2half(v); }
};
template <> struct Cv<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float v) { return v; }
};

__device__ __forceinline__ float ldp(const void* p, int i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

constexpr int MAXV = 12;  // vectors of 4 per lane kept in registers: rows of up to 32 * 4 * 12 = 1536 columns
// The kernels are instantiated for 2, 4, 6, 8 and 12 vectors per lane and the launcher picks the smallest that holds a
// row: with the row of a 768-wide layer in 24 registers instead of 48 three CTAs fit on an SM instead of one
// (the forward kernel ran at 0.19 of the copy bandwidth with 200 registers per thread).

template <typename T>
__device__ __forceinline__ void ld4(const T* p, float (&v)[4]) {
  if (sizeof(T) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = Cv<T>::to(t[k]);
  } else {
    const float4 raw = *reinterpret_cast<const float4*>(p);
    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
  }
}
template <typename T>
__device__ __forceinline__ void st4(T* p, const float (&v)[4]) {
  if (sizeof(T) == 2) {
    uint2 raw;
    T* t = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) t[k] = Cv<T>::from(v[k]);
    *reinterpret_cast<uint2*>(p) = raw;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// mask: one byte per vector of four elements, bit k set when element k is kept
template <typename T, int NV>
__global__ void __launch_bounds__(256)
dropout_add_ln_fwd_kernel(const T* __restrict__ h, const T* __restrict__ res, long long rows, int cols, float p,
                          unsigned long long seed, unsigned long long offset, const void* gamma, const void* beta, int pdt,
                          float eps, T* __restrict__ y, T* __restrict__ s_out, unsigned char* __restrict__ mask,
                          float* __restrict__ mean, float* __restrict__ rstd) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = cols / 4;
  const float keep_scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp; row < rows; row += (long long)gridDim.x * (blockDim.x >> 5)) {
    float s[NV][4];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = j * 32 + lane;
      if (v < nvec) {
        const long long e = row * cols + (long long)v * 4;
        float hv[4], rv[4];
        ld4<T>(h + e, hv);
        ld4<T>(res + e, rv);
        unsigned bits = 0xf;
        if (p > 0.f) {
          const uint4 r = philox4(seed, (unsigned long long)(row * nvec + v), offset);
          bits = (u01(r.x) >= p ? 1u : 0u) | (u01(r.y) >= p ? 2u : 0u) | (u01(r.z) >= p ? 4u : 0u) | (u01(r.w) >= p ? 8u : 0u);
        }
        if (mask) mask[row * nvec + v] = (unsigned char)bits;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // the sum is rounded to the storage type first: the backward recomputes the normalised value from the stored s
          const float t = Cv<T>::to(Cv<T>::from(rv[k] + (((bits >> k) & 1u) ? hv[k] * keep_scale : 0.f)));
          s[j][k] = t;
          sum += t;
        }
        st4<T>(s_out + e, s[j]);
      }
    }
    const float m = warp_sum(sum) / (float)cols;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      if (j * 32 + lane < nvec) {
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float d = s[j][k] - m; sq += d * d; }
      }
    }
    const float r = rsqrtf(warp_sum(sq) / (float)cols + eps);
    if (lane == 0) { mean[row] = m; rstd[row] = r; }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = j * 32 + lane;
      if (v < nvec) {
        float o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = v * 4 + k;
          o[k] = (s[j][k] - m) * r * (gamma ? ldp(gamma, c, pdt) : 1.f) + (beta ? ldp(beta, c, pdt) : 0.f);
        }
        st4<T>(y + row * cols + (long long)v * 4, o);
      }
    }
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(256)
dropout_add_ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ s_in, const unsigned char* __restrict__ mask,
                          long long rows, int cols, float p, const void* gamma, int pdt, const float* __restrict__ mean,
                          const float* __restrict__ rstd, T* __restrict__ ds, T* __restrict__ dh, float* dgamma, float* dbeta) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = cols / 4;
  const float keep_scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  float pg[NV][4], pb[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int k = 0; k < 4; ++k) { pg[j][k] = 0.f; pb[j][k] = 0.f; }
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp; row < rows; row += (long long)gridDim.x * (blockDim.x >> 5)) {
    const float m = mean[row], r = rstd[row];
    float g[NV][4], xh[NV][4];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = j * 32 + lane;
      if (v < nvec) {
        const long long e = row * cols + (long long)v * 4;
        float gy[4], sv[4];
        ld4<T>(dy + e, gy);
        ld4<T>(s_in + e, sv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float x = (sv[k] - m) * r;
          const float gg = gy[k] * (gamma ? ldp(gamma, v * 4 + k, pdt) : 1.f);
          xh[j][k] = x; g[j][k] = gg;
          s1 += gg; s2 += gg * x;
          pg[j][k] += gy[k] * x;
          pb[j][k] += gy[k];
        }
      }
    }
    s1 = warp_sum(s1) / (float)cols;
    s2 = warp_sum(s2) / (float)cols;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = j * 32 + lane;
      if (v < nvec) {
        const long long e = row * cols + (long long)v * 4;
        float d[4], dd[4];
        const unsigned bits = mask ? mask[row * nvec + v] : 0xfu;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          d[k] = r * (g[j][k] - s1 - xh[j][k] * s2);
          dd[k] = ((bits >> k) & 1u) ? d[k] * keep_scale : 0.f;
        }
        st4<T>(ds + e, d);
        st4<T>(dh + e, dd);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = j * 32 + lane;
    if (v < nvec) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (dgamma) atomicAdd(&dgamma[v * 4 + k], pg[j][k]);
        if (dbeta) atomicAdd(&dbeta[v * 4 + k], pb[j][k]);
      }
    }
  }
}

// dx = dy * mask * scale  (mask: one byte per element, as written by the dropout forward kernel)
template <typename T>
__global__ void dropout_bwd_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ mask, long long n, float scale,
                                   T* __restrict__ dx) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dx[i] = Cv<T>::from(mask[i] ? Cv<T>::to(dy[i]) * scale : 0.f);
}

}  // namespace

#define DISPATCH16(dt, T, ...)                                       \
  switch (dt) {                                                      \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }         \
    case B200_F32: { using T = float; __VA_ARGS__; break; }          \
    default: return (int)cudaErrorInvalidValue;                      \
  }

extern "C" int b200_dropout_add_layernorm_max_cols(void) { return 32 * 4 * MAXV; }

extern "C" int b200_dropout_add_layernorm_fwd(const void* h, const void* residual, int dtype, long long rows, int cols, float p,
                                              unsigned long long seed, unsigned long long offset, const void* gamma,
                                              const void* beta, int param_dtype, float eps, void* y, void* s_out,
                                              unsigned char* mask, float* mean, float* rstd, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 4 || cols > 32 * 4 * MAXV) return (int)cudaErrorInvalidValue;
  const int warps = 8;
  long long grid = (rows + warps - 1) / warps;
  if (grid > 148 * 8) grid = 148 * 8;
  const int per_lane = (cols / 4 + 31) / 32;
#define LN_FWD(NV)                                                                                                     \
  DISPATCH16(dtype, T, (dropout_add_ln_fwd_kernel<T, NV><<<(unsigned)grid, warps * 32, 0, (cudaStream_t)stream>>>(     \
                           static_cast<const T*>(h), static_cast<const T*>(residual), rows, cols, p, seed, offset, gamma, beta, \
                           param_dtype, eps, static_cast<T*>(y), static_cast<T*>(s_out), mask, mean, rstd)))
  if (per_lane <= 2) { LN_FWD(2); }
  else if (per_lane <= 4) { LN_FWD(4); }
  else if (per_lane <= 6) { LN_FWD(6); }
  else if (per_lane <= 8) { LN_FWD(8); }
  else { LN_FWD(12); }
#undef LN_FWD
  return (int)cudaGetLastError();
}

extern "C" int b200_dropout_add_layernorm_bwd(const void* dy, const void* s, const unsigned char* mask, int dtype, long long rows,
                                              int cols, float p, const void* gamma, int param_dtype, const float* mean,
                                              const float* rstd, void* ds, void* dh, float* dgamma, float* dbeta, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 4 || cols > 32 * 4 * MAXV) return (int)cudaErrorInvalidValue;
  const int warps = 8;
  long long grid = (rows + warps - 1) / warps;
  if (grid > 148 * 2) grid = 148 * 2;  // fewer, longer-lived warps: fewer atomics for the parameter gradients
  const int per_lane = (cols / 4 + 31) / 32;
#define LN_BWD(NV)                                                                                                     \
  DISPATCH16(dtype, T, (dropout_add_ln_bwd_kernel<T, NV><<<(unsigned)grid, warps * 32, 0, (cudaStream_t)stream>>>(     \
                           static_cast<const T*>(dy), static_cast<const T*>(s), mask, rows, cols, p, gamma, param_dtype, mean, \
                           rstd, static_cast<T*>(ds), static_cast<T*>(dh), dgamma, dbeta)))
  if (per_lane <= 2) { LN_BWD(2); }
  else if (per_lane <= 4) { LN_BWD(4); }
  else if (per_lane <= 6) { LN_BWD(6); }
  else if (per_lane <= 8) { LN_BWD(8); }
  else { LN_BWD(12); }
#undef LN_BWD
  return (int)cudaGetLastError();
}

extern "C" int b200_dropout_bwd(const void* dy, const unsigned char* mask, int dtype, long long n, float scale, void* dx,
                                void* stream) {
  if (n <= 0) return 0;
  long long grid = (n + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  DISPATCH16(dtype, T, (dropout_bwd_kernel<T><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(
                           static_cast<const T*>(dy), mask, n, scale, static_cast<T*>(dx))));
  return (int)cudaGetLastError();
}
