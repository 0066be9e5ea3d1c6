// Batch normalisation (statistics, apply, backward) and layer normalisation
// kernels for channels-innermost data.
//
// Replaces cnnlBatchNormForwardTraining / ForwardInference / Backward /
// FrozenBatchNormBackward (torch_mlu/csrc/aten/operators/cnnl/internal/
// native_batch_norm_internal.cpp:119,137, native_batch_norm_backward_internal.cpp:122,147).
// LayerNorm has no device kernel in the reference.
//
// Column reductions: a CTA owns a slab of rows; thread (tx, ty) accumulates the
// 8-channel vector tx over rows ty, ty+RY, ...; the RY partial vectors are folded
// in shared memory and added to the fp64 totals with one atomic per channel.
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

template <typename T> struct Cv;
template <> struct Cv<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float v) { return v; }
};
template <> struct Cv<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16(v); }
};
template <> struct Cv<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float v) { return __float2half(v); }
};

__device__ __forceinline__ float ldf(const void* p, long long i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == B200_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return (float)static_cast<const double*>(p)[i];
}
__device__ __forceinline__ void stf(void* p, long long i, int dt, float v) {
  if (dt == B200_F32) static_cast<float*>(p)[i] = v;
  else if (dt == B200_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else if (dt == B200_F16) static_cast<__half*>(p)[i] = __float2half(v);
  else static_cast<double*>(p)[i] = v;
}

// VEC elements of type T per 16 bytes (fp32: 4, 16-bit: 8)
template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f) {
  constexpr int V = VecOf<T>::N;
  alignas(16) T t[V];
  *reinterpret_cast<uint4*>(t) = *reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) f[i] = Cv<T>::to(t[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* f) {
  constexpr int V = VecOf<T>::N;
  alignas(16) T t[V];
#pragma unroll
  for (int i = 0; i < V; ++i) t[i] = Cv<T>::from(f[i]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(t);
}

constexpr int RED_THREADS = 256;

// Generic two-quantity column reduction.  F(row, c_vec_start, out_a[V], out_b[V]).
template <typename T, int NQ, typename F, typename P, typename M>
__device__ void column_reduce(long long rows, int C, double* sums, F f, P prep, M fin) {
  constexpr int V = VecOf<T>::N;
  const int cvecs = C / V;                   // C % V == 0 guaranteed by the launcher
  const int tx_n = cvecs < RED_THREADS ? cvecs : RED_THREADS;
  const int ty_n = RED_THREADS / tx_n;
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  extern __shared__ float sh[];              // [ty_n][tx_n*V*NQ]
  const long long rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  // every thread runs the same number of trips (the loop body contains barriers); `on` guards the work
  for (int cv0 = 0; cv0 < cvecs; cv0 += tx_n) {
    const int cv = cv0 + tx;
    const bool on = ty < ty_n && cv < cvecs;
    float acc[NQ][V];
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int i = 0; i < V; ++i) acc[q][i] = 0.f;
    float ctx[V];
    if (on) {
      prep(cv * V, ctx);  // per-column constants, loaded once instead of once per row
#pragma unroll 4
      for (long long r = r0 + ty; r < r1; r += ty_n) f(r, cv * V, acc, ctx);
    }
    // fold the ty_n partials
    float* mine = sh + ((size_t)ty * tx_n + tx) * V * NQ;
    if (ty < ty_n) {
#pragma unroll
      for (int q = 0; q < NQ; ++q)
#pragma unroll
        for (int i = 0; i < V; ++i) mine[q * V + i] = acc[q][i];
    }
    __syncthreads();
    if (ty == 0 && cv < cvecs) {
#pragma unroll
      for (int q = 0; q < NQ; ++q)
#pragma unroll
        for (int i = 0; i < V; ++i) {
          double s = 0.0;
          for (int y = 0; y < ty_n; ++y) s += sh[((size_t)y * tx_n + tx) * V * NQ + q * V + i];
          atomicAdd(&sums[(size_t)q * C + cv * V + i], s * (double)fin(q, cv * V + i));
        }
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(RED_THREADS) bn_stats_kernel(const T* x, long long rows, int C, double* sums) {
  constexpr int V = VecOf<T>::N;
  column_reduce<T, 2>(
      rows, C, sums,
      [&](long long r, int c0, float (*acc)[V], const float*) {
        float v[V];
        load_vec<T>(x + r * C + c0, v);
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[0][i] += v[i]; acc[1][i] += v[i] * v[i]; }
      },
      [](int, float*) {}, [](int, int) { return 1.f; });
}

__global__ void bn_finalize_kernel(const double* sums, long long rows, int C, float eps, float momentum, float* mean,
                                   float* invstd, void* rmean, void* rvar, int rdt) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const double m = sums[c] / (double)rows;
  double var = sums[C + c] / (double)rows - m * m;
  if (var < 0) var = 0;
  mean[c] = (float)m;
  invstd[c] = (float)(1.0 / sqrt(var + (double)eps));
  if (rmean) {
    const double unbiased = rows > 1 ? var * (double)rows / (double)(rows - 1) : var;
    stf(rmean, c, rdt, (float)((1.0 - momentum) * ldf(rmean, c, rdt) + momentum * m));
    stf(rvar, c, rdt, (float)((1.0 - momentum) * ldf(rvar, c, rdt) + momentum * unbiased));
  }
}

__global__ void bn_invstd_kernel(const void* var, int dt, int C, float eps, float* invstd) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) invstd[c] = rsqrtf(ldf(var, c, dt) + eps);
}

template <typename TX, typename TY>
__global__ void __launch_bounds__(256) bn_apply_kernel(const TX* x, TY* y, long long nvec, int C, const void* mean,
                                                       int mdt, const float* invstd, const void* gamma,
                                                       const void* beta, int pdt, const void* res, int rdt, int act) {
  constexpr int V = VecOf<TX>::N > VecOf<TY>::N ? VecOf<TY>::N : VecOf<TX>::N;  // elements per thread-iteration
  const int cvecs = C / V;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % cvecs) * V;
    float v[V], rv[V], o[V];
    constexpr bool kSame = sizeof(TX) == sizeof(TY);
    if constexpr (kSame) {
      load_vec<TX>(x + i * V, v);
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) v[k] = Cv<TX>::to(x[i * V + k]);
    }
    if (res) {
      if (kSame && rdt == (sizeof(TX) == 4 ? B200_F32 : (int)B200_BF16) && sizeof(TX) == 2) {
        load_vec<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(res) + i * V, rv);
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) rv[k] = ldf(res, i * V + k, rdt);
      }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int c = c0 + k;
      const float g = gamma ? ldf(gamma, c, pdt) : 1.f;
      const float b = beta ? ldf(beta, c, pdt) : 0.f;
      float t = (v[k] - ldf(mean, c, mdt)) * invstd[c] * g + b;
      if (res) t += rv[k];
      if (act == 1) t = t > 0.f ? t : 0.f;
      o[k] = t;
    }
    if constexpr (kSame) {
      store_vec<TY>(y + i * V, o);
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) y[i * V + k] = Cv<TY>::from(o[k]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(RED_THREADS)
bn_bwd_reduce_kernel(const T* dy, const T* x, const void* mean, int mdt, const float* invstd, const T* relu_out,
                     const uint8_t* relu_mask, long long rows, int C, double* sums) {
  constexpr int V = VecOf<T>::N;
  // accumulates sum(dy) and sum(dy * (x - mean)); the second is scaled by invstd when folded
  column_reduce<T, 2>(
      rows, C, sums,
      [&](long long r, int c0, float (*acc)[V], const float* mu) {
        float g[V], v[V], o[V];
        load_vec<T>(dy + r * C + c0, g);
        load_vec<T>(x + r * C + c0, v);
        if (relu_out) load_vec<T>(relu_out + r * C + c0, o);
        const unsigned bits = relu_mask ? relu_mask[(r * C + c0) / V] : 0xffu;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float gi = g[i];
          if (relu_out && !(o[i] > 0.f)) gi = 0.f;
          if (!((bits >> i) & 1u)) gi = 0.f;
          acc[0][i] += gi;
          acc[1][i] += gi * (v[i] - mu[i]);
        }
      },
      [&](int c0, float* mu) {
#pragma unroll
        for (int i = 0; i < V; ++i) mu[i] = ldf(mean, c0 + i, mdt);
      },
      [&](int q, int c) { return q == 1 ? invstd[c] : 1.f; });
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const T* dy, const T* x, const void* mean, int mdt, const float* invstd, const void* gamma, int pdt,
                    const T* relu_out, const double* sums, long long rows, int C, int training, TO* dx, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    float g = Cv<T>::to(dy[i]);
    if (relu_out && !(Cv<T>::to(relu_out[i]) > 0.f)) g = 0.f;
    const float is = invstd[c];
    const float ga = gamma ? ldf(gamma, c, pdt) : 1.f;
    float o;
    if (training) {
      const float xh = (Cv<T>::to(x[i]) - ldf(mean, c, mdt)) * is;
      const float sdy = (float)(sums[c] / (double)rows), sdx = (float)(sums[C + c] / (double)rows);
      o = ga * is * (g - sdy - xh * sdx);
    } else {
      o = ga * is * g;
    }
    dx[i] = Cv<TO>::from(o);
  }
}

__global__ void bn_param_grads_kernel(const double* sums, int C, float* dgamma, float* dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  if (dbeta) dbeta[c] = (float)sums[c];
  if (dgamma) dgamma[c] = (float)sums[C + c];
}


// ---- fast paths ---------------------------------------------------------------------------
// Streaming kernels over a [rows][C] activation with 16-byte vectors.  What keeps them at the memory
// system's speed rather than at a fraction of it:
//  * U vectors per thread are loaded before any of them is used, so every thread has U (x number of
//    input tensors) 16-byte loads in flight;
//  * the grid stride is a multiple of the number of channel vectors whenever that number divides the CTA
//    size, so a thread meets the same channels in every iteration and keeps their coefficients in
//    registers (no index division, no shared-memory reads in the loop);
//  * small per-channel kernels are folded in: the forward kernel turns the channel sums into mean / inverse
//    standard deviation itself (CTA 0 stores them and updates the running statistics), the backward kernel
//    writes the parameter gradients and clears the sums for the next call.
constexpr int BN_U = 4;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float* f) {
  constexpr int V = VecOf<T>::N;
  const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < V; ++i) f[i] = Cv<T>::to(t[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack_vec(const float* f) {
  constexpr int V = VecOf<T>::N;
  uint4 raw;
  T* t = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < V; ++i) t[i] = Cv<T>::from(f[i]);
  return raw;
}

// Forward statistics of channel c from its sums (fp64, as accumulated by the statistics pass or by the
// producing convolution's epilogue).
__device__ __forceinline__ void bn_moments(const double* sums, int C, int c, long long rows, float eps, float* mean,
                                           float* invstd, double* var_out) {
  const double m = sums[c] / (double)rows;
  double var = sums[C + c] / (double)rows - m * m;
  if (var < 0) var = 0;
  *mean = (float)m;
  *invstd = (float)(1.0 / sqrt(var + (double)eps));
  if (var_out) *var_out = var;
}

struct BnFinalize {          // optional: statistics come from `sums` instead of mean / invstd tensors
  const double* sums;        // [2 * C] sum and sum of squares; nullptr = use the mean / invstd arguments
  long long rows;
  float eps, momentum;
  float* save_mean;          // written by CTA 0
  float* save_invstd;
  void* rmean;               // running statistics, updated by CTA 0 (may be null)
  void* rvar;
  int rdt;
  long long* batch_counter;  // optional: num_batches_tracked, incremented by CTA 0
};

// y = act(x * S[c] + T[c] + residual) with S = invstd * gamma, T = beta - mean * S
template <typename T>
__global__ void __launch_bounds__(256, 3)  // three CTAs per SM: 16 resident warps left the loads short of the copy bandwidth
bn_apply_fast_kernel(const T* __restrict__ x, T* __restrict__ y, unsigned nvec, int C, const void* mean, int mdt,
                     const float* invstd, const void* gamma, const void* beta, int pdt, const T* __restrict__ res,
                     int act, uint8_t* __restrict__ relu_mask, const BnFinalize fz) {
  constexpr int V = VecOf<T>::N;
  extern __shared__ float coef[];
  float* S = coef;
  float* Tc = coef + C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float mu, is;
    if (fz.sums) {
      double var;
      bn_moments(fz.sums, C, c, fz.rows, fz.eps, &mu, &is, &var);
      if (blockIdx.x == 0) {
        fz.save_mean[c] = mu;
        fz.save_invstd[c] = is;
        if (fz.rmean) {
          const double unbiased = fz.rows > 1 ? var * (double)fz.rows / (double)(fz.rows - 1) : var;
          const double m = fz.sums[c] / (double)fz.rows;
          stf(fz.rmean, c, fz.rdt, (float)((1.0 - fz.momentum) * ldf(fz.rmean, c, fz.rdt) + fz.momentum * m));
          stf(fz.rvar, c, fz.rdt, (float)((1.0 - fz.momentum) * ldf(fz.rvar, c, fz.rdt) + fz.momentum * unbiased));
        }
      }
    } else {
      mu = ldf(mean, c, mdt);
      is = invstd[c];
    }
    const float sc = is * (gamma ? ldf(gamma, c, pdt) : 1.f);
    S[c] = sc;
    Tc[c] = (beta ? ldf(beta, c, pdt) : 0.f) - mu * sc;
  }
  if (fz.batch_counter && blockIdx.x == 0 && threadIdx.x == 0) *fz.batch_counter += 1;
  __syncthreads();
  const unsigned cvecs = C / V;
  const bool fixed = (256u % cvecs) == 0;            // this thread's channels never change
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  float s_r[V], t_r[V];
  if (fixed) {
    const int c0 = (int)(threadIdx.x % cvecs) * V;
#pragma unroll
    for (int k = 0; k < V; ++k) { s_r[k] = S[c0 + k]; t_r[k] = Tc[c0 + k]; }
  }
  for (size_t i0 = first; i0 < nvec; i0 += stride * BN_U) {
    uint4 xr[BN_U], rr[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i < nvec) {
        xr[u] = ld_stream(x + i * V);
        if (res) rr[u] = ld_stream(res + i * V);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= nvec) break;
      float v[V], r[V];
      unpack_vec<T>(xr[u], v);
      if (res) unpack_vec<T>(rr[u], r);
      if (!fixed) {
        const int c0 = (int)(i % cvecs) * V;
#pragma unroll
        for (int k = 0; k < V; ++k) { s_r[k] = S[c0 + k]; t_r[k] = Tc[c0 + k]; }
      }
      unsigned bits = 0;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float t = fmaf(v[k], s_r[k], t_r[k]);
        if (res) t += r[k];
        if (act == 1) {
          bits |= (t > 0.f ? 1u : 0u) << k;
          t = t > 0.f ? t : 0.f;
        }
        v[k] = t;
      }
      *reinterpret_cast<uint4*>(y + i * V) = pack_vec<T>(v);
      if (relu_mask) relu_mask[i] = (uint8_t)bits;  // one bit per element (V == 8): all the backward needs of the output
    }
  }
}

// sums[c] += sum(dy), sums[C + c] += invstd[c] * sum(dy * (x - mean[c])) under the ReLU mask; 16-byte vectors,
// BN_U rows per thread in flight.  Thread (tx, ty) owns channel vector tx of rows ty, ty + ty_n, ...
template <typename T, int U>
__global__ void __launch_bounds__(RED_THREADS)
bn_bwd_reduce_fast_kernel(const T* __restrict__ dy, const T* __restrict__ x, const void* mean, int mdt,
                          const float* invstd, const uint8_t* __restrict__ relu_mask, long long rows, int C, double* sums) {
  constexpr int V = VecOf<T>::N;
  const int cvecs = C / V;  // divides RED_THREADS or is a multiple of it (checked by the launcher)
  const int tx_n = cvecs < RED_THREADS ? cvecs : RED_THREADS;
  const int ty_n = RED_THREADS / tx_n;
  const int tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
  extern __shared__ float sh[];  // [ty_n][tx_n * V * 2]
  const long long rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
  for (int cv = tx; cv < cvecs; cv += tx_n) {  // cvecs % tx_n == 0: the same trip count for every thread
    float a0[V], a1[V], mu[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { a0[k] = 0.f; a1[k] = 0.f; mu[k] = ldf(mean, cv * V + k, mdt); }
    for (long long rb = r0 + ty; rb < r1; rb += (long long)ty_n * U) {
      uint4 gr[U], xr[U];
      unsigned bits[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = rb + (long long)u * ty_n;
        if (r < r1) {
          const size_t i = (size_t)r * cvecs + cv;
          gr[u] = ld_stream(dy + i * V);
          xr[u] = ld_stream(x + i * V);
          bits[u] = relu_mask ? relu_mask[i] : 0xffu;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = rb + (long long)u * ty_n;
        if (r >= r1) break;
        float g[V], v[V];
        unpack_vec<T>(gr[u], g);
        unpack_vec<T>(xr[u], v);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float gi = ((bits[u] >> k) & 1u) ? g[k] : 0.f;
          a0[k] += gi;
          a1[k] = fmaf(gi, v[k] - mu[k], a1[k]);
        }
      }
    }
    float* mine = sh + ((size_t)ty * tx_n + tx) * V * 2;
#pragma unroll
    for (int k = 0; k < V; ++k) { mine[k] = a0[k]; mine[V + k] = a1[k]; }
    __syncthreads();
    if (ty == 0) {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        double s0 = 0.0, s1 = 0.0;
        for (int yy = 0; yy < ty_n; ++yy) {
          const float* q = sh + ((size_t)yy * tx_n + tx) * V * 2;
          s0 += q[k];
          s1 += q[V + k];
        }
        const int c = cv * V + k;
        atomicAdd(&sums[c], s0);
        atomicAdd(&sums[C + c], s1 * (double)invstd[c]);
      }
    }
    __syncthreads();
  }
}

// dx = A[c] * dy + B[c] * x + D[c]   (training), dx = A[c] * dy (eval); dy is masked by the ReLU first.
// CTA 0 also writes the parameter gradients; with `clear_sums` the CTA that finishes last zeroes the sums
// (they are a scratch buffer that the next backward pass expects to find cleared).
template <typename T>
__global__ void __launch_bounds__(256)
bn_bwd_apply_fast_kernel(const T* __restrict__ dy, const T* __restrict__ x, const void* mean, int mdt,
                         const float* invstd, const void* gamma, int pdt, const T* __restrict__ relu_out,
                         double* sums, long long rows, int C, int training, T* __restrict__ dx, unsigned nvec,
                         T* __restrict__ dres, const uint8_t* __restrict__ relu_mask, float* dgamma, float* dbeta,
                         unsigned* clear_counter) {
  constexpr int V = VecOf<T>::N;
  extern __shared__ float coef[];
  float* A = coef;
  float* B = coef + C;
  float* D = coef + 2 * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float is = invstd[c];
    const float a = (gamma ? ldf(gamma, c, pdt) : 1.f) * is;
    A[c] = a;
    if (blockIdx.x == 0) {
      if (dbeta) dbeta[c] = (float)sums[c];
      if (dgamma) dgamma[c] = (float)sums[C + c];
    }
    if (training) {
      const float sdy = (float)(sums[c] / (double)rows), sdx = (float)(sums[C + c] / (double)rows);
      const float b = -a * is * sdx;
      B[c] = b;
      D[c] = -a * sdy - b * ldf(mean, c, mdt);
    } else {
      B[c] = 0.f;
      D[c] = 0.f;
    }
  }
  __syncthreads();
  if (clear_counter) {
    // every CTA has read the sums once it is past the barrier above; the last one to get here clears them
    __shared__ int last_sh;
    if (threadIdx.x == 0) {
      __threadfence();
      last_sh = atomicAdd(clear_counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (last_sh) {
      for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) sums[c] = 0.0;
      if (threadIdx.x == 0) *clear_counter = 0u;
    }
  }
  const unsigned cvecs = C / V;
  const bool fixed = (256u % cvecs) == 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  float a_r[V], b_r[V], d_r[V];
  if (fixed) {
    const int c0 = (int)(threadIdx.x % cvecs) * V;
#pragma unroll
    for (int k = 0; k < V; ++k) { a_r[k] = A[c0 + k]; b_r[k] = B[c0 + k]; d_r[k] = D[c0 + k]; }
  }
  for (size_t i0 = first; i0 < nvec; i0 += stride * BN_U) {
    uint4 gr[BN_U], xr[BN_U], orr[BN_U];
    unsigned bits[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i < nvec) {
        gr[u] = ld_stream(dy + i * V);
        xr[u] = ld_stream(x + i * V);
        if (relu_out) orr[u] = ld_stream(relu_out + i * V);
        bits[u] = relu_mask ? relu_mask[i] : 0xffu;
      }
    }
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= nvec) break;
      float g[V], v[V];
      unpack_vec<T>(gr[u], g);
      unpack_vec<T>(xr[u], v);
      if (relu_out) {
        float o[V];
        unpack_vec<T>(orr[u], o);
#pragma unroll
        for (int k = 0; k < V; ++k)
          if (!(o[k] > 0.f)) g[k] = 0.f;
      }
#pragma unroll
      for (int k = 0; k < V; ++k)
        if (!((bits[u] >> k) & 1u)) g[k] = 0.f;
      if (dres) *reinterpret_cast<uint4*>(dres + i * V) = pack_vec<T>(g);  // gradient of the fused residual input: the masked dy
      if (!fixed) {
        const int c0 = (int)(i % cvecs) * V;
#pragma unroll
        for (int k = 0; k < V; ++k) { a_r[k] = A[c0 + k]; b_r[k] = B[c0 + k]; d_r[k] = D[c0 + k]; }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) g[k] = fmaf(a_r[k], g[k], fmaf(b_r[k], v[k], d_r[k]));
      *reinterpret_cast<uint4*>(dx + i * V) = pack_vec<T>(g);
    }
  }
}

inline int red_grid(long long rows) {
  long long g = (rows + 63) / 64;
  if (g > 148 * 4) g = 148 * 4;
  if (g < 1) g = 1;
  return (int)g;
}
// Grid of a grid-stride apply kernel whose CTAs each rebuild the per-channel coefficients (from fp64 sums) before
// they start: one resident wave, so that this prologue runs once per CTA slot instead of once per 256 x BN_U vectors
// (small activations spent most of their time in it).
template <typename K>
inline int apply_grid_for(K kernel, size_t smem, unsigned nvec) {
  int dev = 0, sms = 148, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, smem) != cudaSuccess || per_sm < 1) per_sm = 2;
  long long g = ((long long)nvec + 256 * BN_U - 1) / (256 * BN_U);
  if (g > (long long)sms * per_sm) g = (long long)sms * per_sm;
  return g < 1 ? 1 : (int)g;
}
// Grid of a column-reduction kernel: every CTA owns an equal slice of the rows, so the grid is exactly one wave of
// resident CTAs (a grid of 4 per SM with only 3 resident ran a one-third-full second wave: 0.65 of the copy
// bandwidth for the batch-norm backward reduction).
template <typename K>
inline int red_grid_for(K kernel, size_t smem, long long rows) {
  int dev = 0, sms = 148, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, RED_THREADS, smem) != cudaSuccess || per_sm < 1) per_sm = 2;
  long long g = (rows + 63) / 64;
  if (g > (long long)sms * per_sm) g = (long long)sms * per_sm;
  if (g < 1) g = 1;
  return (int)g;
}
inline size_t red_smem(int C, int V, int NQ) {
  const int cvecs = C / V;
  const int tx_n = cvecs < RED_THREADS ? cvecs : RED_THREADS;
  const int ty_n = RED_THREADS / tx_n;
  return (size_t)ty_n * tx_n * V * NQ * sizeof(float);
}
inline int ew_grid(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return (int)g;
}

// ------------------------------------------------------------------- layer norm
template <typename T>
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const T* x, long long rows, int cols, const void* gamma,
                                                            const void* beta, int pdt, float eps, T* y, float* mean,
                                                            float* rstd) {
  // one warp per row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= rows) return;
  const T* xr = x + row * cols;
  float s = 0.f, ss = 0.f;
  for (int c = lane; c < cols; c += 32) { const float v = Cv<T>::to(xr[c]); s += v; ss += v * v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffff, s, o); ss += __shfl_xor_sync(0xffffffff, ss, o); }
  const float m = s / cols;
  float var = ss / cols - m * m;
  var = var < 0.f ? 0.f : var;
  const float r = rsqrtf(var + eps);
  if (lane == 0) { mean[row] = m; rstd[row] = r; }
  T* yr = y + row * cols;
  for (int c = lane; c < cols; c += 32) {
    float o = (Cv<T>::to(xr[c]) - m) * r;
    if (gamma) o *= ldf(gamma, c, pdt);
    if (beta) o += ldf(beta, c, pdt);
    yr[c] = Cv<T>::from(o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const T* dy, const T* x, long long rows, int cols,
                                                            const void* gamma, int pdt, const float* mean,
                                                            const float* rstd, T* dx, float* dgamma, float* dbeta) {
  // one warp per row for dx; dgamma/dbeta: each warp keeps partial sums for the
  // columns its lanes own over the rows it processes, added atomically at the end.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  constexpr int MAXC = 48;  // columns per lane kept in registers (cols <= 1536); larger rows use atomics directly
  float pg[MAXC], pb[MAXC];
  const bool keep = cols <= MAXC * 32 && (dgamma || dbeta);
  if (keep) {
#pragma unroll
    for (int i = 0; i < MAXC; ++i) { pg[i] = 0.f; pb[i] = 0.f; }
  }
  for (long long row = (long long)blockIdx.x * warps + warp; row < rows; row += (long long)gridDim.x * warps) {
    const T* xr = x + row * cols;
    const T* gr = dy + row * cols;
    const float m = mean[row], r = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float g = Cv<T>::to(gr[c]) * (gamma ? ldf(gamma, c, pdt) : 1.f);
      const float xh = (Cv<T>::to(xr[c]) - m) * r;
      s1 += g;
      s2 += g * xh;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { s1 += __shfl_xor_sync(0xffffffff, s1, o); s2 += __shfl_xor_sync(0xffffffff, s2, o); }
    s1 /= cols; s2 /= cols;
    T* dr = dx ? dx + row * cols : nullptr;
    int k = 0;
    for (int c = lane; c < cols; c += 32, ++k) {
      const float go = Cv<T>::to(gr[c]);
      const float g = go * (gamma ? ldf(gamma, c, pdt) : 1.f);
      const float xh = (Cv<T>::to(xr[c]) - m) * r;
      if (dr) dr[c] = Cv<T>::from(r * (g - s1 - xh * s2));
      if (keep) {
        if (k < MAXC) { pg[k] += go * xh; pb[k] += go; }
      } else {
        if (dgamma) atomicAdd(&dgamma[c], go * xh);
        if (dbeta) atomicAdd(&dbeta[c], go);
      }
    }
  }
  if (keep) {
    int k = 0;
    for (int c = lane; c < cols; c += 32, ++k) {
      if (k < MAXC) {
        if (dgamma) atomicAdd(&dgamma[c], pg[k]);
        if (dbeta) atomicAdd(&dbeta[c], pb[k]);
      }
    }
  }
}

}  // namespace

#define DISPATCH_FLOAT(dt, T, ...)                                   \
  switch (dt) {                                                      \
    case B200_F32: { using T = float; __VA_ARGS__; break; }          \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }         \
    default: return (int)cudaErrorInvalidValue;                      \
  }

extern "C" int b200_bn_stats(const void* x, int dt, long long rows, int C, double* sums, void* stream) {
  if (rows <= 0 || C <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  DISPATCH_FLOAT(dt, T, {
    constexpr int V = VecOf<T>::N;
    if (C % V) return (int)cudaErrorInvalidValue;
    bn_stats_kernel<T><<<red_grid_for(bn_stats_kernel<T>, red_smem(C, V, 2), rows), RED_THREADS, red_smem(C, V, 2), s>>>(
        static_cast<const T*>(x), rows, C, sums);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_bn_finalize(const double* sums, long long rows, int C, float eps, float momentum, float* mean,
                                float* invstd, void* rmean, void* rvar, int rdt, void* stream) {
  bn_finalize_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(sums, rows, C, eps, momentum, mean, invstd,
                                                                         rmean, rvar, rdt);
  return (int)cudaGetLastError();
}

extern "C" int b200_bn_invstd_from_var(const void* var, int dt, int C, float eps, float* invstd, void* stream) {
  bn_invstd_kernel<<<(C + 127) / 128, 128, 0, (cudaStream_t)stream>>>(var, dt, C, eps, invstd);
  return (int)cudaGetLastError();
}

extern "C" int b200_bn_apply_mask(const void* x, int xdt, void* y, int ydt, long long rows, int C, const void* mean, int mdt,
                                  const float* invstd, const void* gamma, const void* beta, int pdt, const void* res,
                                  int rdt, int act, void* relu_mask, void* stream);
extern "C" int b200_bn_apply(const void* x, int xdt, void* y, int ydt, long long rows, int C, const void* mean, int mdt,
                             const float* invstd, const void* gamma, const void* beta, int pdt, const void* res,
                             int rdt, int act, void* stream) {
  return b200_bn_apply_mask(x, xdt, y, ydt, rows, C, mean, mdt, invstd, gamma, beta, pdt, res, rdt, act, nullptr, stream);
}
static int bn_apply_launch(const void* x, int xdt, void* y, int ydt, long long rows, int C, const void* mean, int mdt,
                           const float* invstd, const void* gamma, const void* beta, int pdt, const void* res, int rdt,
                           int act, void* relu_mask, const BnFinalize& fz, void* stream, bool* done) {
  *done = false;
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = rows * C;
  // fast path: same 16-bit / fp32 type in and out, coefficients fit in shared memory
  if (xdt == ydt && C <= 8192 && (!res || rdt == xdt) && n / (xdt == B200_F32 ? 4 : 8) < 0xffffffffLL) {
    const int V = xdt == B200_F32 ? 4 : 8;
    if (C % V == 0) {
      const unsigned nvec = (unsigned)(n / V);
      const size_t sm = sizeof(float) * 2 * C;
      DISPATCH_FLOAT(xdt, T, (bn_apply_fast_kernel<T><<<apply_grid_for(bn_apply_fast_kernel<T>, sm, nvec), 256, sm, s>>>(
                                 static_cast<const T*>(x), static_cast<T*>(y), nvec, C, mean, mdt, invstd, gamma, beta,
                                 pdt, static_cast<const T*>(res), act, V == 8 ? static_cast<uint8_t*>(relu_mask) : nullptr, fz)));
      *done = true;
    }
  }
  return (int)cudaGetLastError();
}

// Training-mode forward in one launch: statistics from the channel sums, running-statistics update,
// normalisation, optional residual add, optional ReLU and its bit mask.  Returns cudaErrorNotSupported
// when the shape does not qualify for the vector kernel (the caller then runs finalize + apply).
extern "C" int b200_bn_apply_fused(const void* x, int dt, void* y, long long rows, int C, const double* sums, float eps,
                                   float momentum, float* save_mean, float* save_invstd, void* rmean, void* rvar, int rdt,
                                   const void* gamma, const void* beta, int pdt, const void* res, int act, void* relu_mask,
                                   long long* batch_counter, void* stream) {
  if (rows <= 0 || C <= 0) return (int)cudaErrorNotSupported;
  if (relu_mask && (dt == B200_F32 || act != 1)) return (int)cudaErrorInvalidValue;
  BnFinalize fz{sums, rows, eps, momentum, save_mean, save_invstd, rmean, rvar, rdt, batch_counter};
  bool done = false;
  const int rc = bn_apply_launch(x, dt, y, dt, rows, C, nullptr, B200_F32, nullptr, gamma, beta, pdt, res, dt, act, relu_mask,
                                 fz, stream, &done);
  if (rc) return rc;
  return done ? 0 : (int)cudaErrorNotSupported;
}

extern "C" int b200_bn_apply_mask(const void* x, int xdt, void* y, int ydt, long long rows, int C, const void* mean, int mdt,
                                  const float* invstd, const void* gamma, const void* beta, int pdt, const void* res,
                                  int rdt, int act, void* relu_mask, void* stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (relu_mask && (xdt == B200_F32 || act != 1)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = rows * C;
  {
    bool done = false;
    const int rc = bn_apply_launch(x, xdt, y, ydt, rows, C, mean, mdt, invstd, gamma, beta, pdt, res, rdt, act, relu_mask,
                                   BnFinalize{}, stream, &done);
    if (rc || done) return rc;
  }
  if (relu_mask) return (int)cudaErrorInvalidValue;  // the mask is produced by the fast path only
#define BN_APPLY(TX, TY)                                                                                            \
  {                                                                                                                 \
    constexpr int V = VecOf<TX>::N > VecOf<TY>::N ? VecOf<TY>::N : VecOf<TX>::N;                                    \
    if (C % V) return (int)cudaErrorInvalidValue;                                                                   \
    bn_apply_kernel<TX, TY><<<ew_grid(n / V), 256, 0, s>>>(static_cast<const TX*>(x), static_cast<TY*>(y), n / V, C, \
                                                            mean, mdt, invstd, gamma, beta, pdt, res, rdt, act);    \
  }
  if (xdt == B200_BF16 && ydt == B200_BF16) BN_APPLY(__nv_bfloat16, __nv_bfloat16)
  else if (xdt == B200_F16 && ydt == B200_F16) BN_APPLY(__half, __half)
  else if (xdt == B200_F32 && ydt == B200_F32) BN_APPLY(float, float)
  else if (xdt == B200_BF16 && ydt == B200_F32) BN_APPLY(__nv_bfloat16, float)
  else if (xdt == B200_F32 && ydt == B200_BF16) BN_APPLY(float, __nv_bfloat16)
  else if (xdt == B200_F16 && ydt == B200_F32) BN_APPLY(__half, float)
  else if (xdt == B200_F32 && ydt == B200_F16) BN_APPLY(float, __half)
  else return (int)cudaErrorInvalidValue;
#undef BN_APPLY
  return (int)cudaGetLastError();
}

extern "C" int b200_bn_backward_reduce(const void* dy, int dt, const void* x, int xdt, const void* mean, int mdt,
                                       const float* invstd, const void* relu_out, int rdt, long long rows, int C,
                                       double* sums, void* stream) {
  if (rows <= 0 || C <= 0) return 0;
  // rdt == B200_U8: relu_out is a bit mask (one byte per 8 consecutive elements, 16-bit activations only)
  const bool is_mask = relu_out && rdt == B200_U8;
  if (dt != xdt || (relu_out && !is_mask && rdt != dt) || (is_mask && dt == B200_F32)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  DISPATCH_FLOAT(dt, T, {
    constexpr int V = VecOf<T>::N;
    if (C % V) return (int)cudaErrorInvalidValue;
    const int cvecs = C / V;
    const bool fast = (!relu_out || (is_mask && V == 8)) && (RED_THREADS % cvecs == 0 || cvecs % RED_THREADS == 0);
    if (fast) {
      // four rows in flight per thread, four CTAs per SM: eight rows or more CTAs measured the same or slower
      // (7.38 - 8.90 ms against 7.47 ms over ResNet-50's batch norms; more CTAs mean more fp64 atomics per channel)
      bn_bwd_reduce_fast_kernel<T, 4><<<red_grid_for(bn_bwd_reduce_fast_kernel<T, 4>, red_smem(C, V, 2), rows), RED_THREADS,
                                        red_smem(C, V, 2), s>>>(
          static_cast<const T*>(dy), static_cast<const T*>(x), mean, mdt, invstd,
          is_mask ? static_cast<const uint8_t*>(relu_out) : nullptr, rows, C, sums);
    } else {
      bn_bwd_reduce_kernel<T><<<red_grid_for(bn_bwd_reduce_kernel<T>, red_smem(C, V, 2), rows), RED_THREADS, red_smem(C, V, 2), s>>>(
          static_cast<const T*>(dy), static_cast<const T*>(x), mean, mdt, invstd,
          is_mask ? nullptr : static_cast<const T*>(relu_out), (is_mask && V == 8) ? static_cast<const uint8_t*>(relu_out) : nullptr,
          rows, C, sums);
    }
  });
  return (int)cudaGetLastError();
}

// `clear_counter` (optional, a zeroed device word that the kernel leaves zeroed): the sums are a scratch
// buffer and are cleared by the kernel once every CTA has read them.
extern "C" int b200_bn_backward_apply2(const void* dy, int dt, const void* x, int xdt, const void* mean, int mdt,
                                       const float* invstd, const void* gamma, int pdt, const void* relu_out, int rdt,
                                       double* sums, long long rows, int C, int training, void* dx, int dxdt,
                                       float* dgamma, float* dbeta, void* dres, unsigned* clear_counter, void* stream) {
  if (rows <= 0 || C <= 0) return 0;
  const bool is_mask = relu_out && rdt == B200_U8;
  if (dt != xdt || (relu_out && !is_mask && rdt != dt) || (is_mask && dt == B200_F32)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = rows * C;
  if (is_mask && !(dx && dxdt == dt && C <= 8192 && C % 8 == 0 && n / 8 < 0xffffffffLL)) return (int)cudaErrorInvalidValue;
  if (dres && !(dx && dxdt == dt && C <= 8192 && C % (dt == B200_F32 ? 4 : 8) == 0)) return (int)cudaErrorInvalidValue;
  if (dx && dxdt == dt && C <= 8192 && C % (dt == B200_F32 ? 4 : 8) == 0 && n / (dt == B200_F32 ? 4 : 8) < 0xffffffffLL) {
    const int V = dt == B200_F32 ? 4 : 8;
    const unsigned nvec = (unsigned)(n / V);
    const size_t sm = sizeof(float) * 3 * C;
    DISPATCH_FLOAT(dt, T, (bn_bwd_apply_fast_kernel<T><<<apply_grid_for(bn_bwd_apply_fast_kernel<T>, sm, nvec), 256, sm, s>>>(
                               static_cast<const T*>(dy), static_cast<const T*>(x), mean, mdt, invstd, gamma, pdt,
                               is_mask ? nullptr : static_cast<const T*>(relu_out), sums, rows, C, training,
                               static_cast<T*>(dx), nvec, static_cast<T*>(dres),
                               (is_mask && V == 8) ? static_cast<const uint8_t*>(relu_out) : nullptr, dgamma, dbeta,
                               clear_counter)));
    return (int)cudaGetLastError();
  }
  if (clear_counter) return (int)cudaErrorNotSupported;  // only the vector kernel clears the sums
  if (dx) {
#define BN_BWD(T, TO)                                                                                                  \
  bn_bwd_apply_kernel<T, TO><<<ew_grid(n), 256, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x), mean, mdt, \
                                                         invstd, gamma, pdt, static_cast<const T*>(relu_out), sums,     \
                                                         rows, C, training, static_cast<TO*>(dx), n)
    if (dt == B200_BF16 && dxdt == B200_BF16) BN_BWD(__nv_bfloat16, __nv_bfloat16);
    else if (dt == B200_F16 && dxdt == B200_F16) BN_BWD(__half, __half);
    else if (dt == B200_F32 && dxdt == B200_F32) BN_BWD(float, float);
    else return (int)cudaErrorInvalidValue;
#undef BN_BWD
  }
  if (dgamma || dbeta) bn_param_grads_kernel<<<(C + 127) / 128, 128, 0, s>>>(sums, C, dgamma, dbeta);
  return (int)cudaGetLastError();
}

extern "C" int b200_bn_backward_apply(const void* dy, int dt, const void* x, int xdt, const void* mean, int mdt,
                                      const float* invstd, const void* gamma, int pdt, const void* relu_out, int rdt,
                                      const double* sums, long long rows, int C, int training, void* dx, int dxdt,
                                      float* dgamma, float* dbeta, void* dres, void* stream) {
  return b200_bn_backward_apply2(dy, dt, x, xdt, mean, mdt, invstd, gamma, pdt, relu_out, rdt, const_cast<double*>(sums), rows, C,
                                 training, dx, dxdt, dgamma, dbeta, dres, nullptr, stream);
}

extern "C" int b200_layernorm_fwd(const void* x, int dt, long long rows, int cols, const void* gamma, const void* beta,
                                  int pdt, float eps, void* y, float* mean, float* rstd, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int warps = 8;
  DISPATCH_FLOAT(dt, T, {
    layernorm_fwd_kernel<T><<<(unsigned)((rows + warps - 1) / warps), warps * 32, 0, s>>>(
        static_cast<const T*>(x), rows, cols, gamma, beta, pdt, eps, static_cast<T*>(y), mean, rstd);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_layernorm_bwd(const void* dy, const void* x, int dt, long long rows, int cols, const void* gamma,
                                  int pdt, const float* mean, const float* rstd, void* dx, float* dgamma, float* dbeta,
                                  void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int warps = 8;
  long long grid = (rows + warps - 1) / warps;
  if (grid > 148 * 2) grid = 148 * 2;
  DISPATCH_FLOAT(dt, T, {
    layernorm_bwd_kernel<T><<<(unsigned)grid, warps * 32, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),
                                                                  rows, cols, gamma, pdt, mean, rstd,
                                                                  static_cast<T*>(dx), dgamma, dbeta);
  });
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// Allocation-free batch statistics (declared in noalloc_api.h; no counterpart in the
// reference).  Same kernels as b200_bn_stats + b200_bn_finalize, but the fp64 scratch
// lives in a file-scope device array, so callers that may not allocate device memory
// can still use them.  In host code the array's name is only a handle for the runtime:
// the device address is fetched with cudaGetSymbolAddress, once per device.
#include "noalloc_api.h"

static __device__ __align__(256) double g_bn_noalloc_scratch[2 * B200_NOALLOC_BN_MAX_CHANNELS];

static int bn_noalloc_scratch_ptr(double** out) {
  static double* ptrs[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_bn_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    ptrs[dev] = static_cast<double*>(p);
  }
  *out = ptrs[dev];
  return 0;
}

extern "C" int b200_bn_batch_stats_noalloc(const void* x, int x_dtype, long long rows, int C, float eps, float* mean,
                                           float* invstd, void* stream) {
  if (C <= 0 || rows <= 0) return (int)cudaErrorInvalidValue;
  if (C > B200_NOALLOC_BN_MAX_CHANNELS) return (int)cudaErrorInvalidValue;  // beyond the built-in scratch
  const int vec = x_dtype == B200_F32 ? 4 : 8;
  if (x_dtype != B200_F32 && x_dtype != B200_BF16 && x_dtype != B200_F16) return (int)cudaErrorInvalidValue;
  if (C % vec) return (int)cudaErrorInvalidValue;
  double* scratch = nullptr;
  int rc = bn_noalloc_scratch_ptr(&scratch);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  // the sums must start at zero; the array still holds the previous call's values
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(double) * 2 * (size_t)C, s);
  if (e != cudaSuccess) return (int)e;
  rc = b200_bn_stats(x, x_dtype, rows, C, scratch, stream);
  if (rc) return rc;
  return b200_bn_finalize(scratch, rows, C, eps, 0.f, mean, invstd, nullptr, nullptr, B200_F32, stream);
}
