// 2-D pooling kernels (max with flattened indices, average, adaptive average),
// forward and backward, for arbitrary element strides (NCHW or NHWC).
//
// Replaces cnnlPoolingForward / ForwardWithIndex / Backward and
// cnnlAdaptivePoolingForward / Backward (torch_mlu/csrc/aten/operators/cnnl/internal/
// pooling_internal.cpp:129,231,311, adaptive_pooling_internal.cpp:51,72).  Unlike the
// reference, indices are PyTorch-standard flattened h*W+w positions and ceil_mode is
// handled by clamping windows (the output size is computed by the caller).
// Backward kernels are gather-style (one thread per input element), so they are
// deterministic and need no atomics.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>
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

// linear thread index -> (n, c, a, b) with c fastest (channels_last) or b fastest
__device__ __forceinline__ void decode(long long i, int C, int A, int B, int cl, int& n, int& c, int& a, int& b) {
  if (i <= 0xffffffffLL) {
    // 32-bit divisions are several times cheaper than 64-bit ones
    unsigned u = (unsigned)i;
    if (cl) {
      c = (int)(u % (unsigned)C); u /= (unsigned)C;
      b = (int)(u % (unsigned)B); u /= (unsigned)B;
      a = (int)(u % (unsigned)A); n = (int)(u / (unsigned)A);
    } else {
      b = (int)(u % (unsigned)B); u /= (unsigned)B;
      a = (int)(u % (unsigned)A); u /= (unsigned)A;
      c = (int)(u % (unsigned)C); n = (int)(u / (unsigned)C);
    }
    return;
  }
  if (cl) {
    c = (int)(i % C); i /= C;
    b = (int)(i % B); i /= B;
    a = (int)(i % A); n = (int)(i / A);
  } else {
    b = (int)(i % B); i /= B;
    a = (int)(i % A); i /= A;
    c = (int)(i % C); n = (int)(i / C);
  }
}

template <typename T>
__global__ void maxpool_fwd_kernel(const B200PoolParams p, const T* x, T* y, long long* idx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, oh, ow;
    decode(i, p.C, p.P, p.Q, p.channels_last, n, c, oh, ow);
    const T* xp = x + n * p.in_s[0] + c * p.in_s[1];
    int h0 = oh * p.sh - p.ph, w0 = ow * p.sw - p.pw;
    const int h1 = min(h0 + (p.kh - 1) * p.dh + 1, p.H), w1 = min(w0 + (p.kw - 1) * p.dw + 1, p.W);
    while (h0 < 0) h0 += p.dh;
    while (w0 < 0) w0 += p.dw;
    float best = -FLT_MAX * 2.f;  // -inf
    long long bi = (long long)h0 * p.W + w0;
    for (int h = h0; h < h1; h += p.dh)
      for (int w = w0; w < w1; w += p.dw) {
        const float v = Cv<T>::to(xp[h * p.in_s[2] + w * p.in_s[3]]);
        if (v > best || v != v) { best = v; bi = (long long)h * p.W + w; }
      }
    const long long o = n * p.out_s[0] + c * p.out_s[1] + oh * p.out_s[2] + ow * p.out_s[3];
    y[o] = Cv<T>::from(best);
    if (idx) idx[o] = bi;
  }
}

template <typename T>
__global__ void maxpool_bwd_kernel(const B200PoolParams p, const T* dy, const long long* idx, T* dx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, h, w;
    decode(i, p.C, p.H, p.W, p.channels_last, n, c, h, w);
    // output windows that can contain (h, w)
    const int kh_ext = (p.kh - 1) * p.dh + 1, kw_ext = (p.kw - 1) * p.dw + 1;
    int oh0 = (h + p.ph < kh_ext) ? 0 : (h + p.ph - kh_ext) / p.sh + 1;
    int ow0 = (w + p.pw < kw_ext) ? 0 : (w + p.pw - kw_ext) / p.sw + 1;
    const int oh1 = min((h + p.ph) / p.sh + 1, p.P), ow1 = min((w + p.pw) / p.sw + 1, p.Q);
    const long long me = (long long)h * p.W + w;
    float g = 0.f;
    const long long base = n * p.out_s[0] + c * p.out_s[1];
    for (int oh = oh0; oh < oh1; ++oh)
      for (int ow = ow0; ow < ow1; ++ow) {
        const long long o = base + oh * p.out_s[2] + ow * p.out_s[3];
        if (idx[o] == me) g += Cv<T>::to(dy[o]);
      }
    dx[n * p.in_s[0] + c * p.in_s[1] + h * p.in_s[2] + w * p.in_s[3]] = Cv<T>::from(g);
  }
}

__device__ __forceinline__ float avg_divisor(const B200PoolParams& p, int oh, int ow, int* hs, int* he, int* ws, int* we) {
  int h0 = oh * p.sh - p.ph, w0 = ow * p.sw - p.pw;
  int h1 = min(h0 + p.kh, p.H + p.ph), w1 = min(w0 + p.kw, p.W + p.pw);
  const int pool = (h1 - h0) * (w1 - w0);
  h0 = max(h0, 0); w0 = max(w0, 0); h1 = min(h1, p.H); w1 = min(w1, p.W);
  *hs = h0; *he = h1; *ws = w0; *we = w1;
  if (p.divisor_override) return (float)p.divisor_override;
  return p.count_include_pad ? (float)pool : (float)((h1 - h0) * (w1 - w0));
}

template <typename T>
__global__ void avgpool_fwd_kernel(const B200PoolParams p, const T* x, T* y, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, oh, ow, hs, he, ws, we;
    decode(i, p.C, p.P, p.Q, p.channels_last, n, c, oh, ow);
    const float div = avg_divisor(p, oh, ow, &hs, &he, &ws, &we);
    const T* xp = x + n * p.in_s[0] + c * p.in_s[1];
    float s = 0.f;
    for (int h = hs; h < he; ++h)
      for (int w = ws; w < we; ++w) s += Cv<T>::to(xp[h * p.in_s[2] + w * p.in_s[3]]);
    y[n * p.out_s[0] + c * p.out_s[1] + oh * p.out_s[2] + ow * p.out_s[3]] = Cv<T>::from(he > hs && we > ws ? s / div : 0.f);
  }
}

template <typename T>
__global__ void avgpool_bwd_kernel(const B200PoolParams p, const T* dy, T* dx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, h, w;
    decode(i, p.C, p.H, p.W, p.channels_last, n, c, h, w);
    int oh0 = (h + p.ph < p.kh) ? 0 : (h + p.ph - p.kh) / p.sh + 1;
    int ow0 = (w + p.pw < p.kw) ? 0 : (w + p.pw - p.kw) / p.sw + 1;
    const int oh1 = min((h + p.ph) / p.sh + 1, p.P), ow1 = min((w + p.pw) / p.sw + 1, p.Q);
    float g = 0.f;
    const long long base = n * p.out_s[0] + c * p.out_s[1];
    for (int oh = oh0; oh < oh1; ++oh)
      for (int ow = ow0; ow < ow1; ++ow) {
        int hs, he, ws, we;
        const float div = avg_divisor(p, oh, ow, &hs, &he, &ws, &we);
        if (h >= hs && h < he && w >= ws && w < we) g += Cv<T>::to(dy[base + oh * p.out_s[2] + ow * p.out_s[3]]) / div;
      }
    dx[n * p.in_s[0] + c * p.in_s[1] + h * p.in_s[2] + w * p.in_s[3]] = Cv<T>::from(g);
  }
}

__device__ __forceinline__ int a_start(int i, int in, int out) { return (int)(((long long)i * in) / out); }
__device__ __forceinline__ int a_end(int i, int in, int out) { return (int)(((long long)(i + 1) * in + out - 1) / out); }

template <typename T>
__global__ void adaptive_fwd_kernel(const B200PoolParams p, const T* x, T* y, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, oh, ow;
    decode(i, p.C, p.P, p.Q, p.channels_last, n, c, oh, ow);
    const int hs = a_start(oh, p.H, p.P), he = a_end(oh, p.H, p.P), ws = a_start(ow, p.W, p.Q), we = a_end(ow, p.W, p.Q);
    const T* xp = x + n * p.in_s[0] + c * p.in_s[1];
    float s = 0.f;
    for (int h = hs; h < he; ++h)
      for (int w = ws; w < we; ++w) s += Cv<T>::to(xp[h * p.in_s[2] + w * p.in_s[3]]);
    y[n * p.out_s[0] + c * p.out_s[1] + oh * p.out_s[2] + ow * p.out_s[3]] = Cv<T>::from(s / (float)((he - hs) * (we - ws)));
  }
}

template <typename T>
__global__ void adaptive_bwd_kernel(const B200PoolParams p, const T* dy, T* dx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    int n, c, h, w;
    decode(i, p.C, p.H, p.W, p.channels_last, n, c, h, w);
    // windows containing h: all oh with a_start(oh) <= h < a_end(oh)
    int oh_lo = (int)(((long long)h * p.P) / p.H), ow_lo = (int)(((long long)w * p.Q) / p.W);
    while (oh_lo > 0 && a_end(oh_lo - 1, p.H, p.P) > h) --oh_lo;
    while (ow_lo > 0 && a_end(ow_lo - 1, p.W, p.Q) > w) --ow_lo;
    float g = 0.f;
    const long long base = n * p.out_s[0] + c * p.out_s[1];
    for (int oh = oh_lo; oh < p.P && a_start(oh, p.H, p.P) <= h; ++oh) {
      const int hl = a_end(oh, p.H, p.P) - a_start(oh, p.H, p.P);
      for (int ow = ow_lo; ow < p.Q && a_start(ow, p.W, p.Q) <= w; ++ow) {
        const int wl = a_end(ow, p.W, p.Q) - a_start(ow, p.W, p.Q);
        g += Cv<T>::to(dy[base + oh * p.out_s[2] + ow * p.out_s[3]]) / (float)(hl * wl);
      }
    }
    dx[n * p.in_s[0] + c * p.in_s[1] + h * p.in_s[2] + w * p.in_s[3]] = Cv<T>::from(g);
  }
}


// ---- channels-last fast paths: one thread handles 8 consecutive channels ------------------
template <typename T>
__global__ void __launch_bounds__(256) maxpool_fwd_cl8_kernel(const B200PoolParams p, const T* __restrict__ x,
                                                              T* __restrict__ y, long long* __restrict__ idx,
                                                              unsigned total) {
  const unsigned cv = p.C / 8;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    unsigned u = i;
    const int c0 = (int)(u % cv) * 8; u /= cv;
    const int ow = (int)(u % (unsigned)p.Q); u /= (unsigned)p.Q;
    const int oh = (int)(u % (unsigned)p.P);
    const int n = (int)(u / (unsigned)p.P);
    const int h0 = max(oh * p.sh - p.ph, 0), w0 = max(ow * p.sw - p.pw, 0);
    const int h1 = min(oh * p.sh - p.ph + p.kh, p.H), w1 = min(ow * p.sw - p.pw + p.kw, p.W);
    float best[8];
    int bi[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { best[k] = -INFINITY; bi[k] = h0 * p.W + w0; }
    const T* xp = x + (size_t)n * p.in_s[0] + c0;
    for (int h = h0; h < h1; ++h)
      for (int w = w0; w < w1; ++w) {
        alignas(16) T v[8];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(xp + (size_t)h * p.in_s[2] + (size_t)w * p.in_s[3]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float f = Cv<T>::to(v[k]);
          if (f > best[k] || f != f) { best[k] = f; bi[k] = h * p.W + w; }
        }
      }
    const size_t o = (size_t)n * p.out_s[0] + (size_t)oh * p.out_s[2] + (size_t)ow * p.out_s[3] + c0;
    alignas(16) T r[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = Cv<T>::from(best[k]);
    *reinterpret_cast<uint4*>(y + o) = *reinterpret_cast<const uint4*>(r);
    if (idx) {
      alignas(16) long long li[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) li[k] = bi[k];
#pragma unroll
      for (int k = 0; k < 4; ++k) reinterpret_cast<uint4*>(idx + o)[k] = reinterpret_cast<const uint4*>(li)[k];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_cl8_kernel(const B200PoolParams p, const T* __restrict__ dy,
                                                              const long long* __restrict__ idx, T* __restrict__ dx,
                                                              unsigned total) {
  const unsigned cv = p.C / 8;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    unsigned u = i;
    const int c0 = (int)(u % cv) * 8; u /= cv;
    const int w = (int)(u % (unsigned)p.W); u /= (unsigned)p.W;
    const int h = (int)(u % (unsigned)p.H);
    const int n = (int)(u / (unsigned)p.H);
    const int oh0 = (h + p.ph < p.kh) ? 0 : (h + p.ph - p.kh) / p.sh + 1;
    const int ow0 = (w + p.pw < p.kw) ? 0 : (w + p.pw - p.kw) / p.sw + 1;
    const int oh1 = min((h + p.ph) / p.sh + 1, p.P), ow1 = min((w + p.pw) / p.sw + 1, p.Q);
    const long long me = (long long)h * p.W + w;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int oh = oh0; oh < oh1; ++oh)
      for (int ow = ow0; ow < ow1; ++ow) {
        const size_t o = (size_t)n * p.out_s[0] + (size_t)oh * p.out_s[2] + (size_t)ow * p.out_s[3] + c0;
        alignas(16) long long li[8];
        alignas(16) T v[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) reinterpret_cast<uint4*>(li)[k] = reinterpret_cast<const uint4*>(idx + o)[k];
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(dy + o);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (li[k] == me) g[k] += Cv<T>::to(v[k]);
      }
    alignas(16) T r[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) r[k] = Cv<T>::from(g[k]);
    *reinterpret_cast<uint4*>(dx + (size_t)n * p.in_s[0] + (size_t)h * p.in_s[2] + (size_t)w * p.in_s[3] + c0) =
        *reinterpret_cast<const uint4*>(r);
  }
}

// channels-last, 16-bit, C % 8 == 0, unit dilation, 16-byte aligned rows
inline bool cl8_ok(const B200PoolParams* p, const void* a, const void* b, long long total) {
  return p->channels_last && p->dtype != B200_F32 && p->C % 8 == 0 && p->dh == 1 && p->dw == 1 && p->in_s[1] == 1 &&
         p->out_s[1] == 1 && p->in_s[3] % 8 == 0 && p->in_s[2] % 8 == 0 && p->in_s[0] % 8 == 0 && p->out_s[3] % 8 == 0 &&
         p->out_s[2] % 8 == 0 && p->out_s[0] % 8 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0 &&
         total / 8 < 0xffffffffLL;
}

inline int grid_for(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

#define POOL_DISPATCH(dt, T, ...)                                    \
  switch (dt) {                                                      \
    case B200_F32: { using T = float; __VA_ARGS__; break; }          \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }         \
    default: return (int)cudaErrorInvalidValue;                      \
  }

extern "C" int b200_maxpool2d_fwd(const B200PoolParams* p, const void* x, void* y, long long* idx, void* stream) {
  const long long total = (long long)p->N * p->C * p->P * p->Q;
  if (total <= 0) return 0;
  if (cl8_ok(p, x, y, total) && (!idx || (reinterpret_cast<uintptr_t>(idx) & 15) == 0)) {
    const unsigned tv = (unsigned)(total / 8);
    if (p->dtype == B200_BF16)
      maxpool_fwd_cl8_kernel<__nv_bfloat16><<<grid_for(tv), 256, 0, (cudaStream_t)stream>>>(
          *p, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), idx, tv);
    else
      maxpool_fwd_cl8_kernel<__half><<<grid_for(tv), 256, 0, (cudaStream_t)stream>>>(
          *p, static_cast<const __half*>(x), static_cast<__half*>(y), idx, tv);
    return (int)cudaGetLastError();
  }
  POOL_DISPATCH(p->dtype, T, (maxpool_fwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(x), static_cast<T*>(y), idx, total)));
  return (int)cudaGetLastError();
}
extern "C" int b200_maxpool2d_bwd(const B200PoolParams* p, const void* dy, const long long* idx, void* dx, void* stream) {
  const long long total = (long long)p->N * p->C * p->H * p->W;
  if (total <= 0) return 0;
  if (cl8_ok(p, dx, dy, total) && (reinterpret_cast<uintptr_t>(idx) & 15) == 0) {
    const unsigned tv = (unsigned)(total / 8);
    if (p->dtype == B200_BF16)
      maxpool_bwd_cl8_kernel<__nv_bfloat16><<<grid_for(tv), 256, 0, (cudaStream_t)stream>>>(
          *p, static_cast<const __nv_bfloat16*>(dy), idx, static_cast<__nv_bfloat16*>(dx), tv);
    else
      maxpool_bwd_cl8_kernel<__half><<<grid_for(tv), 256, 0, (cudaStream_t)stream>>>(
          *p, static_cast<const __half*>(dy), idx, static_cast<__half*>(dx), tv);
    return (int)cudaGetLastError();
  }
  POOL_DISPATCH(p->dtype, T, (maxpool_bwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(dy), idx, static_cast<T*>(dx), total)));
  return (int)cudaGetLastError();
}
extern "C" int b200_avgpool2d_fwd(const B200PoolParams* p, const void* x, void* y, void* stream) {
  const long long total = (long long)p->N * p->C * p->P * p->Q;
  if (total <= 0) return 0;
  POOL_DISPATCH(p->dtype, T, (avgpool_fwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(x), static_cast<T*>(y), total)));
  return (int)cudaGetLastError();
}
extern "C" int b200_avgpool2d_bwd(const B200PoolParams* p, const void* dy, void* dx, void* stream) {
  const long long total = (long long)p->N * p->C * p->H * p->W;
  if (total <= 0) return 0;
  POOL_DISPATCH(p->dtype, T, (avgpool_bwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(dy), static_cast<T*>(dx), total)));
  return (int)cudaGetLastError();
}
extern "C" int b200_adaptive_avgpool2d_fwd(const B200PoolParams* p, const void* x, void* y, void* stream) {
  const long long total = (long long)p->N * p->C * p->P * p->Q;
  if (total <= 0) return 0;
  POOL_DISPATCH(p->dtype, T, (adaptive_fwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(x), static_cast<T*>(y), total)));
  return (int)cudaGetLastError();
}
extern "C" int b200_adaptive_avgpool2d_bwd(const B200PoolParams* p, const void* dy, void* dx, void* stream) {
  const long long total = (long long)p->N * p->C * p->H * p->W;
  if (total <= 0) return 0;
  POOL_DISPATCH(p->dtype, T, (adaptive_bwd_kernel<T><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>(
                                 *p, static_cast<const T*>(dy), static_cast<T*>(dx), total)));
  return (int)cudaGetLastError();
}
