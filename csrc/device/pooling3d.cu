// Pooling over three spatial dimensions (and, with a depth of one, 2-D adaptive max pooling):
// max with indices, average, adaptive average, adaptive max -- forward and backward, for arbitrary
// element strides (NCDHW or channels-last-3d).
//
// Replaces the reference's cnnlPoolingForward / ForwardWithIndex / Backward calls for 5-D inputs
// (torch_mlu/csrc/aten/operators/cnnl/internal/avg_pool3d_internal.cpp:137,
// avg_pool3d_backward_internal.cpp:146, max_pool3d_with_index_internal.cpp:164,
// max_pool3d_backward_internal.cpp:150) and cnnlAdaptivePoolingForward / Backward for the
// adaptive max and 3-D adaptive average cases (adaptive_pooling_internal.cpp:51,72,
// adaptive_pooling_backward_internal.cpp:51,73).  Indices are PyTorch-standard flattened
// (d*H + h)*W + w positions; ceil_mode is handled by clamping windows.  Backward kernels gather
// (one thread per input element): deterministic, no atomics.
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

struct Idx5 { int n, c, d, h, w; };

// linear index -> (n, c, a, b, e) over extents (N, C, A, B, E); channels fastest when cl
__device__ __forceinline__ Idx5 decode5(long long i, int C, int A, int B, int E, int cl) {
  Idx5 r;
  if (cl) {
    r.c = (int)(i % C); i /= C;
    r.w = (int)(i % E); i /= E;
    r.h = (int)(i % B); i /= B;
    r.d = (int)(i % A); r.n = (int)(i / A);
  } else {
    r.w = (int)(i % E); i /= E;
    r.h = (int)(i % B); i /= B;
    r.d = (int)(i % A); i /= A;
    r.c = (int)(i % C); r.n = (int)(i / C);
  }
  return r;
}

// window of output position o along one axis
__device__ __forceinline__ void window(const B200Pool3Params& p, int axis, int o, int* lo, int* hi, int* step, int* pool) {
  const int I = p.in[axis], O = p.out[axis];
  if (p.adaptive) {
    *lo = (int)(((long long)o * I) / O);
    *hi = (int)((((long long)(o + 1)) * I + O - 1) / O);
    *step = 1;
    *pool = *hi - *lo;
    return;
  }
  int a = o * p.s[axis] - p.p[axis];
  int b = min(a + (p.k[axis] - 1) * p.dil[axis] + 1, I + p.p[axis]);
  *pool = (b - a + p.dil[axis] - 1) / p.dil[axis];   // window size counting the padding (for count_include_pad)
  b = min(b, I);
  while (a < 0) a += p.dil[axis];
  *lo = a; *hi = b; *step = p.dil[axis];
}

template <typename T>
__global__ void pool3_fwd_kernel(const B200Pool3Params p, const T* x, T* y, long long* idx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const Idx5 o = decode5(i, p.C, p.out[0], p.out[1], p.out[2], p.channels_last);
    int d0, d1, ds, dp, h0, h1, hs, hp, w0, w1, ws, wp;
    window(p, 0, o.d, &d0, &d1, &ds, &dp);
    window(p, 1, o.h, &h0, &h1, &hs, &hp);
    window(p, 2, o.w, &w0, &w1, &ws, &wp);
    const T* xp = x + o.n * p.in_s[0] + o.c * p.in_s[1];
    const long long oo = o.n * p.out_s[0] + o.c * p.out_s[1] + o.d * p.out_s[2] + o.h * p.out_s[3] + o.w * p.out_s[4];
    if (p.is_max) {
      float best = -FLT_MAX * 2.f;  // -inf
      long long bi = ((long long)d0 * p.in[1] + h0) * p.in[2] + w0;
      for (int d = d0; d < d1; d += ds)
        for (int h = h0; h < h1; h += hs)
          for (int w = w0; w < w1; w += ws) {
            const float v = Cv<T>::to(xp[d * p.in_s[2] + h * p.in_s[3] + w * p.in_s[4]]);
            if (v > best || v != v) { best = v; bi = ((long long)d * p.in[1] + h) * p.in[2] + w; }
          }
      y[oo] = Cv<T>::from(best);
      if (idx) idx[oo] = bi;
    } else {
      float acc = 0.f;
      int cnt = 0;
      for (int d = d0; d < d1; d += ds)
        for (int h = h0; h < h1; h += hs)
          for (int w = w0; w < w1; w += ws) {
            acc += Cv<T>::to(xp[d * p.in_s[2] + h * p.in_s[3] + w * p.in_s[4]]);
            ++cnt;
          }
      float div = p.divisor_override ? (float)p.divisor_override : (p.count_include_pad && !p.adaptive ? (float)(dp * hp * wp) : (float)cnt);
      y[oo] = Cv<T>::from(cnt > 0 || p.count_include_pad ? acc / div : 0.f);
    }
  }
}

// output positions whose window can contain input position v along one axis: [lo, hi)
__device__ __forceinline__ void owners(const B200Pool3Params& p, int axis, int v, int* lo, int* hi) {
  const int I = p.in[axis], O = p.out[axis];
  if (p.adaptive) {
    // windows [floor(o*I/O), ceil((o+1)*I/O)) : o ranges over floor(v*O/I) +- 1, clipped and checked by the caller
    int a = (int)(((long long)v * O) / I) - 1, b = (int)((((long long)(v + 1)) * O + I - 1) / I) + 1;
    *lo = max(a, 0); *hi = min(b, O);
    return;
  }
  const int ext = (p.k[axis] - 1) * p.dil[axis] + 1;
  *lo = (v + p.p[axis] < ext) ? 0 : (v + p.p[axis] - ext) / p.s[axis] + 1;
  *hi = min((v + p.p[axis]) / p.s[axis] + 1, O);
}

template <typename T>
__global__ void pool3_bwd_kernel(const B200Pool3Params p, const T* dy, const long long* idx, T* dx, long long total) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const Idx5 v = decode5(i, p.C, p.in[0], p.in[1], p.in[2], p.channels_last);
    int od0, od1, oh0, oh1, ow0, ow1;
    owners(p, 0, v.d, &od0, &od1);
    owners(p, 1, v.h, &oh0, &oh1);
    owners(p, 2, v.w, &ow0, &ow1);
    const long long me = ((long long)v.d * p.in[1] + v.h) * p.in[2] + v.w;
    const long long base = v.n * p.out_s[0] + v.c * p.out_s[1];
    float g = 0.f;
    for (int od = od0; od < od1; ++od)
      for (int oh = oh0; oh < oh1; ++oh)
        for (int ow = ow0; ow < ow1; ++ow) {
          const long long o = base + od * p.out_s[2] + oh * p.out_s[3] + ow * p.out_s[4];
          if (p.is_max) {
            if (idx[o] == me) g += Cv<T>::to(dy[o]);
            continue;
          }
          int d0, d1, ds, dp, h0, h1, hs, hp, w0, w1, ws, wp;
          window(p, 0, od, &d0, &d1, &ds, &dp);
          window(p, 1, oh, &h0, &h1, &hs, &hp);
          window(p, 2, ow, &w0, &w1, &ws, &wp);
          if (v.d < d0 || v.d >= d1 || v.h < h0 || v.h >= h1 || v.w < w0 || v.w >= w1) continue;
          const int cnt = (d1 - d0) * (h1 - h0) * (w1 - w0);  // average pooling has no dilation
          const float div = p.divisor_override ? (float)p.divisor_override
                                               : (p.count_include_pad && !p.adaptive ? (float)(dp * hp * wp) : (float)cnt);
          g += Cv<T>::to(dy[o]) / div;
        }
    dx[v.n * p.in_s[0] + v.c * p.in_s[1] + v.d * p.in_s[2] + v.h * p.in_s[3] + v.w * p.in_s[4]] = Cv<T>::from(g);
  }
}

inline int grid_for(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

extern "C" int b200_pool3d_fwd(const B200Pool3Params* p, const void* x, void* y, long long* indices, void* stream) {
  const long long total = (long long)p->N * p->C * p->out[0] * p->out[1] * p->out[2];
  if (total <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  switch (p->dtype) {
    case B200_F32: pool3_fwd_kernel<float><<<grid_for(total), 256, 0, s>>>(*p, (const float*)x, (float*)y, indices, total); break;
    case B200_BF16: pool3_fwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(*p, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, indices, total); break;
    case B200_F16: pool3_fwd_kernel<__half><<<grid_for(total), 256, 0, s>>>(*p, (const __half*)x, (__half*)y, indices, total); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_pool3d_bwd(const B200Pool3Params* p, const void* dy, const long long* indices, void* dx, void* stream) {
  const long long total = (long long)p->N * p->C * p->in[0] * p->in[1] * p->in[2];
  if (total <= 0) return 0;
  if (p->is_max && !indices) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  switch (p->dtype) {
    case B200_F32: pool3_bwd_kernel<float><<<grid_for(total), 256, 0, s>>>(*p, (const float*)dy, indices, (float*)dx, total); break;
    case B200_BF16: pool3_bwd_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, s>>>(*p, (const __nv_bfloat16*)dy, indices, (__nv_bfloat16*)dx, total); break;
    case B200_F16: pool3_bwd_kernel<__half><<<grid_for(total), 256, 0, s>>>(*p, (const __half*)dy, indices, (__half*)dx, total); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
