// Embedding gather / scatter-add, row gather, Philox random numbers, dropout and
// the debug dump kernel.
//
// Embedding and dropout have no device kernels in the reference (they go through
// its CPU fallback); the dump kernel replaces the BANG debug kernel
// (torch_mlu/csrc/aten/operators/bang/internal/dump_internal.mlu:5-24); the
// generator replaces the MTGP32 state of generator_impl.cpp:176-208 with a
// counter-based Philox 4x32-10 stream keyed by (seed, offset).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdio.h>
#include "kernels_api.h"
#include "philox.cuh"

namespace {

__device__ __forceinline__ float ldf(const void* p, long long i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == B200_F16) return __half2float(static_cast<const __half*>(p)[i]);
  if (dt == B200_F64) return (float)static_cast<const double*>(p)[i];
  return 0.f;
}
__device__ __forceinline__ void stf(void* p, long long i, int dt, float v) {
  if (dt == B200_F32) static_cast<float*>(p)[i] = v;
  else if (dt == B200_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else if (dt == B200_F16) static_cast<__half*>(p)[i] = __float2half(v);
  else if (dt == B200_F64) static_cast<double*>(p)[i] = v;
  else if (dt == B200_BOOL || dt == B200_U8) static_cast<unsigned char*>(p)[i] = (unsigned char)v;
  else if (dt == B200_I64) static_cast<long long*>(p)[i] = (long long)v;
  else if (dt == B200_I32) static_cast<int*>(p)[i] = (int)v;
}

// one CTA-row per index; 16-byte copies when possible
__global__ void gather_rows_kernel(const char* src, const long long* idx, long long n_idx, long long row_bytes,
                                   long long n_src_rows, long long skip_idx, char* out) {
  for (long long r = blockIdx.x; r < n_idx; r += gridDim.x) {
    long long j = idx[r];
    if (j < 0) j += n_src_rows;
    char* o = out + r * row_bytes;
    const bool zero = j < 0 || j >= n_src_rows;
    const char* s = src + (zero ? 0 : j) * row_bytes;
    if ((row_bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(o)) & 15) == 0) {
      for (long long b = threadIdx.x * 16LL; b < row_bytes; b += blockDim.x * 16LL)
        *reinterpret_cast<uint4*>(o + b) = zero ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(s + b);
    } else {
      for (long long b = threadIdx.x; b < row_bytes; b += blockDim.x) o[b] = zero ? 0 : s[b];
    }
  }
  (void)skip_idx;
}

__global__ void embedding_bwd_kernel(const void* dy, int dt, const long long* idx, long long n_idx, int dim,
                                     long long pad, void* dw, int wdt) {
  for (long long r = blockIdx.x; r < n_idx; r += gridDim.x) {
    const long long j = idx[r];
    if (j == pad) continue;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float g = ldf(dy, r * dim + c, dt);
      if (wdt == B200_F32) atomicAdd(static_cast<float*>(dw) + j * dim + c, g);
      else if (wdt == B200_BF16) atomicAdd(static_cast<__nv_bfloat16*>(dw) + j * dim + c, __float2bfloat16(g));
      else atomicAdd(static_cast<__half*>(dw) + j * dim + c, __float2half(g));
    }
  }
}

// mode 0 uniform[lo,hi), 1 normal(mean,std), 2 bernoulli(p)
__global__ void rng_kernel(void* out, int dt, long long n, unsigned long long seed, unsigned long long offset, int mode,
                           float a, float b) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  for (long long base = tid * 4, it = 0; base < n; base += nthreads * 4, ++it) {
    const uint4 r = philox4(seed, (unsigned long long)tid, offset / 4 + it);
    float v[4];
    if (mode == 1) {
      const float u0 = u01(r.x), u1 = u01(r.y), u2 = u01(r.z), u3 = u01(r.w);
      const float r0 = sqrtf(-2.f * logf(u0)), r1 = sqrtf(-2.f * logf(u2));
      v[0] = r0 * cospif(2.f * u1); v[1] = r0 * sinpif(2.f * u1);
      v[2] = r1 * cospif(2.f * u3); v[3] = r1 * sinpif(2.f * u3);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = v[k] * b + a;
    } else {
      v[0] = u01(r.x); v[1] = u01(r.y); v[2] = u01(r.z); v[3] = u01(r.w);
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = mode == 0 ? a + (b - a) * v[k] : (v[k] < a ? 1.f : 0.f);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (base + k < n) stf(out, base + k, dt, v[k]);
  }
}

__global__ void dropout_kernel(const void* x, int dt, long long n, unsigned long long seed, unsigned long long offset,
                               float p, void* y, unsigned char* mask) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const float scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  for (long long base = tid * 4, it = 0; base < n; base += nthreads * 4, ++it) {
    const uint4 r = philox4(seed, (unsigned long long)tid, offset / 4 + it);
    const float u[4] = {u01(r.x), u01(r.y), u01(r.z), u01(r.w)};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long i = base + k;
      if (i < n) {
        const bool keep = u[k] >= p;
        mask[i] = keep ? 1 : 0;
        stf(y, i, dt, keep ? ldf(x, i, dt) * scale : 0.f);
      }
    }
  }
}

__global__ void dump_kernel(const void* x, int dt, long long count) {
  for (long long i = 0; i < count; ++i) printf("%lld : %f\n", i, (double)ldf(x, i, dt));
}

inline int rng_grid(long long n) {
  long long g = (n / 4 + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

extern "C" int b200_embedding_fwd(const void* weight, int dtype, const long long* idx, long long n_idx, int dim,
                                  long long padding_idx, void* out, void* stream) {
  if (n_idx <= 0 || dim <= 0) return 0;
  const int es = dtype == B200_F32 ? 4 : (dtype == B200_F64 ? 8 : 2);
  const unsigned grid = (unsigned)(n_idx < 148 * 16 ? n_idx : 148 * 16);
  gather_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(static_cast<const char*>(weight), idx, n_idx,
                                                             (long long)dim * es, 1LL << 60, padding_idx,
                                                             static_cast<char*>(out));
  return (int)cudaGetLastError();
}
extern "C" int b200_embedding_bwd(const void* dy, int dtype, const long long* idx, long long n_idx, int dim,
                                  long long padding_idx, void* dweight, int dw_dtype, void* stream) {
  if (n_idx <= 0 || dim <= 0) return 0;
  const unsigned grid = (unsigned)(n_idx < 148 * 16 ? n_idx : 148 * 16);
  embedding_bwd_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(dy, dtype, idx, n_idx, dim, padding_idx, dweight, dw_dtype);
  return (int)cudaGetLastError();
}
extern "C" int b200_index_select_rows(const void* src, int elem_bytes, const long long* idx, long long n_idx,
                                      long long row_elems, long long n_src_rows, void* out, void* stream) {
  if (n_idx <= 0 || row_elems <= 0) return 0;
  const unsigned grid = (unsigned)(n_idx < 148 * 16 ? n_idx : 148 * 16);
  gather_rows_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(static_cast<const char*>(src), idx, n_idx,
                                                             row_elems * elem_bytes, n_src_rows, -1,
                                                             static_cast<char*>(out));
  return (int)cudaGetLastError();
}
extern "C" int b200_rng_uniform(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                                double lo, double hi, void* stream) {
  if (n <= 0) return 0;
  rng_kernel<<<rng_grid(n), 256, 0, (cudaStream_t)stream>>>(out, dtype, n, seed, offset, 0, (float)lo, (float)hi);
  return (int)cudaGetLastError();
}
extern "C" int b200_rng_normal(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                               double mean, double std, void* stream) {
  if (n <= 0) return 0;
  rng_kernel<<<rng_grid(n), 256, 0, (cudaStream_t)stream>>>(out, dtype, n, seed, offset, 1, (float)mean, (float)std);
  return (int)cudaGetLastError();
}
extern "C" int b200_rng_bernoulli(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                                  double p, void* stream) {
  if (n <= 0) return 0;
  rng_kernel<<<rng_grid(n), 256, 0, (cudaStream_t)stream>>>(out, dtype, n, seed, offset, 2, (float)p, 0.f);
  return (int)cudaGetLastError();
}
extern "C" int b200_dropout_fwd(const void* x, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                                float p, void* y, unsigned char* mask, void* stream) {
  if (n <= 0) return 0;
  dropout_kernel<<<rng_grid(n), 256, 0, (cudaStream_t)stream>>>(x, dtype, n, seed, offset, p, y, mask);
  return (int)cudaGetLastError();
}
extern "C" int b200_dump_device(const void* x, int dtype, long long count, void* stream) {
  if (count <= 0) return 0;
  dump_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(x, dtype, count);
  return (int)cudaGetLastError();
}
