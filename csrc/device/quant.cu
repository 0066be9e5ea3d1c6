// Int8 quantisation kernels: per-tensor activation quantisation, per-row (output
// channel) symmetric weight quantisation, abs-max for calibration.
//
// Replaces cnnlQuantizeV1/V2 and cnnlQuantizeParam of the reference
// (torch_mlu/csrc/aten/operators/cnnl/internal/quantify.cpp:93,130, quantize_param.cpp:85).
// The reference's fixed-point "position + scale" pairs become plain symmetric scales:
// q = clamp(rint(x * scale), -127, 127) with scale = 127 / absmax.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

__device__ __forceinline__ float ldf(const void* p, long long i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ signed char q8(float v, float scale) {
  float r = rintf(v * scale);
  r = fminf(fmaxf(r, -127.f), 127.f);
  return (signed char)r;
}

__global__ void quantize_kernel(const void* x, int dt, long long n, float scale, signed char* q) {
  const long long nt = (long long)gridDim.x * blockDim.x;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 16; i < n; i += nt * 16) {
    if (i + 16 <= n) {
      alignas(16) signed char out[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) out[k] = q8(ldf(x, i + k, dt), scale);
      *reinterpret_cast<uint4*>(q + i) = *reinterpret_cast<const uint4*>(out);
    } else {
      for (long long k = i; k < n; ++k) q[k] = q8(ldf(x, k, dt), scale);
    }
  }
}

__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffff, v, o));
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? sh[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffff, r, o));
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(256) quantize_rows_kernel(const void* w, int dt, long long cols, signed char* q, float* scale) {
  __shared__ float sh[32];
  const long long row = blockIdx.x, base = row * cols;
  float m = 0.f;
  for (long long c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, fabsf(ldf(w, base + c, dt)));
  m = block_max(m, sh);
  const float s = m > 0.f ? 127.f / m : 1.f;
  if (threadIdx.x == 0) scale[row] = s;
  for (long long c = threadIdx.x; c < cols; c += blockDim.x) q[base + c] = q8(ldf(w, base + c, dt), s);
}

__global__ void __launch_bounds__(256) absmax_kernel(const void* x, int dt, long long n, float* out) {
  __shared__ float sh[32];
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(ldf(x, i, dt)));
  m = block_max(m, sh);
  // non-negative floats order like their bit patterns
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(m));
}

}  // namespace

extern "C" int b200_quantize_int8(const void* x, int x_dtype, long long n, float scale, void* q, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(q) & 15) != 0) return (int)cudaErrorInvalidValue;
  long long g = (n / 16 + 255) / 256;
  g = g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g);
  quantize_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(x, x_dtype, n, scale, static_cast<signed char*>(q));
  return (int)cudaGetLastError();
}
extern "C" int b200_quantize_int8_rows(const void* w, int w_dtype, long long rows, long long cols, void* q, float* scale,
                                       void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  quantize_rows_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(w, w_dtype, cols, static_cast<signed char*>(q), scale);
  return (int)cudaGetLastError();
}
extern "C" int b200_absmax(const void* x, int x_dtype, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  long long g = (n + 255) / 256;
  g = g > 148 * 8 ? 148 * 8 : g;
  absmax_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>(x, x_dtype, n, out);
  return (int)cudaGetLastError();
}
