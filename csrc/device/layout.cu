// Layout kernels: channel-padded NHWC packing for the first convolution layer.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

__device__ __forceinline__ float ld_any(const void* p, long long i, int dt) {
  switch (dt) {
    case B200_F32: return static_cast<const float*>(p)[i];
    case B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case B200_F64: return (float)static_cast<const double*>(p)[i];
    case B200_U8: return (float)static_cast<const unsigned char*>(p)[i];
    default: return 0.f;
  }
}

// one thread per output pixel (8 channels = one 16-byte store)
__global__ void pack_nhwc8_kernel(const void* in, int in_dt, long long sn, long long sc, long long sh, long long sw,
                                  int N, int C, int H, int W, uint4* out, int out_dt, int Hp, int Wp, int pt, int pl) {
  const long long total = (long long)N * Hp * Wp;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int wp = (int)(i % Wp);
    const int hp = (int)((i / Wp) % Hp);
    const int n = (int)(i / ((long long)Wp * Hp));
    const int h = hp - pt, w = wp - pl;
    alignas(16) unsigned short v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (h >= 0 && h < H && w >= 0 && w < W) {
      const long long base = n * sn + h * sh + w * sw;
      for (int c = 0; c < C; ++c) {
        const float f = ld_any(in, base + c * sc, in_dt);
        v[c] = out_dt == B200_BF16 ? __bfloat16_as_ushort(__float2bfloat16(f)) : __half_as_ushort(__float2half(f));
      }
    }
    out[i] = *reinterpret_cast<const uint4*>(v);
  }
}

}  // namespace

extern "C" int b200_pack_nhwc8(const void* in, int in_dtype, long long sn, long long sc, long long sh, long long sw,
                               int N, int C, int H, int W, void* out, int out_dtype, int Hp, int Wp, int pad_top,
                               int pad_left, void* stream) {
  if (C > 8 || C <= 0) return (int)cudaErrorInvalidValue;
  const long long total = (long long)N * Hp * Wp;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pack_nhwc8_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(in, in_dtype, sn, sc, sh, sw, N, C, H, W,
                                                                   static_cast<uint4*>(out), out_dtype, Hp, Wp, pad_top,
                                                                   pad_left);
  return (int)cudaGetLastError();
}
