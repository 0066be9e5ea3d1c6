// float-compute instantiation of the element-wise family + the public entry point.
#include "elementwise_impl.cuh"

namespace b200ew {
int dispatch_f64(const B200EwDesc& d, cudaStream_t s);
int dispatch_i64(const B200EwDesc& d, cudaStream_t s);

template <typename SO, typename SI>
static int launch_cast(const B200EwDesc& d, cudaStream_t s) {
  ew_cast<SO, SI><<<grid_for((d.numel + 7) / 8, 256), 256, 0, s>>>(static_cast<SO*>(d.ptr[0]),
                                                                    static_cast<const SI*>(d.ptr[1]), d.numel);
  return (int)cudaGetLastError();
}
}  // namespace b200ew

extern "C" int b200_elementwise(const B200EwDesc* desc, void* stream) {
  using namespace b200ew;
  const B200EwDesc& d = *desc;
  cudaStream_t s = (cudaStream_t)stream;
  if (d.numel <= 0) return 0;
  if (d.ndim > B200_EW_MAX_DIMS || d.noperands > B200_EW_MAX_OPERANDS) return (int)cudaErrorInvalidValue;
  // Dense floating-point casts get their own fully vectorised kernels.
  if (d.op == EW_COPY && d.contiguous && d.noperands == 2 && d.scalar_mask == 0 && d.dtype[0] != d.dtype[1] &&
      aligned16(d.ptr[0]) && aligned16(d.ptr[1])) {
    const int o = d.dtype[0], i = d.dtype[1];
    if (o == B200_BF16 && i == B200_F32) return launch_cast<__nv_bfloat16, float>(d, s);
    if (o == B200_F32 && i == B200_BF16) return launch_cast<float, __nv_bfloat16>(d, s);
    if (o == B200_F16 && i == B200_F32) return launch_cast<__half, float>(d, s);
    if (o == B200_F32 && i == B200_F16) return launch_cast<float, __half>(d, s);
  }
  switch (d.compute) {
    case 0: return dispatch<float>(d, s);
    case 1: return dispatch_f64(d, s);
    default: return dispatch_i64(d, s);
  }
}
