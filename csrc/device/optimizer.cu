// Fused multi-tensor optimizers: SGD with momentum and AdamW, one launch for up
// to 48 parameter tensors, fp32 master parameters and state, optional refresh of
// a 16-bit parameter copy in the same pass.
//
// The reference has no fused optimizer: stock torch.optim runs dozens of tiny
// element-wise launches per parameter (see its training call stack).  The update
// formulas match torch.optim.SGD / torch.optim.AdamW so optimizer state stays
// interchangeable (momentum_buffer, exp_avg, exp_avg_sq, step).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

constexpr int CHUNK = 4096;  // elements per CTA-iteration

__device__ __forceinline__ float ld_grad(const void* p, long long i, int dt) {
  if (dt == B200_F32) return static_cast<const float*>(p)[i];
  if (dt == B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void st_lowp(void* p, long long i, int dt, float v) {
  if (dt == B200_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else static_cast<__half*>(p)[i] = __float2half(v);
}

struct ChunkMap {
  int first_chunk[B200_OPT_MAX_TENSORS + 1];
};

__device__ __forceinline__ int find_tensor(const ChunkMap& m, int count, int chunk) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (m.first_chunk[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(256) sgd_kernel(const B200OptTensors t, const ChunkMap m, float lr, float mu,
                                                  float damp, float wd, int nesterov, int first, float gscale) {
  const int ti = find_tensor(m, t.count, blockIdx.x);
  const long long start = (long long)(blockIdx.x - m.first_chunk[ti]) * CHUNK;
  const long long end = start + CHUNK < t.numel[ti] ? start + CHUNK : t.numel[ti];
  float* p = static_cast<float*>(t.param[ti]);
  float* buf = static_cast<float*>(t.state1[ti]);
  const void* g = t.grad[ti];
  void* lp = t.lowp[ti];
  for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
    float w = p[i];
    float d = ld_grad(g, i, t.grad_dtype) * gscale + wd * w;
    if (mu != 0.f) {
      float b = first ? d : mu * buf[i] + (1.f - damp) * d;
      buf[i] = b;
      d = nesterov ? d + mu * b : b;
    }
    w -= lr * d;
    p[i] = w;
    if (lp) st_lowp(lp, i, t.lowp_dtype, w);
  }
}

__global__ void __launch_bounds__(256) adamw_kernel(const B200OptTensors t, const ChunkMap m, float lr, float b1, float b2,
                                                    float eps, float wd, float bc1, float bc2_sqrt, float gscale,
                                                    int l2_mode) {
  const int ti = find_tensor(m, t.count, blockIdx.x);
  const long long start = (long long)(blockIdx.x - m.first_chunk[ti]) * CHUNK;
  const long long end = start + CHUNK < t.numel[ti] ? start + CHUNK : t.numel[ti];
  float* p = static_cast<float*>(t.param[ti]);
  float* m1 = static_cast<float*>(t.state1[ti]);
  float* m2 = static_cast<float*>(t.state2[ti]);
  const void* g = t.grad[ti];
  void* lp = t.lowp[ti];
  for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
    float w = p[i];
    float d = ld_grad(g, i, t.grad_dtype) * gscale;
    if (l2_mode) d += wd * w; else w *= 1.f - lr * wd;
    const float a = b1 * m1[i] + (1.f - b1) * d;
    const float v = b2 * m2[i] + (1.f - b2) * d * d;
    m1[i] = a;
    m2[i] = v;
    const float denom = sqrtf(v) / bc2_sqrt + eps;
    w -= (lr / bc1) * (a / denom);
    p[i] = w;
    if (lp) st_lowp(lp, i, t.lowp_dtype, w);
  }
}

int build_map(const B200OptTensors* t, ChunkMap* m) {
  int chunks = 0;
  for (int i = 0; i < t->count; ++i) {
    m->first_chunk[i] = chunks;
    chunks += (int)((t->numel[i] + CHUNK - 1) / CHUNK);
  }
  m->first_chunk[t->count] = chunks;
  return chunks;
}

}  // namespace

extern "C" int b200_sgd_step(const B200OptTensors* t, float lr, float momentum, float dampening, float weight_decay,
                             int nesterov, int first_step, float grad_scale, void* stream) {
  if (t->count <= 0) return 0;
  if (t->count > B200_OPT_MAX_TENSORS) return (int)cudaErrorInvalidValue;
  ChunkMap m;
  const int chunks = build_map(t, &m);
  if (chunks == 0) return 0;
  sgd_kernel<<<chunks, 256, 0, (cudaStream_t)stream>>>(*t, m, lr, momentum, dampening, weight_decay, nesterov, first_step,
                                                       grad_scale);
  return (int)cudaGetLastError();
}

extern "C" int b200_adamw_step(const B200OptTensors* t, float lr, float beta1, float beta2, float eps, float weight_decay,
                               long long step, float grad_scale, int adam_l2_mode, void* stream) {
  if (t->count <= 0) return 0;
  if (t->count > B200_OPT_MAX_TENSORS) return (int)cudaErrorInvalidValue;
  ChunkMap m;
  const int chunks = build_map(t, &m);
  if (chunks == 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step);
  const float bc2 = sqrtf(1.f - powf(beta2, (float)step));
  adamw_kernel<<<chunks, 256, 0, (cudaStream_t)stream>>>(*t, m, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale,
                                                         adam_l2_mode);
  return (int)cudaGetLastError();
}
