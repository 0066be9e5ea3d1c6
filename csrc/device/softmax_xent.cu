// Softmax / log-softmax (forward, backward), NLL loss and a fused softmax +
// cross-entropy kernel over contiguous rows.
//
// Replaces cnnlSoftmaxForward / Backward and cnnlNlllossForward / Backward
// (torch_mlu/csrc/aten/operators/cnnl/internal/softmax_internal.cpp:75,126,
// nllloss_internal.cpp:118, nllloss_backward_internal.cpp:108).  One CTA of 256
// threads per row; rows are read once into registers when they fit.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>
#include "kernels_api.h"

namespace {

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

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffff, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float r = (lane < nw) ? sh[lane] : (is_max ? -FLT_MAX : 0.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffff, r, o);
    r = is_max ? fmaxf(r, t) : r + t;
  }
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(256) softmax_fwd_kernel(const void* x, int idt, void* y, int odt, int cols, int log_mode) {
  __shared__ float sh[32];
  const long long base = (long long)blockIdx.x * cols;
  float m = -FLT_MAX;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, ldf(x, base + c, idt));
  m = block_reduce(m, true, sh);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(ldf(x, base + c, idt) - m);
  s = block_reduce(s, false, sh);
  const float ls = __logf(s), inv = 1.f / s;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = ldf(x, base + c, idt) - m;
    stf(y, base + c, odt, log_mode ? v - ls : __expf(v) * inv);
  }
}

__global__ void __launch_bounds__(256) softmax_bwd_kernel(const void* dy, const void* y, int dt, void* dx, int xdt, int cols,
                                                          int log_mode) {
  __shared__ float sh[32];
  const long long base = (long long)blockIdx.x * cols;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float g = ldf(dy, base + c, dt);
    s += log_mode ? g : g * ldf(y, base + c, dt);
  }
  s = block_reduce(s, false, sh);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float g = ldf(dy, base + c, dt), o = ldf(y, base + c, dt);
    stf(dx, base + c, xdt, log_mode ? g - __expf(o) * s : o * (g - s));
  }
}

// single CTA: rows are few (batch size); deterministic
__global__ void __launch_bounds__(256) nll_fwd_kernel(const void* logp, int dt, const long long* target, const void* w,
                                                      long long rows, int cols, int reduction, long long ignore,
                                                      void* out, void* total_w) {
  __shared__ float sh[32];
  float loss = 0.f, wsum = 0.f;
  for (long long r = threadIdx.x; r < rows; r += blockDim.x) {
    const long long t = target[r];
    float l = 0.f, wt = 0.f;
    if (t != ignore && t >= 0 && t < cols) {
      wt = w ? ldf(w, t, dt) : 1.f;
      l = -ldf(logp, r * cols + t, dt) * wt;
    }
    if (reduction == 0) stf(out, r, dt, l);
    loss += l;
    wsum += wt;
  }
  loss = block_reduce(loss, false, sh);
  wsum = block_reduce(wsum, false, sh);
  if (threadIdx.x == 0) {
    if (reduction == 1) stf(out, 0, dt, loss / wsum);
    else if (reduction == 2) stf(out, 0, dt, loss);
    stf(total_w, 0, dt, wsum);
  }
}

__global__ void nll_bwd_kernel(const void* go, int dt, const long long* target, const void* w, const void* total_w,
                               long long rows, int cols, int reduction, long long ignore, void* gi) {
  const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const long long t = target[r];
  if (t == ignore || t < 0 || t >= cols) return;
  const float wt = w ? ldf(w, t, dt) : 1.f;
  float g = reduction == 0 ? ldf(go, r, dt) : ldf(go, 0, dt);
  if (reduction == 1) g /= ldf(total_w, 0, dt);
  stf(gi, r * cols + t, dt, -g * wt);
}

__global__ void count_valid_kernel(const long long* target, long long rows, long long ignore, float* n_valid) {
  __shared__ float sh[32];
  float c = 0.f;
  for (long long r = threadIdx.x; r < rows; r += blockDim.x) c += (target[r] != ignore) ? 1.f : 0.f;
  c = block_reduce(c, false, sh);
  if (threadIdx.x == 0) *n_valid = c;
}

__global__ void __launch_bounds__(256) softmax_xent_kernel(const void* x, int dt, const long long* target, int cols,
                                                           long long ignore, float smooth, float* row_loss,
                                                           const float* n_valid, void* dl, int ddt, float gscale) {
  __shared__ float sh[32];
  const long long row = blockIdx.x, base = row * cols;
  const long long t = target[row];
  const bool valid = t != ignore && t >= 0 && t < cols;
  float m = -FLT_MAX;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, ldf(x, base + c, dt));
  m = block_reduce(m, true, sh);
  float s = 0.f, sx = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = ldf(x, base + c, dt) - m;
    s += __expf(v);
    sx += v;
  }
  s = block_reduce(s, false, sh);
  sx = block_reduce(sx, false, sh);
  const float ls = __logf(s);
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (valid) {
      const float lp_t = ldf(x, base + t, dt) - m - ls;
      const float mean_lp = sx / cols - ls;
      l = -((1.f - smooth) * lp_t + smooth * mean_lp);
    }
    row_loss[row] = l;
  }
  if (dl) {
    const float scale = valid ? gscale / fmaxf(*n_valid, 1.f) : 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float p = __expf(ldf(x, base + c, dt) - m - ls);
      const float tgt = (c == t ? 1.f - smooth : 0.f) + smooth / cols;
      stf(dl, base + c, ddt, (p - tgt) * scale);
    }
  }
}

// ---- rows cached in shared memory: one read of the input, 16-byte loads and stores --------------------------
// The kernels above read a row three times, two bytes per thread and load.  For rows of some length (a 30522-word
// vocabulary in bf16 is 61 KB) that is a third of the memory roofline at best and in practice far less; here a CTA
// copies its row into shared memory with 16-byte loads while it takes the maximum, and the remaining passes run out of
// shared memory.  Used when the row fits (up to 200 KB) and rows start on 16-byte boundaries.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

// Copies cols elements of one row into shared memory and returns this thread's running maximum.  Rows need not
// start on 16-byte boundaries (30522 bf16 columns do not): the shared copy is placed at the same 16-byte phase as
// the source row, a scalar head runs up to the first boundary, 16-byte vectors follow, a scalar tail ends the row.
template <typename T>
__device__ __forceinline__ T* row_in_smem(unsigned char* smem, const T* src) {
  return reinterpret_cast<T*>(smem + (reinterpret_cast<uintptr_t>(src) & 15));
}
template <typename T>
__device__ __forceinline__ int head_elems(const T* p, int cols) {
  const int h = (int)(((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) / sizeof(T));
  return h < cols ? h : cols;
}
template <typename T>
__device__ __forceinline__ float stage_row(const T* __restrict__ src, T* row, int cols) {
  constexpr int V = Vec16<T>::N;
  float m = -FLT_MAX;
  const int head = head_elems(src, cols);
  const int nvec = (cols - head) / V;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + head) + i);
    reinterpret_cast<uint4*>(row + head)[i] = raw;
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < V; ++k) m = fmaxf(m, to_f<T>(e[k]));
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    if (c >= head && c < head + nvec * V) continue;
    const T v = src[c];
    row[c] = v;
    m = fmaxf(m, to_f<T>(v));
  }
  return m;
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256) softmax_xent_smem_kernel(const T* __restrict__ x, const long long* target, int cols,
                                                                long long ignore, float smooth, float* row_loss,
                                                                const float* n_valid, TO* __restrict__ dl, float gscale) {
  extern __shared__ __align__(16) unsigned char smem_row[];
  __shared__ float sh[32];
  const long long r = blockIdx.x, base = r * cols;
  T* row = row_in_smem<T>(smem_row, x + base);
  const long long t = target[r];
  const bool valid = t != ignore && t >= 0 && t < cols;
  float m = stage_row<T>(x + base, row, cols);
  m = block_reduce(m, true, sh);  // its barriers also publish the staged row
  float s = 0.f, sx = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = to_f<T>(row[c]) - m;
    s += __expf(v);
    sx += v;
  }
  s = block_reduce(s, false, sh);
  sx = block_reduce(sx, false, sh);
  const float ls = __logf(s);
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (valid) {
      const float lp_t = to_f<T>(row[t]) - m - ls;
      const float mean_lp = sx / cols - ls;
      l = -((1.f - smooth) * lp_t + smooth * mean_lp);
    }
    row_loss[r] = l;
  }
  if (!dl) return;
  const float scale = valid ? gscale / fmaxf(*n_valid, 1.f) : 0.f;
  const float base_t = smooth / cols;
  constexpr int VO = Vec16<TO>::N;
  TO* out = dl + base;
  const int head = head_elems(out, cols);
  const int nvec = (cols - head) / VO;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    alignas(16) TO o[VO];
#pragma unroll
    for (int k = 0; k < VO; ++k) {
      const int c = head + i * VO + k;
      const float p = __expf(to_f<T>(row[c]) - m - ls);
      o[k] = from_f<TO>((p - ((c == t ? 1.f - smooth : 0.f) + base_t)) * scale);
    }
    reinterpret_cast<uint4*>(out + head)[i] = *reinterpret_cast<const uint4*>(o);
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    if (c >= head && c < head + nvec * VO) continue;
    const float p = __expf(to_f<T>(row[c]) - m - ls);
    out[c] = from_f<TO>((p - ((c == t ? 1.f - smooth : 0.f) + base_t)) * scale);
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256) softmax_fwd_smem_kernel(const T* __restrict__ x, TO* __restrict__ y, int cols, int log_mode) {
  extern __shared__ __align__(16) unsigned char smem_row[];
  __shared__ float sh[32];
  const long long base = (long long)blockIdx.x * cols;
  T* row = row_in_smem<T>(smem_row, x + base);
  float m = stage_row<T>(x + base, row, cols);
  m = block_reduce(m, true, sh);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += __expf(to_f<T>(row[c]) - m);
  s = block_reduce(s, false, sh);
  const float ls = __logf(s), inv = 1.f / s;
  constexpr int VO = Vec16<TO>::N;
  TO* out = y + base;
  const int head = head_elems(out, cols);
  const int nvec = (cols - head) / VO;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    alignas(16) TO o[VO];
#pragma unroll
    for (int k = 0; k < VO; ++k) {
      const float v = to_f<T>(row[head + i * VO + k]) - m;
      o[k] = from_f<TO>(log_mode ? v - ls : __expf(v) * inv);
    }
    reinterpret_cast<uint4*>(out + head)[i] = *reinterpret_cast<const uint4*>(o);
  }
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    if (c >= head && c < head + nvec * VO) continue;
    const float v = to_f<T>(row[c]) - m;
    out[c] = from_f<TO>(log_mode ? v - ls : __expf(v) * inv);
  }
}

constexpr int kMaxRowBytes = 200 * 1024;

template <typename K>
inline int allow_big_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return 0;
  return (int)cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxRowBytes);
}

}  // namespace

extern "C" int b200_softmax_fwd(const void* x, int idt, void* y, int odt, long long rows, int cols, int log_mode,
                                void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (idt == odt && cols >= 1024 && (idt == B200_BF16 || idt == B200_F16 || idt == B200_F32)) {
    const int es = idt == B200_F32 ? 4 : 2;
    const size_t bytes = (size_t)cols * es + 16;  // + the row's 16-byte phase
    if (bytes <= (size_t)kMaxRowBytes) {
      int rc = 0;
#define SM_FWD(T)                                                                                              \
  do {                                                                                                         \
    rc = allow_big_smem(softmax_fwd_smem_kernel<T, T>, bytes);                                                 \
    if (!rc) softmax_fwd_smem_kernel<T, T><<<(unsigned)rows, 256, bytes, (cudaStream_t)stream>>>(              \
        static_cast<const T*>(x), static_cast<T*>(y), cols, log_mode);                                         \
  } while (0)
      if (idt == B200_BF16) SM_FWD(__nv_bfloat16);
      else if (idt == B200_F16) SM_FWD(__half);
      else SM_FWD(float);
#undef SM_FWD
      return rc ? rc : (int)cudaGetLastError();
    }
  }
  softmax_fwd_kernel<<<(unsigned)rows, cols >= 256 ? 256 : (cols >= 64 ? 64 : 32), 0, (cudaStream_t)stream>>>(
      x, idt, y, odt, cols, log_mode);
  return (int)cudaGetLastError();
}
extern "C" int b200_softmax_bwd(const void* dy, const void* y, int dt, void* dx, int xdt, long long rows, int cols,
                                int log_mode, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  softmax_bwd_kernel<<<(unsigned)rows, cols >= 256 ? 256 : (cols >= 64 ? 64 : 32), 0, (cudaStream_t)stream>>>(
      dy, y, dt, dx, xdt, cols, log_mode);
  return (int)cudaGetLastError();
}
extern "C" int b200_nll_loss_fwd(const void* logp, int dt, const long long* target, const void* w, long long rows,
                                 int cols, int reduction, long long ignore, void* out, void* total_w, void* stream) {
  nll_fwd_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(logp, dt, target, w, rows, cols, reduction, ignore, out, total_w);
  return (int)cudaGetLastError();
}
extern "C" int b200_nll_loss_bwd(const void* go, int dt, const long long* target, const void* w, const void* total_w,
                                 long long rows, int cols, int reduction, long long ignore, void* gi, void* stream) {
  if (rows <= 0) return 0;
  nll_bwd_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, (cudaStream_t)stream>>>(go, dt, target, w, total_w, rows, cols,
                                                                                   reduction, ignore, gi);
  return (int)cudaGetLastError();
}
extern "C" int b200_softmax_xent(const void* logits, int dt, const long long* target, long long rows, int cols,
                                 long long ignore, float smooth, float* row_loss, float* n_valid, void* dl, int ddt,
                                 float gscale, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  count_valid_kernel<<<1, 256, 0, s>>>(target, rows, ignore, n_valid);
  const int es = dt == B200_F32 ? 4 : 2;
  const size_t bytes = (size_t)cols * es + 16;  // + the row's 16-byte phase
  if (cols >= 1024 && (!dl || ddt == dt) && (dt == B200_BF16 || dt == B200_F16 || dt == B200_F32) &&
      bytes <= (size_t)kMaxRowBytes) {
    int rc = 0;
#define SM_XENT(T)                                                                                                   \
  do {                                                                                                               \
    rc = allow_big_smem(softmax_xent_smem_kernel<T, T>, bytes);                                                      \
    if (!rc) softmax_xent_smem_kernel<T, T><<<(unsigned)rows, 256, bytes, s>>>(                                      \
        static_cast<const T*>(logits), target, cols, ignore, smooth, row_loss, n_valid, static_cast<T*>(dl), gscale); \
  } while (0)
    if (dt == B200_BF16) SM_XENT(__nv_bfloat16);
    else if (dt == B200_F16) SM_XENT(__half);
    else SM_XENT(float);
#undef SM_XENT
    return rc ? rc : (int)cudaGetLastError();
  }
  softmax_xent_kernel<<<(unsigned)rows, 256, 0, s>>>(logits, dt, target, cols, ignore, smooth, row_loss, n_valid, dl, ddt,
                                                     gscale);
  return (int)cudaGetLastError();
}
