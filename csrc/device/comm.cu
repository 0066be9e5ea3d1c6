// Collective kernels over peer-mapped memory: the hand-written replacement of the
// vendor collective library (cnclAllReduce / Broadcast / Reduce / AllGather / Send /
// Recv, torch_mlu/csrc/distributed/process_group_cncl.cpp:349-572).
//
// Transport: plain global loads and stores on peer pointers obtained through CUDA IPC;
// through NVSwitch every peer is reachable at full NVLink bandwidth.  No copy-engine
// or tensor-map loads touch peer memory.  Synchronisation: per-peer 64-bit sequence
// flags written with st.release.sys and polled with ld.acquire.sys; polls are bounded
// and report a timeout in a host-mapped status word instead of hanging.
//
// The all-reduce is two-shot (reduce-scatter + all-gather in one kernel): rank r owns
// shard r, pulls that shard from every peer with 16-byte loads, reduces in fp32, applies
// the scale (1/world for DDP), optionally runs the optimizer on its shard of the master
// parameters, and pushes the result to every peer with 16-byte stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "kernels_api.h"

namespace {

constexpr int READY = 0, DONE = 16, COUNTER = 64;  // slots 32..63: point-to-point ready / done
constexpr unsigned long long kDefaultTimeoutNs = 10000000000ull;

__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Wait until *flag >= seq.  Returns false on timeout (status set) or if another
// waiter already reported a failure.
__device__ bool bounded_wait(const unsigned long long* flag, unsigned long long seq, int* status, int peer,
                             unsigned long long limit_ns) {
  if (ld_acquire_sys(flag) >= seq) return true;
  const unsigned long long t0 = gtimer();
  unsigned spins = 0;
  while (ld_acquire_sys(flag) < seq) {
    if ((++spins & 0xff) == 0) {
      if (*((volatile int*)status) != 0) return false;
      if (gtimer() - t0 > limit_ns) {
        atomicCAS(status, 0, B200_COMM_TIMEOUT | (peer << 8));
        __threadfence_system();
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

// accumulate type: float for floating inputs, the type itself for integers / double
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<int> { using type = long long; };
template <> struct AccOf<long long> { using type = long long; };
template <> struct AccOf<double> { using type = double; };
template <> __device__ __forceinline__ float to_f<int>(int v) { return (float)v; }

template <typename A> __device__ __forceinline__ A comb(int op, A a, A b) {
  switch (op) {
    case COMM_PROD: return a * b;
    case COMM_MIN: return a < b ? a : b;
    case COMM_MAX: return a > b ? a : b;
    default: return a + b;
  }
}
template <typename T, typename A> __device__ __forceinline__ A widen(T v) { return (A)v; }
template <> __device__ __forceinline__ float widen<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float widen<__half, float>(__half v) { return __half2float(v); }
template <typename T, typename A> __device__ __forceinline__ T narrow(A v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half narrow<__half, float>(float v) { return __float2half(v); }

// Start barrier: block 0 announces "my data is ready" to every peer; every block waits
// for every peer's announcement.  Returns false if a wait gave up.
__device__ bool start_barrier(const B200CommCtx& c, unsigned long long seq, int no_signal, unsigned long long limit) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < c.world && !no_signal) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + READY + c.rank, seq);
  }
  if (threadIdx.x < c.world) {
    if (!bounded_wait(c.flags[c.rank] + READY + threadIdx.x, seq, c.status, threadIdx.x, limit)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}

// End barrier: the last block to finish tells every peer "I am done writing to you" and
// waits until every peer has said the same, so the kernel only completes when this
// rank's arena holds the full result and nobody still reads it.
__device__ void end_barrier(const B200CommCtx& c, unsigned long long seq, unsigned long long limit) {
  __threadfence_system();
  __syncthreads();
  __shared__ int last_sh;
  if (threadIdx.x == 0) {
    const unsigned long long old = atomicAdd(c.flags[c.rank] + COUNTER, 1ull);
    last_sh = (old == gridDim.x - 1) ? 1 : 0;
    if (last_sh) c.flags[c.rank][COUNTER] = 0;
  }
  __syncthreads();
  if (!last_sh) return;
  if (threadIdx.x < c.world) {
    st_release_sys(c.flags[threadIdx.x] + DONE + c.rank, seq);
    bounded_wait(c.flags[c.rank] + DONE + threadIdx.x, seq, c.status, threadIdx.x, limit);
  }
}

template <typename T>
__global__ void __launch_bounds__(512) allreduce_kernel(const B200CommCtx c, size_t offset, long long n, int op,
                                                        float scale, unsigned long long seq, int no_signal) {
  using A = typename AccOf<T>::type;
  constexpr int V = Vec<T>::N;
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  if (!start_barrier(c, seq, no_signal, limit)) return;
  const long long nvec = (n + V - 1) / V;                    // arena regions are padded to 16 bytes
  const long long per = (nvec + c.world - 1) / c.world;
  const long long v0 = per * c.rank, v1 = (v0 + per < nvec) ? v0 + per : nvec;
  const bool avg = op == COMM_AVG;
  // Four 16-byte vectors per thread and step: the four peer loads of a round are in flight together,
  // which is what keeps enough bytes on the links to cover their latency.
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * U) {
    A acc[U][V];
    uint4 raw[U];
    // read the peers in a rotated order so the ranks do not all hit the same peer at once
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(c.arena[peer]) + offset);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) raw[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T* tv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const A v = widen<T, A>(tv[k]);
          acc[u][k] = p == 0 ? v : comb<A>(avg ? COMM_SUM : op, acc[u][k], v);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      T* tv = reinterpret_cast<T*>(&raw[u]);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        A a = acc[u][k];
        if (scale != 1.f) a = (A)(a * (A)scale);
        if (avg) a = a / (A)c.world;
        tv[k] = narrow<T, A>(a);
      }
    }
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(c.arena[peer]) + offset);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < v1) dst[i] = raw[u];
      }
    }
  }
  end_barrier(c, seq, limit);
}

template <typename T>
__global__ void __launch_bounds__(512) allreduce_opt_kernel(const B200CommCtx c, size_t goff, size_t poff, long long n,
                                                            float scale, const B200FusedOptArgs o,
                                                            unsigned long long seq) {
  constexpr int V = Vec<T>::N;
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  if (!start_barrier(c, seq, 0, limit)) return;
  const long long nvec = (n + V - 1) / V;
  const long long per = (nvec + c.world - 1) / c.world;
  const long long v0 = per * c.rank, v1 = (v0 + per < nvec) ? v0 + per : nvec;
  for (long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += (long long)gridDim.x * blockDim.x) {
    float g[V];
    alignas(16) T tmp[V];
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      *reinterpret_cast<uint4*>(tmp) = reinterpret_cast<const uint4*>(static_cast<const char*>(c.arena[peer]) + goff)[i];
#pragma unroll
      for (int k = 0; k < V; ++k) g[k] = p == 0 ? to_f<T>(tmp[k]) : g[k] + to_f<T>(tmp[k]);
    }
    // optimizer on this rank's shard of the fp32 master parameters (local arena)
    float* pw = reinterpret_cast<float*>(static_cast<char*>(c.arena[c.rank]) + poff) + i * V;
    const long long s = (i - v0) * V;  // index into the local state shards
    alignas(16) float w[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float wk = pw[k];
      float d = g[k] * scale;
      if (o.kind == 0) {
        d += o.weight_decay * wk;
        if (o.momentum != 0.f) {
          const float b = o.first_step ? d : o.momentum * o.state1[s + k] + (1.f - o.dampening) * d;
          o.state1[s + k] = b;
          d = o.nesterov ? d + o.momentum * b : b;
        }
        wk -= o.lr * d;
      } else {
        wk *= 1.f - o.lr * o.weight_decay;
        const float a = o.beta1 * o.state1[s + k] + (1.f - o.beta1) * d;
        const float v = o.beta2 * o.state2[s + k] + (1.f - o.beta2) * d * d;
        o.state1[s + k] = a;
        o.state2[s + k] = v;
        wk -= (o.lr / o.bc1) * (a / (sqrtf(v) / o.bc2_sqrt + o.eps));
      }
      w[k] = wk;
    }
    // all-gather of the updated parameters: push to every peer (fp32 master copy and
    // the optional 16-bit copy used by autocast forward passes)
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      float* dst = reinterpret_cast<float*>(static_cast<char*>(c.arena[peer]) + poff) + i * V;
#pragma unroll
      for (int k = 0; k < V; k += 4) *reinterpret_cast<float4*>(dst + k) = *reinterpret_cast<const float4*>(w + k);
      if (o.lowp_offset) {
        unsigned short* lp = reinterpret_cast<unsigned short*>(static_cast<char*>(c.arena[peer]) + o.lowp_offset) + i * V;
#pragma unroll
        for (int k = 0; k < V; ++k)
          lp[k] = o.lowp_dtype == B200_BF16 ? __bfloat16_as_ushort(__float2bfloat16(w[k])) : __half_as_ushort(__float2half(w[k]));
      }
    }
  }
  end_barrier(c, seq, limit);
}

__global__ void signal_kernel(const B200CommCtx c, int which, int peer, unsigned long long seq) {
  const int t = threadIdx.x;
  if (t >= c.world || (peer >= 0 && t != peer)) return;
  __threadfence_system();
  st_release_sys(c.flags[t] + which * 16 + c.rank, seq);
}
__global__ void wait_kernel(const B200CommCtx c, int which, int peer, unsigned long long seq) {
  const int t = threadIdx.x;
  if (t >= c.world || (peer >= 0 && t != peer)) return;
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  bounded_wait(c.flags[c.rank] + which * 16 + t, seq, c.status, t, limit);
}
__global__ void copy_kernel(char* dst, const char* src, size_t bytes) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const size_t nv = bytes / 16;
    for (size_t i = tid; i < nv; i += nt) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (size_t i = nv * 16 + tid; i < bytes; i += nt) dst[i] = src[i];
  } else {
    for (size_t i = tid; i < bytes; i += nt) dst[i] = src[i];
  }
}
template <typename T>
__global__ void accumulate_kernel(T* dst, const T* src, long long n, int op) {
  using A = typename AccOf<T>::type;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = narrow<T, A>(comb<A>(op == COMM_AVG ? COMM_SUM : op, widen<T, A>(dst[i]), widen<T, A>(src[i])));
}

inline int comm_grid(long long work_items, int threads, int cap) {
  long long g = (work_items + threads - 1) / threads;
  if (g > cap) g = cap;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

#define COMM_DISPATCH(dt, T, ...)                                    \
  switch (dt) {                                                      \
    case B200_F32: { using T = float; __VA_ARGS__; break; }          \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case B200_F16: { using T = __half; __VA_ARGS__; break; }         \
    case B200_F64: { using T = double; __VA_ARGS__; break; }         \
    case B200_I32: { using T = int; __VA_ARGS__; break; }            \
    case B200_I64: { using T = long long; __VA_ARGS__; break; }      \
    default: return (int)cudaErrorInvalidValue;                      \
  }

extern "C" long long b200_comm_shard_elems(long long n, int world, int dtype) {
  const int es = (dtype == B200_F32 || dtype == B200_I32) ? 4 : ((dtype == B200_F64 || dtype == B200_I64) ? 8 : 2);
  const int V = 16 / es;
  const long long nvec = (n + V - 1) / V;
  return ((nvec + world - 1) / world) * V;
}

extern "C" int b200_comm_allreduce(const B200CommCtx* ctx, size_t offset, long long n, int dtype, int op, float scale,
                                   unsigned long long seq, int no_signal, void* stream) {
  if (n <= 0) return 0;
  if (ctx->world > B200_COMM_MAX_RANKS || (offset & 15)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  COMM_DISPATCH(dtype, T, {
    const long long per = (((n + Vec<T>::N - 1) / Vec<T>::N) + ctx->world - 1) / ctx->world;
    // enough CTAs to saturate NVLink, few enough that all of them are resident
    // large messages are bound by link bandwidth: more CTAs put more loads in flight
    const int grid = comm_grid((per + 3) / 4, 512, per * 16 >= (8LL << 20) ? 128 : 64);
    allreduce_kernel<T><<<grid, 512, 0, s>>>(*ctx, offset, n, op, scale, seq, no_signal);
  });
  return (int)cudaGetLastError();
}

extern "C" int b200_comm_allreduce_opt(const B200CommCtx* ctx, size_t goff, size_t poff, long long n, int grad_dtype,
                                       float scale, const B200FusedOptArgs* opt, unsigned long long seq, void* stream) {
  if (n <= 0) return 0;
  if (ctx->world > B200_COMM_MAX_RANKS || (goff & 15) || (poff & 15)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  switch (grad_dtype) {
    case B200_F32: {
      const long long per = (((n + 3) / 4) + ctx->world - 1) / ctx->world;
      allreduce_opt_kernel<float><<<comm_grid(per, 512, 64), 512, 0, s>>>(*ctx, goff, poff, n, scale, *opt, seq);
      break;
    }
    case B200_BF16: {
      const long long per = (((n + 7) / 8) + ctx->world - 1) / ctx->world;
      allreduce_opt_kernel<__nv_bfloat16><<<comm_grid(per, 512, 64), 512, 0, s>>>(*ctx, goff, poff, n, scale, *opt, seq);
      break;
    }
    case B200_F16: {
      const long long per = (((n + 7) / 8) + ctx->world - 1) / ctx->world;
      allreduce_opt_kernel<__half><<<comm_grid(per, 512, 64), 512, 0, s>>>(*ctx, goff, poff, n, scale, *opt, seq);
      break;
    }
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_comm_signal(const B200CommCtx* ctx, int which, int peer, unsigned long long seq, void* stream) {
  signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*ctx, which, peer, seq);
  return (int)cudaGetLastError();
}
extern "C" int b200_comm_wait(const B200CommCtx* ctx, int which, int peer, unsigned long long seq, void* stream) {
  wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*ctx, which, peer, seq);
  return (int)cudaGetLastError();
}
extern "C" int b200_comm_copy(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return 0;
  copy_kernel<<<comm_grid((long long)(bytes / 16 + 1), 512, 128), 512, 0, (cudaStream_t)stream>>>(
      static_cast<char*>(dst), static_cast<const char*>(src), bytes);
  return (int)cudaGetLastError();
}
extern "C" int b200_comm_accumulate(void* dst, const void* src, long long n, int dtype, int op, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  COMM_DISPATCH(dtype, T, (accumulate_kernel<T><<<comm_grid(n, 256, 148 * 8), 256, 0, s>>>(
                              static_cast<T*>(dst), static_cast<const T*>(src), n, op)));
  return (int)cudaGetLastError();
}
