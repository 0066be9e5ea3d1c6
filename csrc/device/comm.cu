// Collective kernels over peer-mapped memory: the hand-written replacement of the
// vendor collective library (cnclAllReduce / Broadcast / Reduce / AllGather / Send /
// Recv, torch_mlu/csrc/distributed/process_group_cncl.cpp:349-572).
//
// Transport: plain global loads and stores on peer pointers (CUDA IPC or shared cuMemCreate
// allocations); through NVSwitch every peer is reachable at full NVLink bandwidth.  When the
// arena is also bound to an NVSwitch multicast object, sums of floating types use multimem
// loads / stores (reduction and broadcast inside the switch).  No copy-engine or tensor-map
// loads touch peer memory.  Synchronisation: per-peer 64-bit sequence
// flags written with st.release.sys and polled with ld.acquire.sys; polls are bounded
// and report a timeout in a host-mapped status word instead of hanging.
//
// The all-reduce is two-shot (reduce-scatter + all-gather in one kernel): rank r owns
// shard r, pulls that shard from every peer with 16-byte loads, reduces in fp32, applies
// the scale (1/world for DDP), optionally runs the optimizer on its shard of the master
// parameters, and pushes the result to every peer with 16-byte stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include "kernels_api.h"

namespace {

constexpr int READY = 0, DONE = 16, COUNTER = B200_COMM_COUNTER_SLOT;  // slots 32..63: point-to-point ready / done;
                                                                    // COUNTER + 1: CTAs done with the cast phase
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

// ---- NVSwitch multicast accesses -------------------------------------------------------------------
// A multimem load with .add on a multicast address returns the SUM over every rank's copy of that 16-byte
// vector, computed inside the switch; a multimem store writes every rank's copy.  The per-rank link
// traffic of an all-reduce drops from 2 * (world - 1) / world to about one message size per direction.
template <typename T> struct Multimem;
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_sum(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st8(void* mc, const uint2& v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
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
// scale is a float; integer accumulators are scaled in double so that 1/world does not truncate to zero
template <typename A> __device__ __forceinline__ A apply_scale(A a, float scale) { return (A)(a * (A)scale); }
template <> __device__ __forceinline__ long long apply_scale<long long>(long long a, float scale) {
  return (long long)llrint((double)a * (double)scale);
}
template <typename T, typename A> __device__ __forceinline__ A widen(T v) { return (A)v; }
template <> __device__ __forceinline__ float widen<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float widen<__half, float>(__half v) { return __half2float(v); }
template <typename T, typename A> __device__ __forceinline__ T narrow(A v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half narrow<__half, float>(float v) { return __float2half(v); }

// Start barrier: one CTA (`this_cta_announces`) tells every peer "my data is ready"; every CTA waits for
// every peer's announcement.  no_signal (tests only) suppresses the announcement so that peers run into
// their bounded wait.  Returns false if a wait gave up.
__device__ bool start_barrier(const B200CommCtx& c, unsigned long long seq, int no_signal, unsigned long long limit,
                              bool this_cta_announces) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (this_cta_announces && threadIdx.x < c.world && !no_signal) {
    __threadfence_system();
    st_release_sys(c.flags[threadIdx.x] + READY + c.rank, seq);
  }
  if (threadIdx.x < c.world) {
    if (!bounded_wait(c.flags[c.rank] + READY + threadIdx.x, seq, c.status, threadIdx.x, limit)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}
__device__ bool start_barrier(const B200CommCtx& c, unsigned long long seq, int no_signal, unsigned long long limit) {
  return start_barrier(c, seq, no_signal, limit, blockIdx.x == 0);
}

// End barrier: the last CTA to finish tells every peer "I am done reading from and writing to you" and
// waits until every peer has said the same, so the kernel only completes when this rank's arena holds
// the full result and nobody still reads it.  With all_ctas_wait every CTA waits for the peers (and
// may then reuse memory that the peers were reading); returns false if a wait gave up.
__device__ bool end_barrier(const B200CommCtx& c, unsigned long long seq, unsigned long long limit, bool all_ctas_wait) {
  __threadfence_system();
  __syncthreads();
  __shared__ int last_sh, ok_sh;
  if (threadIdx.x == 0) {
    const unsigned long long old = atomicAdd(c.flags[c.rank] + COUNTER, 1ull);
    last_sh = (old == gridDim.x - 1) ? 1 : 0;
    if (last_sh) c.flags[c.rank][COUNTER] = 0;
    ok_sh = 1;
  }
  __syncthreads();
  if (last_sh && threadIdx.x < c.world) st_release_sys(c.flags[threadIdx.x] + DONE + c.rank, seq);
  if (!last_sh && !all_ctas_wait) return true;
  if (threadIdx.x < c.world) {
    if (!bounded_wait(c.flags[c.rank] + DONE + threadIdx.x, seq, c.status, threadIdx.x, limit)) ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
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
        if (scale != 1.f) a = apply_scale<A>(a, scale);
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
  end_barrier(c, seq, limit, false);
}

// In-switch all-reduce (sum / average of fp32, bf16 or fp16): rank r reduces shard r with multimem loads
// and publishes it with multimem stores.  Same barriers as the peer-memory kernel.
template <typename T>
__global__ void __launch_bounds__(512) allreduce_nvls_kernel(const B200CommCtx c, size_t offset, long long n, int op,
                                                             float scale, unsigned long long seq, int no_signal) {
  constexpr int V = Vec<T>::N;
  constexpr int U = 4;
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  if (!start_barrier(c, seq, no_signal, limit)) return;
  const long long nvec = (n + V - 1) / V;
  const long long per = (nvec + c.world - 1) / c.world;
  const long long v0 = per * c.rank, v1 = (v0 + per < nvec) ? v0 + per : nvec;
  float mul = scale;
  if (op == COMM_AVG) mul /= (float)c.world;
  char* mc = static_cast<char*>(c.mc) + offset;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < v1; i0 += stride * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < v1) raw[u] = Multimem<T>::ld_sum(mc + i * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= v1) break;
      if (mul != 1.f) {
        T* tv = reinterpret_cast<T*>(&raw[u]);
#pragma unroll
        for (int k = 0; k < V; ++k) tv[k] = from_f<T>(to_f<T>(tv[k]) * mul);
      }
      multimem_st16(mc + i * 16, raw[u]);
    }
  }
  end_barrier(c, seq, limit, false);
}

// One element of the optimizer update on the fp32 master parameter `wk` with reduced gradient `d`
// (already scaled); `s` indexes this rank's state shards.
__device__ __forceinline__ float opt_update(const B200FusedOptArgs& o, float wk, float d, long long s) {
  if (o.kind == 0) {
    d += o.weight_decay * wk;
    if (o.momentum != 0.f) {
      const float b = o.first_step ? d : o.momentum * o.state1[s] + (1.f - o.dampening) * d;
      o.state1[s] = b;
      d = o.nesterov ? d + o.momentum * b : b;
    }
    return wk - o.lr * d;
  }
  wk *= 1.f - o.lr * o.weight_decay;
  const float a = o.beta1 * o.state1[s] + (1.f - o.beta1) * d;
  const float v = o.beta2 * o.state2[s] + (1.f - o.beta2) * d * d;
  o.state1[s] = a;
  o.state2[s] = v;
  return wk - (o.lr / o.bc1) * (a / (sqrtf(v) / o.bc2_sqrt + o.eps));
}

// Fused bucket step.  T is the dtype of the gradients that cross NVLink.
//   phase 0 (only with o.cast_src): every CTA converts its slice of this rank's local fp32 gradients
//            into the T-typed exchange region of the arena and clears the source; the CTA that finishes
//            last announces "ready" (so peers only ever read a complete exchange region);
//   phase 1: reduce-scatter of the exchange regions (U vectors per thread in flight per peer), scale,
//            optimizer update of this rank's shard of the fp32 master parameters;
//   phase 2: the updated shard (and its optional 16-bit copy) is written to every peer;
//   phase 3 (only with o.zero_grads and no cast_src): once every peer has said "done", nobody reads this
//            rank's gradient region any more and the CTAs clear it for the next backward pass.
//
// NVLS: with a multicast mapping of the arena the reduce-scatter is one multimem load per vector (the
// switch adds the ranks' gradients) and the parameter all-gather one multimem store.
template <typename T, bool NVLS>
__global__ void __launch_bounds__(512) allreduce_opt_kernel(const B200CommCtx c, size_t goff, size_t poff, long long n,
                                                            float scale, const B200FusedOptArgs o,
                                                            unsigned long long seq) {
  constexpr int V = Vec<T>::N;
  constexpr int U = V == 4 ? 4 : 2;   // 16 floats of gradient per thread and step either way
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  const long long nvec = (n + V - 1) / V;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  __shared__ int flag_sh;
  if (o.cast_src) {
    T* mine = reinterpret_cast<T*>(static_cast<char*>(c.arena[c.rank]) + goff);
    float* src = o.cast_src;
    for (long long i = gtid; i < nvec; i += gstride) {
      alignas(16) T tmp[V];
#pragma unroll
      for (int k = 0; k < V; k += 4) {
        // the fp32 source is padded to whole vectors like every arena region
        const float4 f = *reinterpret_cast<const float4*>(src + i * V + k);
        tmp[k] = from_f<T>(f.x); tmp[k + 1] = from_f<T>(f.y); tmp[k + 2] = from_f<T>(f.z); tmp[k + 3] = from_f<T>(f.w);
        if (o.zero_grads) *reinterpret_cast<float4*>(src + i * V + k) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      reinterpret_cast<uint4*>(mine)[i] = *reinterpret_cast<const uint4*>(tmp);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned long long old = atomicAdd(c.flags[c.rank] + COUNTER + 1, 1ull);
      flag_sh = old == gridDim.x - 1;
      if (flag_sh) c.flags[c.rank][COUNTER + 1] = 0;
    }
    __syncthreads();
    // only the last CTA may announce that the exchange region is complete
    if (!start_barrier(c, seq, 0, limit, flag_sh != 0)) return;
  } else {
    if (!start_barrier(c, seq, 0, limit)) return;
  }
  const long long per = (nvec + c.world - 1) / c.world;
  const long long v0 = per * c.rank, v1 = (v0 + per < nvec) ? v0 + per : nvec;
  for (long long i0 = v0 + gtid; i0 < v1; i0 += gstride * U) {
    float g[U][V];
    if (NVLS) {
      const char* mcg = static_cast<const char*>(c.mc) + goff;
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * gstride;
        if (i < v1) raw[u] = Multimem<T>::ld_sum(mcg + i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const T* tv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
        for (int k = 0; k < V; ++k) g[u][k] = to_f<T>(tv[k]);
      }
    } else {
      for (int p = 0; p < c.world; ++p) {
        const int peer = (c.rank + p) % c.world;
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(c.arena[peer]) + goff);
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * gstride;
          if (i < v1) raw[u] = src[i];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const T* tv = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int k = 0; k < V; ++k) g[u][k] = p == 0 ? to_f<T>(tv[k]) : g[u][k] + to_f<T>(tv[k]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * gstride;
      if (i >= v1) continue;
      // optimizer on this rank's shard of the fp32 master parameters (local arena)
      const float* pw = reinterpret_cast<const float*>(static_cast<const char*>(c.arena[c.rank]) + poff) + i * V;
      const long long s = (i - v0) * V;  // index into the local state shards
      alignas(16) float w[V];
#pragma unroll
      for (int k = 0; k < V; k += 4) *reinterpret_cast<float4*>(w + k) = *reinterpret_cast<const float4*>(pw + k);
#pragma unroll
      for (int k = 0; k < V; ++k) w[k] = opt_update(o, w[k], g[u][k] * scale, s + k);
      alignas(16) unsigned short lw[V];
      if (o.lowp_offset) {
#pragma unroll
        for (int k = 0; k < V; ++k)
          lw[k] = o.lowp_dtype == B200_BF16 ? __bfloat16_as_ushort(__float2bfloat16(w[k])) : __half_as_ushort(__float2half(w[k]));
      }
      // all-gather of the updated parameters: push to every peer (fp32 master copy and the optional
      // 16-bit copy that autocast forward passes read)
      if (NVLS) {
        char* mcp = static_cast<char*>(c.mc) + poff + (size_t)i * V * 4;
#pragma unroll
        for (int k = 0; k < V; k += 4) multimem_st16(mcp + k * 4, *reinterpret_cast<const uint4*>(w + k));
        if (o.lowp_offset) {
          char* mcl = static_cast<char*>(c.mc) + o.lowp_offset + (size_t)i * V * 2;
          if (V == 8) multimem_st16(mcl, *reinterpret_cast<const uint4*>(lw));
          else multimem_st8(mcl, *reinterpret_cast<const uint2*>(lw));
        }
        continue;
      }
      for (int p = 0; p < c.world; ++p) {
        const int peer = (c.rank + p) % c.world;
        float* dst = reinterpret_cast<float*>(static_cast<char*>(c.arena[peer]) + poff) + i * V;
#pragma unroll
        for (int k = 0; k < V; k += 4) *reinterpret_cast<float4*>(dst + k) = *reinterpret_cast<const float4*>(w + k);
        if (o.lowp_offset) {
          unsigned short* lp = reinterpret_cast<unsigned short*>(static_cast<char*>(c.arena[peer]) + o.lowp_offset) + i * V;
          if (V == 8) *reinterpret_cast<uint4*>(lp) = *reinterpret_cast<const uint4*>(lw);
          else *reinterpret_cast<uint2*>(lp) = *reinterpret_cast<const uint2*>(lw);
        }
      }
    }
  }
  if (o.zero_grads && !o.cast_src) {
    // Every CTA waits for every peer's "done": the grid is at most 128 CTAs of 512 threads, all of which
    // become resident on an otherwise idle GPU, and compute kernels never wait on this one.
    const bool ok = end_barrier(c, seq, limit, /*all_ctas_wait=*/true);
    if (!ok) return;
    uint4* mine = reinterpret_cast<uint4*>(static_cast<char*>(c.arena[c.rank]) + goff);
    for (long long i = gtid; i < nvec; i += gstride) mine[i] = make_uint4(0u, 0u, 0u, 0u);
  } else {
    end_barrier(c, seq, limit, false);
  }
}

// out[i - e0] = op over ranks of arena[rank][offset + i] for i in [e0, e1): the pull half of reduce
// (root: the whole message, everybody else: nothing) and of reduce_scatter (rank r: piece r).  Ranks
// with an empty range still take part in the two barriers.
template <typename T>
__global__ void __launch_bounds__(512) reduce_range_kernel(const B200CommCtx c, size_t offset, long long e0, long long e1,
                                                           T* out, int op, unsigned long long seq) {
  using A = typename AccOf<T>::type;
  const unsigned long long limit = c.timeout_ns ? c.timeout_ns : kDefaultTimeoutNs;
  if (!start_barrier(c, seq, 0, limit)) return;
  const bool avg = op == COMM_AVG;
  for (long long i = e0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < e1; i += (long long)gridDim.x * blockDim.x) {
    A acc = 0;
    for (int p = 0; p < c.world; ++p) {
      const int peer = (c.rank + p) % c.world;
      const A v = widen<T, A>(reinterpret_cast<const T*>(static_cast<const char*>(c.arena[peer]) + offset)[i]);
      acc = p == 0 ? v : comb<A>(avg ? COMM_SUM : op, acc, v);
    }
    if (avg) acc = acc / (A)c.world;
    out[i - e0] = narrow<T, A>(acc);
  }
  end_barrier(c, seq, limit, false);
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

// Smallest message that takes the in-switch path (CATCH_B200_NVLS_MIN_KB, default 256 KiB).
extern "C" long long b200_comm_nvls_min_bytes(void) {
  static const long long v = [] {
    const char* e = getenv("CATCH_B200_NVLS_MIN_KB");
    return (e && *e) ? atoll(e) * 1024 : 256LL * 1024;
  }();
  return v;
}

// The fused bucket kernel takes the in-switch path only on request (CATCH_B200_NVLS_FUSED=1): at the 25 MB bucket
// size peer loads / stores are faster at 4 and 8 ranks (95.6 vs 111.0 us and 110.1 vs 115.8 us per bucket); the
// in-switch reduction pays off from about 64 MB per message.
static bool nvls_for_fused() {
  static const bool v = [] {
    const char* e = getenv("CATCH_B200_NVLS_FUSED");
    return e && e[0] == '1';
  }();
  return v;
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
  // In-switch reduction for sums / averages of floating types once the message is large enough for the
  // switch's higher per-access latency to pay off.
  const bool nvls = ctx->mc != nullptr && (op == COMM_SUM || op == COMM_AVG) &&
                    (dtype == B200_F32 || dtype == B200_BF16 || dtype == B200_F16) &&
                    n * (dtype == B200_F32 ? 4 : 2) >= b200_comm_nvls_min_bytes();
  if (nvls) {
    const int V = dtype == B200_F32 ? 4 : 8;
    const long long per = (((n + V - 1) / V) + ctx->world - 1) / ctx->world;
    const int grid = comm_grid((per + 3) / 4, 512, 128);
    if (dtype == B200_F32) allreduce_nvls_kernel<float><<<grid, 512, 0, s>>>(*ctx, offset, n, op, scale, seq, no_signal);
    else if (dtype == B200_BF16) allreduce_nvls_kernel<__nv_bfloat16><<<grid, 512, 0, s>>>(*ctx, offset, n, op, scale, seq, no_signal);
    else allreduce_nvls_kernel<__half><<<grid, 512, 0, s>>>(*ctx, offset, n, op, scale, seq, no_signal);
    return (int)cudaGetLastError();
  }
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
  if (ctx->world > B200_COMM_MAX_RANKS || (goff & 15) || (poff & 15) || (opt->lowp_offset & 15)) return (int)cudaErrorInvalidValue;
  if (opt->cast_src && (reinterpret_cast<uintptr_t>(opt->cast_src) & 15)) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  // Grid: enough CTAs to keep the links busy (the same sizing as the plain all-reduce), never more than
  // 128 so that all of them are resident at once (the cast phase and the clearing phase rely on that).
  const int V = grad_dtype == B200_F32 ? 4 : 8, U = grad_dtype == B200_F32 ? 4 : 2;
  const long long nvec = (n + V - 1) / V;
  const long long per = (nvec + ctx->world - 1) / ctx->world;
  long long work = (per + U - 1) / U;
  if (opt->cast_src || opt->zero_grads) work = work > nvec / 8 ? work : nvec / 8;  // the local passes cover the whole bucket
  const int grid = comm_grid(work, 512, per * 16 >= (2LL << 20) ? 128 : 64);
  const bool nvls = ctx->mc != nullptr && nvls_for_fused() && n * (grad_dtype == B200_F32 ? 4 : 2) >= b200_comm_nvls_min_bytes();
#define OPT_LAUNCH(T)                                                                                          \
  do {                                                                                                         \
    if (nvls) allreduce_opt_kernel<T, true><<<grid, 512, 0, s>>>(*ctx, goff, poff, n, scale, *opt, seq);       \
    else allreduce_opt_kernel<T, false><<<grid, 512, 0, s>>>(*ctx, goff, poff, n, scale, *opt, seq);           \
  } while (0)
  switch (grad_dtype) {
    case B200_F32:
      if (opt->cast_src) return (int)cudaErrorInvalidValue;  // fp32 gradients are exchanged in place
      OPT_LAUNCH(float);
      break;
    case B200_BF16: OPT_LAUNCH(__nv_bfloat16); break;
    case B200_F16: OPT_LAUNCH(__half); break;
    default: return (int)cudaErrorInvalidValue;
  }
#undef OPT_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int b200_comm_reduce_range(const B200CommCtx* ctx, size_t offset, long long e0, long long e1, void* out,
                                      int dtype, int op, unsigned long long seq, void* stream) {
  if (ctx->world > B200_COMM_MAX_RANKS) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = e1 > e0 ? e1 - e0 : 0;
  COMM_DISPATCH(dtype, T, (reduce_range_kernel<T><<<comm_grid(n, 512, 128), 512, 0, s>>>(*ctx, offset, e0, e1,
                                                                                         static_cast<T*>(out), op, seq)));
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
