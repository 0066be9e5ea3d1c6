// Reductions over arbitrary dimension sets: sum / mean / prod / max / min /
// any / all / norms / argmax / argmin.
//
// Replaces cnnlReduce (torch_mlu/csrc/aten/operators/cnnl/internal/reduceOps_internal.cpp:210).
// One CTA (or one warp for short reductions) produces one output element; when
// there are few outputs and many inputs the reduced range is split over several
// CTAs that write partials, and a second pass folds them.  Accumulation is fp32
// (fp64 for double inputs is not offered here; the host layer routes those to the
// CPU path), integer inputs accumulate in fp32 for sum/mean only through the host's
// dtype choice -- exact integer sums use the int64 path.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>
#include "kernels_api.h"

namespace {

__device__ __forceinline__ float ldf(const void* p, long long i, int dt) {
  switch (dt) {
    case B200_F32: return static_cast<const float*>(p)[i];
    case B200_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_F16: return __half2float(static_cast<const __half*>(p)[i]);
    case B200_F64: return (float)static_cast<const double*>(p)[i];
    case B200_I64: return (float)static_cast<const long long*>(p)[i];
    case B200_I32: return (float)static_cast<const int*>(p)[i];
    case B200_I16: return (float)static_cast<const short*>(p)[i];
    case B200_I8: return (float)static_cast<const signed char*>(p)[i];
    case B200_U8: return (float)static_cast<const unsigned char*>(p)[i];
    case B200_BOOL: return static_cast<const unsigned char*>(p)[i] ? 1.f : 0.f;
  }
  return 0.f;
}
__device__ __forceinline__ void st_out(void* p, long long i, int dt, float v) {
  switch (dt) {
    case B200_F32: static_cast<float*>(p)[i] = v; break;
    case B200_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v); break;
    case B200_F16: static_cast<__half*>(p)[i] = __float2half(v); break;
    case B200_F64: static_cast<double*>(p)[i] = v; break;
    case B200_I64: static_cast<long long*>(p)[i] = (long long)v; break;
    case B200_I32: static_cast<int*>(p)[i] = (int)v; break;
    case B200_I16: static_cast<short*>(p)[i] = (short)v; break;
    case B200_I8: static_cast<signed char*>(p)[i] = (signed char)v; break;
    case B200_U8: static_cast<unsigned char*>(p)[i] = (unsigned char)v; break;
    case B200_BOOL: static_cast<unsigned char*>(p)[i] = v != 0.f; break;
  }
}

struct Acc {
  float v;
  long long idx;
};

__device__ __forceinline__ Acc identity(int op) {
  Acc a;
  a.idx = -1;
  switch (op) {
    case RED_PROD: a.v = 1.f; break;
    case RED_MAX: case RED_ARGMAX: a.v = -INFINITY; break;
    case RED_MIN: case RED_ARGMIN: a.v = INFINITY; break;
    case RED_ALL: a.v = 1.f; break;
    default: a.v = 0.f;
  }
  return a;
}
__device__ __forceinline__ float pre(int op, float x) {
  switch (op) {
    case RED_NORM1: case RED_NORM_INF: return fabsf(x);
    case RED_NORM2: case RED_SUMSQ: return x * x;
    case RED_ANY: case RED_ALL: return x != 0.f ? 1.f : 0.f;
    default: return x;
  }
}
__device__ __forceinline__ Acc combine(int op, Acc a, Acc b) {
  switch (op) {
    case RED_PROD: a.v *= b.v; return a;
    case RED_MAX: case RED_ARGMAX: case RED_NORM_INF:
      // NaN propagates; ties keep the smaller index
      if (b.idx >= 0 && (a.idx < 0 || b.v > a.v || (b.v != b.v && a.v == a.v) || (b.v == a.v && b.idx < a.idx))) return b;
      return a;
    case RED_MIN: case RED_ARGMIN:
      if (b.idx >= 0 && (a.idx < 0 || b.v < a.v || (b.v != b.v && a.v == a.v) || (b.v == a.v && b.idx < a.idx))) return b;
      return a;
    case RED_ANY: a.v = (a.v != 0.f || b.v != 0.f) ? 1.f : 0.f; return a;
    case RED_ALL: a.v = (a.v != 0.f && b.v != 0.f) ? 1.f : 0.f; return a;
    default: a.v += b.v; return a;
  }
}
__device__ __forceinline__ bool is_minmax(int op) {
  return op == RED_MAX || op == RED_MIN || op == RED_ARGMAX || op == RED_ARGMIN || op == RED_NORM_INF;
}

__device__ __forceinline__ Acc block_fold(int op, Acc a, Acc* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.v = __shfl_xor_sync(0xffffffff, a.v, o);
    b.idx = __shfl_xor_sync(0xffffffff, a.idx, o);
    a = combine(op, a, b);
  }
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  Acc r = lane < nw ? sh[lane] : identity(op);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.v = __shfl_xor_sync(0xffffffff, r.v, o);
    b.idx = __shfl_xor_sync(0xffffffff, r.idx, o);
    r = combine(op, r, b);
  }
  __syncthreads();
  return r;
}

__device__ __forceinline__ float finish(int op, float v, long long n_red) {
  if (op == RED_MEAN) return v / (float)n_red;
  if (op == RED_NORM2) return sqrtf(v);
  return v;
}

// grid: (n_out, splits)
__global__ void __launch_bounds__(256) reduce_kernel(const B200ReduceParams p) {
  __shared__ Acc sh[32];
  const long long o = blockIdx.x;
  long long rem = o, base = 0;
  for (int d = p.n_kept - 1; d >= 0; --d) {
    base += (rem % p.kept_size[d]) * p.kept_in_stride[d];
    rem /= p.kept_size[d];
  }
  const long long per = (p.n_red + p.splits - 1) / p.splits;
  const long long j0 = (long long)blockIdx.y * per;
  const long long j1 = j0 + per < p.n_red ? j0 + per : p.n_red;
  Acc a = identity(p.op);
  for (long long j = j0 + threadIdx.x; j < j1; j += blockDim.x) {
    long long r = j, off = base;
    for (int d = p.n_reduced - 1; d >= 0; --d) {
      off += (r % p.red_size[d]) * p.red_in_stride[d];
      r /= p.red_size[d];
    }
    Acc b;
    b.v = pre(p.op, ldf(p.in, off, p.in_dtype));
    b.idx = j;
    if (is_minmax(p.op)) a = combine(p.op, a, b);
    else { b.idx = -1; a = combine(p.op, a, b); }
  }
  a = block_fold(p.op, a, sh);
  if (threadIdx.x != 0) return;
  if (p.splits > 1) {
    p.workspace[(o * p.splits + blockIdx.y) * 2] = a.v;
    reinterpret_cast<long long*>(p.workspace + (size_t)p.n_out * p.splits * 2)[o * p.splits + blockIdx.y] = a.idx;
    return;
  }
  if (p.op == RED_ARGMAX || p.op == RED_ARGMIN) {
    static_cast<long long*>(p.out)[o] = a.idx;
  } else {
    st_out(p.out, o, p.out_dtype, finish(p.op, a.v, p.n_red));
    if (p.out_index) p.out_index[o] = a.idx;
  }
}

// Short reductions with many outputs (global average pooling over a channels-last tensor: 49 elements per
// output, half a million outputs): one thread per output, adjacent threads take adjacent outputs, so when the
// innermost kept dimension is dense in memory every load of a warp is one coalesced line.
__global__ void __launch_bounds__(256) reduce_per_thread_kernel(const B200ReduceParams p) {
  const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= p.n_out) return;
  long long rem = o, base = 0;
  for (int d = p.n_kept - 1; d >= 0; --d) {
    base += (rem % p.kept_size[d]) * p.kept_in_stride[d];
    rem /= p.kept_size[d];
  }
  Acc a = identity(p.op);
  const bool mm = is_minmax(p.op);
  if (p.n_reduced == 1) {
    const long long st = p.red_in_stride[0];
    for (long long j = 0; j < p.n_red; ++j) {
      Acc b;
      b.v = pre(p.op, ldf(p.in, base + j * st, p.in_dtype));
      b.idx = mm ? j : -1;
      a = combine(p.op, a, b);
    }
  } else {
    for (long long j = 0; j < p.n_red; ++j) {
      long long r = j, off = base;
      for (int d = p.n_reduced - 1; d >= 0; --d) {
        off += (r % p.red_size[d]) * p.red_in_stride[d];
        r /= p.red_size[d];
      }
      Acc b;
      b.v = pre(p.op, ldf(p.in, off, p.in_dtype));
      b.idx = mm ? j : -1;
      a = combine(p.op, a, b);
    }
  }
  if (p.op == RED_ARGMAX || p.op == RED_ARGMIN) {
    static_cast<long long*>(p.out)[o] = a.idx;
  } else {
    st_out(p.out, o, p.out_dtype, finish(p.op, a.v, p.n_red));
    if (p.out_index) p.out_index[o] = a.idx;
  }
}

__global__ void reduce_final_kernel(const B200ReduceParams p) {
  const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= p.n_out) return;
  const long long* idxs = reinterpret_cast<const long long*>(p.workspace + (size_t)p.n_out * p.splits * 2);
  Acc a = identity(p.op);
  for (int s = 0; s < p.splits; ++s) {
    Acc b;
    b.v = p.workspace[(o * p.splits + s) * 2];
    b.idx = idxs[o * p.splits + s];
    if (!is_minmax(p.op)) b.idx = -1;
    else if (b.idx < 0) continue;
    a = combine(p.op, a, b);
  }
  if (p.op == RED_ARGMAX || p.op == RED_ARGMIN) {
    static_cast<long long*>(p.out)[o] = a.idx;
  } else {
    st_out(p.out, o, p.out_dtype, finish(p.op, a.v, p.n_red));
    if (p.out_index) p.out_index[o] = a.idx;
  }
}

// Sum / mean over the rows of a dense [n_red, n_out] view (bias gradients, channel sums): a warp reads
// 32 adjacent columns of a row, eight warps take different rows, so every load is coalesced.
__global__ void __launch_bounds__(256) reduce_outer_kernel(const B200ReduceParams p) {
  __shared__ float sh[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long col = (long long)blockIdx.x * 32 + tx;
  const long long per = (p.n_red + p.splits - 1) / p.splits;
  const long long r0 = (long long)blockIdx.y * per;
  const long long r1 = r0 + per < p.n_red ? r0 + per : p.n_red;
  float acc = 0.f;
  if (col < p.n_out) {
    long long r = r0 + ty;
    for (; r + 24 < r1; r += 32) {
      const float a = ldf(p.in, r * p.n_out + col, p.in_dtype), b = ldf(p.in, (r + 8) * p.n_out + col, p.in_dtype);
      const float c = ldf(p.in, (r + 16) * p.n_out + col, p.in_dtype), d = ldf(p.in, (r + 24) * p.n_out + col, p.in_dtype);
      acc += (a + b) + (c + d);
    }
    for (; r < r1; r += 8) acc += ldf(p.in, r * p.n_out + col, p.in_dtype);
  }
  sh[ty][tx] = acc;
  __syncthreads();
  if (ty != 0 || col >= p.n_out) return;
  float s = 0.f;
#pragma unroll
  for (int y = 0; y < 8; ++y) s += sh[y][tx];
  if (p.splits > 1) p.workspace[(long long)blockIdx.y * p.n_out + col] = s;
  else st_out(p.out, col, p.out_dtype, finish(p.op, s, p.n_red));
}
__global__ void reduce_outer_final_kernel(const B200ReduceParams p) {
  const long long col = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= p.n_out) return;
  float s = 0.f;
  for (int k = 0; k < p.splits; ++k) s += p.workspace[(long long)k * p.n_out + col];
  st_out(p.out, col, p.out_dtype, finish(p.op, s, p.n_red));
}

// true when the kept dimensions are one dense inner block and the reduced ones one dense outer block
static bool is_outer_reduction(const B200ReduceParams* p) {
  if (p->op != RED_SUM && p->op != RED_MEAN) return false;
  if (p->n_kept < 1 || p->n_reduced < 1 || p->n_out < 32 || p->n_red < 64) return false;
  long long expect = 1;
  for (int d = p->n_kept - 1; d >= 0; --d) {
    if (p->kept_size[d] != 1 && p->kept_in_stride[d] != expect) return false;
    expect *= p->kept_size[d];
  }
  for (int d = p->n_reduced - 1; d >= 0; --d) {
    if (p->red_size[d] != 1 && p->red_in_stride[d] != expect) return false;
    expect *= p->red_size[d];
  }
  return true;
}

}  // namespace

extern "C" int b200_reduce_plan(B200ReduceParams* p) {
  p->splits = 1;
  p->outer = 0;
  p->per_thread = 0;
  if (p->n_red <= 512 && p->n_out >= 148 * 256 && p->n_kept >= 1 && p->n_reduced >= 1) {
    // one thread per output pays off when adjacent outputs are adjacent in memory (else the block-per-output
    // kernel reads lines at least as well)
    int inner = p->n_kept - 1;
    while (inner > 0 && p->kept_size[inner] == 1) --inner;
    if (p->kept_in_stride[inner] == 1 && p->kept_size[inner] >= 32) {
      p->per_thread = 1;
      return 0;
    }
  }
  if (is_outer_reduction(p)) {
    p->outer = 1;
    const long long col_blocks = (p->n_out + 31) / 32;
    long long s = (148 * 4 + col_blocks - 1) / col_blocks;
    const long long max_s = p->n_red / 64;
    if (s > max_s) s = max_s;
    if (s > 256) s = 256;
    p->splits = s > 1 ? (int)s : 1;
    return p->splits > 1 ? (int)(p->n_out * p->splits) : 0;
  }
  if (p->n_out < 148 * 2 && p->n_red >= 1 << 16) {
    long long s = (148 * 4) / (p->n_out > 0 ? p->n_out : 1);
    const long long max_s = p->n_red / 8192;
    if (s > max_s) s = max_s;
    if (s > 1024) s = 1024;
    if (s > 1) p->splits = (int)s;
  }
  // floats: 2 per partial + 2 (an int64 index) per partial
  return p->splits > 1 ? (int)(p->n_out * p->splits * 4) : 0;
}

extern "C" int b200_reduce(const B200ReduceParams* p, void* stream) {
  if (p->n_out <= 0) return 0;
  if (p->n_kept > B200_RED_MAX_DIMS || p->n_reduced > B200_RED_MAX_DIMS) return (int)cudaErrorInvalidValue;
  if (p->n_out > 2147483647LL) return (int)cudaErrorInvalidValue;
  cudaStream_t s = (cudaStream_t)stream;
  if (p->per_thread) {
    reduce_per_thread_kernel<<<(unsigned)((p->n_out + 255) / 256), 256, 0, s>>>(*p);
    return (int)cudaGetLastError();
  }
  if (p->outer) {
    dim3 ogrid((unsigned)((p->n_out + 31) / 32), (unsigned)p->splits);
    reduce_outer_kernel<<<ogrid, 256, 0, s>>>(*p);
    if (p->splits > 1) reduce_outer_final_kernel<<<(unsigned)((p->n_out + 127) / 128), 128, 0, s>>>(*p);
    return (int)cudaGetLastError();
  }
  const int threads = p->n_red >= 1024 ? 256 : (p->n_red >= 128 ? 128 : 32);
  dim3 grid((unsigned)p->n_out, (unsigned)p->splits);
  reduce_kernel<<<grid, threads, 0, s>>>(*p);
  if (p->splits > 1) reduce_final_kernel<<<(unsigned)((p->n_out + 127) / 128), 128, 0, s>>>(*p);
  return (int)cudaGetLastError();
}
