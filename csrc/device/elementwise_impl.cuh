// Element-wise kernel family (copy/cast, arithmetic, comparisons, activations
// and their gradients, ternary ops) for arbitrary strides, broadcasting and
// mixed dtypes, with a 128-bit vectorised path for dense same-dtype operands.
//
// Replaces the reference's per-op vendor calls cnnlOpTensor / cnnlTransform /
// cnnlActivationForward/Backward / cnnlCastDataType / cnnlCopy / cnnlLogicOp...
// (torch_mlu/csrc/aten/operators/cnnl/internal/{optensor,transform,activation,
// cast,copy,logic}_internal.cpp) with one templated kernel family.
// This file is included once per compute type (see elementwise_f32.cu etc.).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <type_traits>
#include "kernels_api.h"

namespace b200ew {

template <typename C>
__device__ __forceinline__ C load_as(const void* p, int64_t i, int dt) {
  switch (dt) {
    case B200_F32: return (C) static_cast<const float*>(p)[i];
    case B200_BF16: return (C) __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    case B200_F16: return (C) __half2float(static_cast<const __half*>(p)[i]);
    case B200_F64: return (C) static_cast<const double*>(p)[i];
    case B200_I64: return (C) static_cast<const int64_t*>(p)[i];
    case B200_I32: return (C) static_cast<const int32_t*>(p)[i];
    case B200_I16: return (C) static_cast<const int16_t*>(p)[i];
    case B200_I8: return (C) static_cast<const int8_t*>(p)[i];
    case B200_U8: return (C) static_cast<const uint8_t*>(p)[i];
    case B200_BOOL: return (C)(static_cast<const uint8_t*>(p)[i] != 0);
  }
  return C(0);
}

template <typename C>
__device__ __forceinline__ void store_as(void* p, int64_t i, int dt, C v) {
  switch (dt) {
    case B200_F32: static_cast<float*>(p)[i] = (float)v; break;
    case B200_BF16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16((float)v); break;
    case B200_F16: static_cast<__half*>(p)[i] = __float2half((float)v); break;
    case B200_F64: static_cast<double*>(p)[i] = (double)v; break;
    case B200_I64: static_cast<int64_t*>(p)[i] = (int64_t)v; break;
    case B200_I32: static_cast<int32_t*>(p)[i] = (int32_t)v; break;
    case B200_I16: static_cast<int16_t*>(p)[i] = (int16_t)v; break;
    case B200_I8: static_cast<int8_t*>(p)[i] = (int8_t)v; break;
    case B200_U8: static_cast<uint8_t*>(p)[i] = (uint8_t)v; break;
    case B200_BOOL: static_cast<uint8_t*>(p)[i] = (v != C(0)) ? 1 : 0; break;
  }
}

template <typename C>
__device__ __forceinline__ C c_floor_div(C a, C b) {
  if constexpr (std::is_floating_point<C>::value) {
    return floor(a / b);
  } else {
    if (b == 0) return 0;
    C q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
    return q;
  }
}

// One switch-free body per op thanks to `if constexpr`.
template <typename C, int OP>
__device__ __forceinline__ C apply(C a, C b, C c, C s0, C s1) {
  constexpr bool F = std::is_floating_point<C>::value;
  if constexpr (OP == EW_COPY) return a;
  else if constexpr (OP == EW_ADD) return a + s0 * b;
  else if constexpr (OP == EW_SUB) return a - s0 * b;
  else if constexpr (OP == EW_MUL) return a * b;
  else if constexpr (OP == EW_DIV) { if constexpr (F) return a / b; else return b == 0 ? C(0) : a / b; }
  else if constexpr (OP == EW_DIV_TRUNC) { if constexpr (F) return trunc(a / b); else return b == 0 ? C(0) : a / b; }
  else if constexpr (OP == EW_DIV_FLOOR) return c_floor_div<C>(a, b);
  else if constexpr (OP == EW_REMAINDER) {
    if constexpr (F) { C r = fmod(a, b); if (r != 0 && ((r < 0) != (b < 0))) r += b; return r; }
    else { if (b == 0) return C(0); C r = a % b; if (r != 0 && ((r < 0) != (b < 0))) r += b; return r; }
  }
  else if constexpr (OP == EW_FMOD) { if constexpr (F) return fmod(a, b); else return b == 0 ? C(0) : a % b; }
  else if constexpr (OP == EW_POW) {
    if constexpr (F) return pow(a, b);
    else { C r = 1; C base = a; C e = b; if (e < 0) return (a == 1) ? C(1) : (a == -1 ? ((e & 1) ? C(-1) : C(1)) : C(0));
           while (e) { if (e & 1) r *= base; base *= base; e >>= 1; } return r; }
  }
  else if constexpr (OP == EW_MAXIMUM) { if constexpr (F) { if (a != a) return a; if (b != b) return b; } return a > b ? a : b; }
  else if constexpr (OP == EW_MINIMUM) { if constexpr (F) { if (a != a) return a; if (b != b) return b; } return a < b ? a : b; }
  else if constexpr (OP == EW_ATAN2) { if constexpr (F) return atan2(a, b); else return C(0); }
  else if constexpr (OP == EW_EQ) return C(a == b);
  else if constexpr (OP == EW_NE) return C(a != b);
  else if constexpr (OP == EW_LT) return C(a < b);
  else if constexpr (OP == EW_LE) return C(a <= b);
  else if constexpr (OP == EW_GT) return C(a > b);
  else if constexpr (OP == EW_GE) return C(a >= b);
  else if constexpr (OP == EW_LOGICAL_AND) return C((a != 0) && (b != 0));
  else if constexpr (OP == EW_LOGICAL_OR) return C((a != 0) || (b != 0));
  else if constexpr (OP == EW_LOGICAL_XOR) return C((a != 0) != (b != 0));
  else if constexpr (OP == EW_BIT_AND) { if constexpr (F) return C(0); else return a & b; }
  else if constexpr (OP == EW_BIT_OR) { if constexpr (F) return C(0); else return a | b; }
  else if constexpr (OP == EW_BIT_XOR) { if constexpr (F) return C(0); else return a ^ b; }
  else if constexpr (OP == EW_NEG) return -a;
  else if constexpr (OP == EW_ABS) return a < 0 ? -a : a;
  else if constexpr (OP == EW_SIGN) return C((a > 0) - (a < 0));
  else if constexpr (OP == EW_LOGICAL_NOT) return C(a == 0);
  else if constexpr (OP == EW_BIT_NOT) { if constexpr (F) return C(0); else return ~a; }
  else if constexpr (OP == EW_RELU) return a > 0 ? a : (a != a ? a : C(0));
  else if constexpr (OP == EW_FILL) return s0;
  else if constexpr (OP == EW_ADD_SCALAR) return a * s1 + s0;
  else if constexpr (OP == EW_CLAMP) {
    C r = a;
    if constexpr (F) { if (s0 == s0 && r < s0) r = s0; if (s1 == s1 && r > s1) r = s1; }
    else { if (r < s0) r = s0; if (r > s1) r = s1; }
    return r;
  }
  else if constexpr (OP == EW_THRESHOLD) return a <= s0 ? s1 : a;
  else if constexpr (OP == EW_THRESHOLD_BWD) return b <= s0 ? C(0) : a;
  else if constexpr (OP == EW_WHERE) return a != 0 ? b : c;
  else if constexpr (OP == EW_ADDCMUL) return a + s0 * b * c;
  else if constexpr (OP == EW_MASKED_FILL) return b != 0 ? s0 : a;
  else if constexpr (OP == EW_ISFINITE) { if constexpr (F) return C(isfinite(a)); else return C(1); }
  else if constexpr (OP == EW_ISNAN) return C(a != a);
  else if constexpr (OP == EW_HARDTANH_BWD) return (b <= s0 || b >= s1) ? C(0) : a;
  else if constexpr (OP == EW_LEAKY_RELU) return a > 0 ? a : a * s0;
  else if constexpr (OP == EW_LEAKY_RELU_BWD) return b > 0 ? a : a * s0;
  else if constexpr (F) {
    // Floating-point only ops.
    if constexpr (OP == EW_SQRT) return sqrt(a);
    else if constexpr (OP == EW_RSQRT) return C(1) / sqrt(a);
    else if constexpr (OP == EW_RECIPROCAL) return C(1) / a;
    else if constexpr (OP == EW_EXP) return exp(a);
    else if constexpr (OP == EW_LOG) return log(a);
    else if constexpr (OP == EW_LOG2) return log2(a);
    else if constexpr (OP == EW_LOG10) return log10(a);
    else if constexpr (OP == EW_LOG1P) return log1p(a);
    else if constexpr (OP == EW_EXPM1) return expm1(a);
    else if constexpr (OP == EW_SIN) return sin(a);
    else if constexpr (OP == EW_COS) return cos(a);
    else if constexpr (OP == EW_TANH) return tanh(a);
    else if constexpr (OP == EW_SIGMOID) return C(1) / (C(1) + exp(-a));
    else if constexpr (OP == EW_GELU) return C(0.5) * a * (C(1) + erf(a * C(0.70710678118654752440)));
    else if constexpr (OP == EW_GELU_TANH) {
      const C k = C(0.79788456080286535588), k2 = C(0.044715);
      return C(0.5) * a * (C(1) + tanh(k * (a + k2 * a * a * a)));
    }
    else if constexpr (OP == EW_SILU) return a / (C(1) + exp(-a));
    else if constexpr (OP == EW_CEIL) return ceil(a);
    else if constexpr (OP == EW_FLOOR) return floor(a);
    else if constexpr (OP == EW_ROUND) return nearbyint(a);
    else if constexpr (OP == EW_TRUNC) return trunc(a);
    else if constexpr (OP == EW_ERF) return erf(a);
    else if constexpr (OP == EW_SOFTPLUS) return (a * s0 > s1) ? a : log1p(exp(a * s0)) / s0;
    else if constexpr (OP == EW_ELU) return a > 0 ? a : s0 * expm1(a);
    else if constexpr (OP == EW_HARDSWISH) { C t = a + C(3); t = t < 0 ? C(0) : (t > 6 ? C(6) : t); return a * t / C(6); }
    else if constexpr (OP == EW_HARDSIGMOID) { C t = a + C(3); t = t < 0 ? C(0) : (t > 6 ? C(6) : t); return t / C(6); }
    else if constexpr (OP == EW_POW_SCALAR) return pow(a, s0);
    else if constexpr (OP == EW_RPOW_SCALAR) return pow(s0, a);
    else if constexpr (OP == EW_GELU_BWD) {
      const C kA = C(0.70710678118654752440), kB = C(0.39894228040143267794);
      C cdf = C(0.5) * (C(1) + erf(b * kA));
      C pdf = kB * exp(C(-0.5) * b * b);
      return a * (cdf + b * pdf);
    }
    else if constexpr (OP == EW_GELU_TANH_BWD) {
      const C k = C(0.79788456080286535588), k2 = C(0.044715);
      C x = b, x3 = x * x * x;
      C t = tanh(k * (x + k2 * x3));
      C dt = (C(1) - t * t) * k * (C(1) + C(3) * k2 * x * x);
      return a * (C(0.5) * (C(1) + t) + C(0.5) * x * dt);
    }
    else if constexpr (OP == EW_SIGMOID_BWD) return a * (C(1) - b) * b;
    else if constexpr (OP == EW_TANH_BWD) return a * (C(1) - b * b);
    else if constexpr (OP == EW_SOFTPLUS_BWD) { C z = exp(b * s0); return (b * s0 > s1) ? a : a * z / (z + C(1)); }
    else if constexpr (OP == EW_SILU_BWD) { C s = C(1) / (C(1) + exp(-b)); return a * s * (C(1) + b * (C(1) - s)); }
    else if constexpr (OP == EW_ELU_BWD) return b > 0 ? a : a * s0 * exp(b);
    else if constexpr (OP == EW_ADDCDIV) return a + s0 * b / c;
    else if constexpr (OP == EW_LERP) return (c < C(0.5)) ? a + c * (b - a) : b - (b - a) * (C(1) - c);
    else if constexpr (OP == EW_LERP_SCALAR) return (s0 < C(0.5)) ? a + s0 * (b - a) : b - (b - a) * (C(1) - s0);
    else return a;
  } else {
    if constexpr (OP == EW_ADDCDIV) return c == 0 ? a : a + s0 * b / c;
    else if constexpr (OP == EW_POW_SCALAR) return apply<C, EW_POW>(a, s0, c, s0, s1);
    else if constexpr (OP == EW_RPOW_SCALAR) return apply<C, EW_POW>(s0, a, c, s0, s1);
    else return a;
  }
}

// ------------------------------------------------------------- generic kernel
// IDX = unsigned (fast 32-bit index arithmetic, used whenever every offset fits) or
// long long.
template <typename C, int OP, typename IDX>
__global__ void __launch_bounds__(256) ew_generic(const B200EwDesc d) {
  const IDX stride_t = (IDX)gridDim.x * blockDim.x;
  const C s0 = (C)d.scalar[0], s1 = (C)d.scalar[1];
  const IDX numel = (IDX)d.numel;
  for (IDX i = (IDX)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride_t) {
    IDX off[B200_EW_MAX_OPERANDS] = {0, 0, 0, 0};
    if (d.contiguous) {
#pragma unroll
      for (int k = 0; k < B200_EW_MAX_OPERANDS; ++k) off[k] = i;
    } else {
      IDX rem = i;
      for (int dim = 0; dim < d.ndim; ++dim) {
        const IDX sz = (IDX)d.shape[dim];
        const IDX idx = rem % sz;
        rem /= sz;
#pragma unroll
        for (int k = 0; k < B200_EW_MAX_OPERANDS; ++k) off[k] += idx * (IDX)d.strides[k][dim];
      }
    }
    C v[3] = {C(0), C(0), C(0)};
#pragma unroll
    for (int k = 1; k < B200_EW_MAX_OPERANDS; ++k) {
      if (k < d.noperands) {
        v[k - 1] = (d.scalar_mask >> k) & 1 ? (C)d.scalar_operand[k] : load_as<C>(d.ptr[k], (int64_t)off[k], d.dtype[k]);
      }
    }
    store_as<C>(d.ptr[0], (int64_t)off[0], d.dtype[0], apply<C, OP>(v[0], v[1], v[2], s0, s1));
  }
}

// ---------------------------------------------------------- vectorised kernel
// Dense operands that all have storage type S (compute type float): 16-byte
// loads/stores, grid-stride over vectors, scalar tail.
template <typename S> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to(float v) { return v; }
  static __device__ __forceinline__ float from(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from(float v) { return __float2bfloat16(v); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from(float v) { return __float2half(v); }
};

template <typename S, int OP, int NIN>
__global__ void __launch_bounds__(256) ew_vec(S* __restrict__ out, const S* __restrict__ a, const S* __restrict__ b,
                                              const S* __restrict__ c, int64_t n, float s0, float s1, int scalar_mask,
                                              float sa, float sb, float sc) {
  constexpr int V = 16 / sizeof(S);
  const int64_t nvec = n / V;
  const int64_t stride_t = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t i = tid; i < nvec; i += stride_t) {
    alignas(16) S va[V], vb[V], vc[V], vo[V];
    if (NIN >= 1 && !(scalar_mask & 2)) *reinterpret_cast<uint4*>(va) = reinterpret_cast<const uint4*>(a)[i];
    if (NIN >= 2 && !(scalar_mask & 4)) *reinterpret_cast<uint4*>(vb) = reinterpret_cast<const uint4*>(b)[i];
    if (NIN >= 3 && !(scalar_mask & 8)) *reinterpret_cast<uint4*>(vc) = reinterpret_cast<const uint4*>(c)[i];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float x = NIN >= 1 ? ((scalar_mask & 2) ? sa : Cvt<S>::to(va[k])) : 0.f;
      float y = NIN >= 2 ? ((scalar_mask & 4) ? sb : Cvt<S>::to(vb[k])) : 0.f;
      float z = NIN >= 3 ? ((scalar_mask & 8) ? sc : Cvt<S>::to(vc[k])) : 0.f;
      vo[k] = Cvt<S>::from(apply<float, OP>(x, y, z, s0, s1));
    }
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<uint4*>(vo);
  }
  // tail
  for (int64_t i = nvec * V + tid; i < n; i += stride_t) {
    float x = NIN >= 1 ? ((scalar_mask & 2) ? sa : Cvt<S>::to(a[i])) : 0.f;
    float y = NIN >= 2 ? ((scalar_mask & 4) ? sb : Cvt<S>::to(b[i])) : 0.f;
    float z = NIN >= 3 ? ((scalar_mask & 8) ? sc : Cvt<S>::to(c[i])) : 0.f;
    out[i] = Cvt<S>::from(apply<float, OP>(x, y, z, s0, s1));
  }
}

// Dense cast kernel (EW_COPY between two different floating storage types).
template <typename SO, typename SI>
__global__ void __launch_bounds__(256) ew_cast(SO* __restrict__ out, const SI* __restrict__ in, int64_t n) {
  constexpr int V = 8;
  const int64_t nvec = n / V;
  const int64_t stride_t = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t i = tid; i < nvec; i += stride_t) {
    alignas(16) SI vi[V];
    alignas(16) SO vo[V];
    if constexpr (sizeof(SI) == 2) {
      *reinterpret_cast<uint4*>(vi) = reinterpret_cast<const uint4*>(in)[i];
    } else {
      reinterpret_cast<uint4*>(vi)[0] = reinterpret_cast<const uint4*>(in)[2 * i];
      reinterpret_cast<uint4*>(vi)[1] = reinterpret_cast<const uint4*>(in)[2 * i + 1];
    }
#pragma unroll
    for (int k = 0; k < V; ++k) vo[k] = Cvt<SO>::from(Cvt<SI>::to(vi[k]));
    if constexpr (sizeof(SO) == 2) {
      reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<uint4*>(vo);
    } else {
      reinterpret_cast<uint4*>(out)[2 * i] = reinterpret_cast<uint4*>(vo)[0];
      reinterpret_cast<uint4*>(out)[2 * i + 1] = reinterpret_cast<uint4*>(vo)[1];
    }
  }
  for (int64_t i = nvec * V + tid; i < n; i += stride_t) out[i] = Cvt<SO>::from(Cvt<SI>::to(in[i]));
}

inline int grid_for(int64_t work, int block) {
  int64_t g = (work + block - 1) / block;
  const int64_t cap = 148 * 16;  // enough resident CTAs to cover every SM several times
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// true when every element offset of every operand fits in 32 bits (strides are >= 0)
inline bool fits_32bit(const B200EwDesc& d) {
  if (d.numel >= 0xffffffffLL) return false;
  for (int k = 0; k < d.noperands; ++k) {
    long long span = 0;
    for (int dim = 0; dim < d.ndim; ++dim) {
      if (d.strides[k][dim] < 0) return false;
      span += (d.shape[dim] - 1) * d.strides[k][dim];
    }
    if (span >= 0xffffffffLL) return false;
  }
  return true;
}

template <typename C, int OP>
int launch_generic(const B200EwDesc& d, cudaStream_t s) {
  if (fits_32bit(d)) ew_generic<C, OP, unsigned><<<grid_for(d.numel, 256), 256, 0, s>>>(d);
  else ew_generic<C, OP, long long><<<grid_for(d.numel, 256), 256, 0, s>>>(d);
  return (int)cudaGetLastError();
}

template <typename S, int OP>
int launch_vec(const B200EwDesc& d, cudaStream_t s) {
  constexpr int V = 16 / sizeof(S);
  const int g = grid_for((d.numel + V - 1) / V, 256);
  const float s0 = (float)d.scalar[0], s1 = (float)d.scalar[1];
  const float sa = (float)d.scalar_operand[1], sb = (float)d.scalar_operand[2], sc = (float)d.scalar_operand[3];
  S* o = static_cast<S*>(d.ptr[0]);
  const S* a = static_cast<const S*>(d.ptr[1]);
  const S* b = static_cast<const S*>(d.ptr[2]);
  const S* c = static_cast<const S*>(d.ptr[3]);
  switch (d.noperands) {
    case 1: ew_vec<S, OP, 0><<<g, 256, 0, s>>>(o, a, b, c, d.numel, s0, s1, d.scalar_mask, sa, sb, sc); break;
    case 2: ew_vec<S, OP, 1><<<g, 256, 0, s>>>(o, a, b, c, d.numel, s0, s1, d.scalar_mask, sa, sb, sc); break;
    case 3: ew_vec<S, OP, 2><<<g, 256, 0, s>>>(o, a, b, c, d.numel, s0, s1, d.scalar_mask, sa, sb, sc); break;
    default: ew_vec<S, OP, 3><<<g, 256, 0, s>>>(o, a, b, c, d.numel, s0, s1, d.scalar_mask, sa, sb, sc); break;
  }
  return (int)cudaGetLastError();
}

// True when the dense vector path applies: float compute, all tensor operands
// share one floating storage type and are 16-byte aligned.
inline int vec_storage_type(const B200EwDesc& d) {
  if (!d.contiguous || d.compute != 0) return -1;
  const int dt = d.dtype[0];
  if (dt != B200_F32 && dt != B200_BF16 && dt != B200_F16) return -1;
  if (!aligned16(d.ptr[0])) return -1;
  for (int k = 1; k < d.noperands; ++k) {
    if ((d.scalar_mask >> k) & 1) continue;
    if (d.dtype[k] != dt || !aligned16(d.ptr[k])) return -1;
  }
  return dt;
}

template <typename C, int OP>
int launch_op(const B200EwDesc& d, cudaStream_t s) {
  if constexpr (std::is_same<C, float>::value) {
    switch (vec_storage_type(d)) {
      case B200_F32: return launch_vec<float, OP>(d, s);
      case B200_BF16: return launch_vec<__nv_bfloat16, OP>(d, s);
      case B200_F16: return launch_vec<__half, OP>(d, s);
      default: break;
    }
  }
  return launch_generic<C, OP>(d, s);
}

#define B200_EW_CASE(OPNAME) case OPNAME: return launch_op<C, OPNAME>(d, s);

template <typename C>
int dispatch(const B200EwDesc& d, cudaStream_t s) {
  switch (d.op) {
    B200_EW_CASE(EW_COPY) B200_EW_CASE(EW_ADD) B200_EW_CASE(EW_SUB) B200_EW_CASE(EW_MUL) B200_EW_CASE(EW_DIV)
    B200_EW_CASE(EW_DIV_TRUNC) B200_EW_CASE(EW_DIV_FLOOR) B200_EW_CASE(EW_REMAINDER) B200_EW_CASE(EW_FMOD)
    B200_EW_CASE(EW_POW) B200_EW_CASE(EW_MAXIMUM) B200_EW_CASE(EW_MINIMUM) B200_EW_CASE(EW_ATAN2)
    B200_EW_CASE(EW_EQ) B200_EW_CASE(EW_NE) B200_EW_CASE(EW_LT) B200_EW_CASE(EW_LE) B200_EW_CASE(EW_GT)
    B200_EW_CASE(EW_GE) B200_EW_CASE(EW_LOGICAL_AND) B200_EW_CASE(EW_LOGICAL_OR) B200_EW_CASE(EW_LOGICAL_XOR)
    B200_EW_CASE(EW_BIT_AND) B200_EW_CASE(EW_BIT_OR) B200_EW_CASE(EW_BIT_XOR) B200_EW_CASE(EW_NEG)
    B200_EW_CASE(EW_ABS) B200_EW_CASE(EW_SQRT) B200_EW_CASE(EW_RSQRT) B200_EW_CASE(EW_RECIPROCAL)
    B200_EW_CASE(EW_EXP) B200_EW_CASE(EW_LOG) B200_EW_CASE(EW_LOG2) B200_EW_CASE(EW_LOG10) B200_EW_CASE(EW_LOG1P)
    B200_EW_CASE(EW_EXPM1) B200_EW_CASE(EW_SIN) B200_EW_CASE(EW_COS) B200_EW_CASE(EW_TANH) B200_EW_CASE(EW_SIGMOID)
    B200_EW_CASE(EW_RELU) B200_EW_CASE(EW_GELU) B200_EW_CASE(EW_GELU_TANH) B200_EW_CASE(EW_SILU)
    B200_EW_CASE(EW_CEIL) B200_EW_CASE(EW_FLOOR) B200_EW_CASE(EW_ROUND) B200_EW_CASE(EW_TRUNC) B200_EW_CASE(EW_SIGN)
    B200_EW_CASE(EW_ERF) B200_EW_CASE(EW_ISFINITE) B200_EW_CASE(EW_ISNAN) B200_EW_CASE(EW_LOGICAL_NOT)
    B200_EW_CASE(EW_BIT_NOT) B200_EW_CASE(EW_SOFTPLUS) B200_EW_CASE(EW_LEAKY_RELU) B200_EW_CASE(EW_CLAMP)
    B200_EW_CASE(EW_THRESHOLD) B200_EW_CASE(EW_ELU) B200_EW_CASE(EW_HARDSWISH) B200_EW_CASE(EW_HARDSIGMOID)
    B200_EW_CASE(EW_ADD_SCALAR) B200_EW_CASE(EW_POW_SCALAR) B200_EW_CASE(EW_RPOW_SCALAR) B200_EW_CASE(EW_FILL)
    B200_EW_CASE(EW_THRESHOLD_BWD) B200_EW_CASE(EW_GELU_BWD) B200_EW_CASE(EW_GELU_TANH_BWD)
    B200_EW_CASE(EW_SIGMOID_BWD) B200_EW_CASE(EW_TANH_BWD) B200_EW_CASE(EW_LEAKY_RELU_BWD)
    B200_EW_CASE(EW_SOFTPLUS_BWD) B200_EW_CASE(EW_HARDTANH_BWD) B200_EW_CASE(EW_SILU_BWD) B200_EW_CASE(EW_ELU_BWD)
    B200_EW_CASE(EW_WHERE) B200_EW_CASE(EW_ADDCMUL) B200_EW_CASE(EW_ADDCDIV) B200_EW_CASE(EW_LERP)
    B200_EW_CASE(EW_LERP_SCALAR) B200_EW_CASE(EW_MASKED_FILL)
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace b200ew
