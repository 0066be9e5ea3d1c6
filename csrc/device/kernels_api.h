// C ABI of the sm_100a kernels (second half of libcatch_b200_device.so).
//
// All launchers take raw device pointers plus a stream and return 0 or a CUDA
// error code; none of them allocates memory (workspaces are passed in by the
// host runtime, which owns the caching allocator).
#pragma once
#include <stddef.h>
#include <stdint.h>
#include "device_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Element types (values match c10::ScalarType so the host can pass them through).
enum B200DType {
  B200_U8 = 0, B200_I8 = 1, B200_I16 = 2, B200_I32 = 3, B200_I64 = 4, B200_F16 = 5,
  B200_F32 = 6, B200_F64 = 7, B200_BOOL = 11, B200_BF16 = 15
};

// ---- element-wise ------------------------------------------------------------
enum B200EwOp {
  // copy / cast
  EW_COPY = 0,
  // binary arithmetic; ADD/SUB use scalar[0] as alpha: a + alpha*b
  EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_DIV_TRUNC, EW_DIV_FLOOR, EW_REMAINDER, EW_FMOD, EW_POW,
  EW_MAXIMUM, EW_MINIMUM, EW_ATAN2,
  // comparisons (bool result)
  EW_EQ, EW_NE, EW_LT, EW_LE, EW_GT, EW_GE,
  // logical / bitwise
  EW_LOGICAL_AND, EW_LOGICAL_OR, EW_LOGICAL_XOR, EW_BIT_AND, EW_BIT_OR, EW_BIT_XOR,
  // unary
  EW_NEG, EW_ABS, EW_SQRT, EW_RSQRT, EW_RECIPROCAL, EW_EXP, EW_LOG, EW_LOG2, EW_LOG10, EW_LOG1P, EW_EXPM1,
  EW_SIN, EW_COS, EW_TANH, EW_SIGMOID, EW_RELU, EW_GELU, EW_GELU_TANH, EW_SILU, EW_CEIL, EW_FLOOR,
  EW_ROUND, EW_TRUNC, EW_SIGN, EW_ERF, EW_ISFINITE, EW_ISNAN, EW_LOGICAL_NOT, EW_BIT_NOT,
  // unary with scalar parameters scalar[0], scalar[1]
  EW_SOFTPLUS /*beta,threshold*/, EW_LEAKY_RELU /*slope*/, EW_CLAMP /*min,max (nan = unset)*/,
  EW_THRESHOLD /*threshold,value : x<=thr ? value : x*/, EW_ELU /*alpha*/, EW_HARDSWISH, EW_HARDSIGMOID,
  EW_ADD_SCALAR /* a*scalar[1] + scalar[0] */, EW_POW_SCALAR /* a ^ scalar[0] */, EW_RPOW_SCALAR /* scalar[0]^a */,
  EW_FILL /* out = scalar[0] */,
  // backward helpers: (grad, x)
  EW_THRESHOLD_BWD /*threshold: x<=thr ? 0 : grad*/, EW_GELU_BWD, EW_GELU_TANH_BWD, EW_SIGMOID_BWD /*(grad,out)*/,
  EW_TANH_BWD /*(grad,out)*/, EW_LEAKY_RELU_BWD /*slope*/, EW_SOFTPLUS_BWD /*beta,threshold*/,
  EW_HARDTANH_BWD /*min,max*/, EW_SILU_BWD, EW_ELU_BWD,
  // ternary
  EW_WHERE /*(cond,a,b)*/, EW_ADDCMUL /*(self,t1,t2) value=scalar[0]*/, EW_ADDCDIV, EW_LERP /*(a,b,w)*/,
  EW_LERP_SCALAR /*(a,b) w=scalar[0]*/, EW_MASKED_FILL /*(self,mask) value=scalar[0]*/,
  EW_NUM_OPS
};

#define B200_EW_MAX_DIMS 8
#define B200_EW_MAX_OPERANDS 4
typedef struct B200EwDesc {
  int op;
  int ndim;                       // <= B200_EW_MAX_DIMS
  int noperands;                  // operand 0 is the output
  int contiguous;                 // 1: every operand is dense with the same linear order
  int64_t numel;
  int64_t shape[B200_EW_MAX_DIMS];
  int64_t strides[B200_EW_MAX_OPERANDS][B200_EW_MAX_DIMS];  // in elements
  void* ptr[B200_EW_MAX_OPERANDS];
  int dtype[B200_EW_MAX_OPERANDS];
  int scalar_mask;                // bit i: operand i is the host scalar scalar_operand[i]
  double scalar_operand[B200_EW_MAX_OPERANDS];
  double scalar[2];               // op parameters
  int compute;                    // 0 = float, 1 = double, 2 = int64, 3 = bool
} B200EwDesc;
B200_API int b200_elementwise(const B200EwDesc* desc, void* stream);

#ifdef __cplusplus
}
#endif
