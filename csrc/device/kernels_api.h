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


// ---- device-side error flag -------------------------------------------------------
// Kernels with bounded waits record a non-zero code here instead of hanging.
// Returns the flag's value on the current device and clears it.
B200_API int b200_read_and_clear_error_flag(int* value);

// ---- tcgen05 GEMM ---------------------------------------------------------------------
// D[M,N] = act(alpha * A[M,K] * B[N,K]^T + bias + beta * R[M,N])   (row-major D / R)
// A and B are 16-bit (bf16/f16) or fp32 (computed as tf32); accumulation is fp32 in
// tensor memory.  "K-major" operand X: element (row,k) at X[row*ld + k];
// "MN-major": element (row,k) at X[k*ld + row].  Leading dimensions must be
// multiples of 16 bytes and base pointers 16-byte aligned.
typedef struct B200GemmParams {
  int M, N, K, batch;
  const void* A;
  const void* B;
  void* D;
  int64_t lda, ldb, ldd;                 // elements
  int64_t stride_a, stride_b, stride_d;  // batch strides, elements
  int a_mn_major, b_mn_major;
  int ab_dtype;                          // B200_BF16 / B200_F16 / B200_F32
  int d_dtype;                           // B200_BF16 / B200_F16 / B200_F32
  const void* bias;                      // optional
  int bias_dtype;                        // dtype of bias (f32 / bf16 / f16)
  int bias_per_row;                      // 0: bias[n], 1: bias[m]
  const void* residual;                  // optional, same logical shape as D
  int64_t ldr, stride_r;
  int res_dtype;
  float alpha, beta;
  int act;                               // 0 none, 1 relu, 2 gelu (erf)
  int tile_n;                            // 0 = choose automatically (32..256, multiple of 32)
  int max_ctas;                          // 0 = one per SM
} B200GemmParams;
B200_API int b200_gemm(const B200GemmParams* p, void* stream);
// Test hook: override the MN-major descriptor fields (bytes); negative = default.
B200_API void b200_gemm_debug_override(int lbo, int sbo, int kstep);

// ---- tcgen05 implicit-GEMM convolution --------------------------------------------------
// Activations are NHWC 16-bit tensors.  The kernel walks a list of filter taps; for
// each tap the A tile (128 output pixels x 64 input channels) is one tiled tensor-map
// load from a (possibly strided) view of the input, shifted by the tap's offset with
// out-of-bounds elements read as zero.  Strided convolutions use one view per input
// parity.  The same kernel serves the data gradient (input = dy, flipped weights,
// optional strided output addressing).
#define B200_CONV_MAX_TAPS 49
#define B200_CONV_MAX_MAPS 4
typedef struct B200ConvTap {
  short dh, dw;   // offset added to the tile's (h, w) origin in the tap's view
  short map;      // which input view
  short wtap;     // index of the [Cout][Cin] weight slice
} B200ConvTap;

typedef struct B200ConvView {
  const void* base;
  long long dims[4];     // {C, W, H, N} extents of the view
  long long strides[3];  // element strides of W, H, N (C is contiguous)
} B200ConvView;

typedef struct B200ConvParams {
  int N, P, Q;           // pixel grid covered by this launch (tiles are boxes of it)
  int Cin, Cout;         // Cin: channels per tap seen by the kernel (multiple of 8)
  int ab_dtype;          // B200_BF16 / B200_F16
  int num_views;
  B200ConvView views[B200_CONV_MAX_MAPS];
  int ntaps;
  B200ConvTap taps[B200_CONV_MAX_TAPS];
  // weight element (tap, n = output channel, k = input channel) lives at
  //   weight + tap*w_stride_tap + n*w_stride_n + k*w_stride_k   (elements);
  // exactly one of w_stride_n / w_stride_k is 1 (k contiguous: forward with
  // channels-last filters; n contiguous: data gradient reading the same filters).
  const void* weight;
  long long w_stride_tap, w_stride_n, w_stride_k;
  int wtaps;
  // element (n,p,q,c) of the result goes to
  //   out + n*o_sn + (p*o_mul_h + o_off_h)*o_sh + (q*o_mul_w + o_off_w)*o_sw + c
  void* out;
  int out_dtype;
  long long o_sn, o_sh, o_sw;
  int o_mul_h, o_off_h, o_mul_w, o_off_w;
  const void* scale;     // optional per-Cout fp32 multiplier (folded batch norm)
  const void* bias;      // optional per-Cout bias
  int bias_dtype;
  const void* residual;  // optional, addressed like `out`
  int res_dtype;
  int act;               // 0 none, 1 relu
  int tile_n;            // 0 = automatic
} B200ConvParams;
B200_API int b200_conv_fprop(const B200ConvParams* p, void* stream);

// Weight gradient: dw_acc[co][tap*Cin + ci] += sum over pixels dy[n,p,q,co] * x_tap[n,p,q,ci]
// (fp32, zero-initialised by the caller; CTAs that share a tile add atomically).
typedef struct B200ConvWgradParams {
  int N, P, Q;           // pixel grid of dy
  int Cin, Cout;
  int ab_dtype;
  const void* dy;        // NHWC [N,P,Q,Cout]
  long long dy_sn, dy_sh, dy_sw;
  int num_views;
  B200ConvView views[B200_CONV_MAX_MAPS];
  int ntaps;
  B200ConvTap taps[B200_CONV_MAX_TAPS];  // wtap = destination tap slot
  float* dw_acc;         // [Cout][wtaps*Cin]
  int wtaps;
  int splits;            // 0 = automatic
} B200ConvWgradParams;
B200_API int b200_conv_wgrad(const B200ConvWgradParams* p, void* stream);

// ---- layout helpers -----------------------------------------------------------------------
// Pack an [N,C<=8,H,W] tensor with arbitrary element strides into a zero-bordered
// NHWC buffer with 8 channels: out[n][h+pad_top][w+pad_left][c] (16-bit `out_dtype`),
// out dims [N][Hp][Wp][8].  Used by the first-layer convolution (C = 3).
B200_API int b200_pack_nhwc8(const void* in, int in_dtype, long long sn, long long sc, long long sh, long long sw,
                             int N, int C, int H, int W, void* out, int out_dtype, int Hp, int Wp, int pad_top,
                             int pad_left, void* stream);

#ifdef __cplusplus
}
#endif
