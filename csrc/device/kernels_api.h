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
  int ab_dtype;                          // B200_BF16 / B200_F16 / B200_F32 (tf32) / B200_I8 (int32 accumulate)
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
  const float* col_scale;                // optional fp32 multiplier per output column (applied after alpha)
  // Two-level batches (e.g. [batch, heads] views of [batch, seq, heads, dim] tensors): batch = outer x batch_inner and
  // matrix (o, i) of an operand starts at i * stride_x + o * stride_x2.  batch_inner == 0: one level (stride_x only).
  int batch_inner;
  int64_t stride_a2, stride_b2, stride_d2, stride_r2;
  int accumulate;                        // 1: D (fp32) += alpha * A * B, added with tensor-map reductions (no bias /
                                         // residual / activation); the K loop may then be split among CTAs
  int splits;                            // accumulate only: K splits per output tile (0 = fill the GPU once)
} B200GemmParams;
B200_API int b200_gemm(const B200GemmParams* p, void* stream);

// ---- tcgen05 implicit-GEMM convolution --------------------------------------------------
// Activations are NHWC 16-bit tensors.  The kernel walks a list of filter taps; for
// each tap the A tile (128 output pixels x 64 input channels) is one tiled tensor-map
// load from a (possibly strided) view of the input, shifted by the tap's offset with
// out-of-bounds elements read as zero.  Strided convolutions use one view per input
// parity.  The same kernel serves the data gradient (input = dy, flipped weights,
// optional strided output addressing).
#define B200_CONV_MAX_TAPS 49
#define B200_CONV_MAX_MAPS 16   // input views: one per parity of a stride up to 4 x 4
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
  int ab_dtype;          // B200_BF16 / B200_F16 / B200_I8 (signed, int32 accumulate; Cin multiple of 16)
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
  int out_dtype;         // B200_BF16 / B200_F16 / B200_F32 / B200_I8 (see out_qscale)
  long long o_sn, o_sh, o_sw;
  int o_mul_h, o_off_h, o_mul_w, o_off_w;
  const void* scale;     // optional per-Cout fp32 multiplier (folded batch norm)
  const void* bias;      // optional per-Cout bias
  int bias_dtype;
  const void* residual;  // optional, addressed like `out`
  int res_dtype;
  int act;               // 0 none, 1 relu
  int tile_n;            // 0 = automatic
  float alpha;           // accumulator multiplier applied first (0 is treated as 1)
  // Optional fp64 [2 * Cout], zeroed by the caller: the kernel adds, per output channel, the sum
  // and the sum of squares of the values it stores (16-bit outputs, Cout a multiple of 8, tile
  // widths that are multiples of 64 only) so that a following batch norm needs no statistics pass.
  double* stats;
  // out_dtype == B200_I8: the finished value (after scale / bias / residual / activation) is stored as
  // clamp(round(v * out_qscale), -127, 127), i.e. already quantized for a consumer whose input scale is out_qscale.
  float out_qscale;
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
// Stride-1 multi-tap weight gradients use the shared-window kernel (conv_wgrad_halo.cu): 0 = never, 1 = yes (default),
// 2 = yes with one N = 64 MMA per window.  A negative argument only reads the setting; returns the previous one.
B200_API int b200_conv_wgrad_halo_mode(int mode);

// ---- layout helpers -----------------------------------------------------------------------
// Pack an [N,C<=8,H,W] tensor with arbitrary element strides into a zero-bordered
// NHWC buffer with 8 channels: out[n][h+pad_top][w+pad_left][c] (16-bit `out_dtype`),
// out dims [N][Hp][Wp][8].  Used by the first-layer convolution (C = 3).
B200_API int b200_pack_nhwc8(const void* in, int in_dtype, long long sn, long long sc, long long sh, long long sw,
                             int N, int C, int H, int W, void* out, int out_dtype, int Hp, int Wp, int pad_top,
                             int pad_left, void* stream);

// ---- batch norm (channels innermost: x is [rows, C] with row pitch C) -----------------
// Statistics accumulate in fp64 (zero `sums` before the call): sums[c] = sum x,
// sums[C + c] = sum x^2.
B200_API int b200_bn_stats(const void* x, int x_dtype, long long rows, int C, double* sums, void* stream);
// mean / invstd from the sums; optionally updates running statistics
// (running = (1-momentum)*running + momentum*batch, unbiased variance).
B200_API int b200_bn_finalize(const double* sums, long long rows, int C, float eps, float momentum, float* mean,
                              float* invstd, void* running_mean, void* running_var, int running_dtype, void* stream);
// invstd from running_var (inference).
B200_API int b200_bn_invstd_from_var(const void* var, int var_dtype, int C, float eps, float* invstd, void* stream);
// y = act((x - mean) * invstd * gamma + beta + residual); mean given as fp32 or, for
// inference, in `mean_dtype`.  act: 0 none, 1 relu.
B200_API int b200_bn_apply(const void* x, int x_dtype, void* y, int y_dtype, long long rows, int C, const void* mean,
                           int mean_dtype, const float* invstd, const void* gamma, const void* beta, int param_dtype,
                           const void* residual, int res_dtype, int act, void* stream);
// Same, and with act == 1 on 16-bit activations also writes one bit per element (byte i holds elements
// 8i .. 8i+7, bit set when the output is positive) to relu_mask: the backward kernels accept that mask in
// place of the ReLU output (pass it as relu_out with dtype B200_U8) and then read 1/16 of the bytes.
B200_API int b200_bn_apply_mask(const void* x, int x_dtype, void* y, int y_dtype, long long rows, int C, const void* mean,
                                int mean_dtype, const float* invstd, const void* gamma, const void* beta, int param_dtype,
                                const void* residual, int res_dtype, int act, void* relu_mask, void* stream);
// Training-mode forward in one launch: mean / invstd are computed from the channel sums inside the kernel
// (CTA 0 stores them and updates the running statistics), then y = act((x - mean) * invstd * gamma + beta +
// residual) and, if relu_mask is given, the bit mask of the positive outputs.  x, y and residual share one dtype.
// Returns cudaErrorNotSupported (801) when the shape does not qualify for the vector kernel.
B200_API int b200_bn_apply_fused(const void* x, int dtype, void* y, long long rows, int C, const double* sums, float eps,
                                 float momentum, float* save_mean, float* save_invstd, void* running_mean, void* running_var,
                                 int running_dtype, const void* gamma, const void* beta, int param_dtype, const void* residual,
                                 int act, void* relu_mask, long long* batch_counter /* optional, += 1 */, void* stream);
// Backward reductions (fp64, zero `sums` first): sums[c] = sum dy, sums[C+c] = sum dy * xhat.
// If `relu_out` is given dy is first masked by relu_out > 0 (fused ReLU backward).
B200_API int b200_bn_backward_reduce(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* mean,
                                     int mean_dtype, const float* invstd, const void* relu_out, int relu_dtype,
                                     long long rows, int C, double* sums, void* stream);
// dx = gamma*invstd*(dy - sum_dy/rows - xhat*sum_dy_xhat/rows) (training) or gamma*invstd*dy (eval);
// writes dgamma / dbeta (fp32) when non-null; `dres` (optional, same dtype as dy) receives the relu-masked dy,
// i.e. the gradient of a residual input that was added before the fused ReLU.
B200_API int b200_bn_backward_apply(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* mean,
                                    int mean_dtype, const float* invstd, const void* gamma, int param_dtype,
                                    const void* relu_out, int relu_dtype, const double* sums, long long rows, int C,
                                    int training, void* dx, int dx_dtype, float* dgamma, float* dbeta, void* dres,
                                    void* stream);

// Same; with `clear_counter` (a zeroed device word, left zeroed) the kernel also clears `sums` after every CTA
// has read them, so a persistent scratch buffer is ready for the next call without a memset launch.
B200_API int b200_bn_backward_apply2(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* mean,
                                     int mean_dtype, const float* invstd, const void* gamma, int param_dtype,
                                     const void* relu_out, int relu_dtype, double* sums, long long rows, int C,
                                     int training, void* dx, int dx_dtype, float* dgamma, float* dbeta, void* dres,
                                     unsigned* clear_counter, void* stream);

// ---- layer norm over the last dimension ---------------------------------------------------
B200_API int b200_layernorm_fwd(const void* x, int dtype, long long rows, int cols, const void* gamma, const void* beta,
                                int param_dtype, float eps, void* y, float* mean, float* rstd, void* stream);
// dx per row; dgamma/dbeta partial sums are accumulated with atomics into fp32 buffers (zeroed by caller).
B200_API int b200_layernorm_bwd(const void* dy, const void* x, int dtype, long long rows, int cols, const void* gamma,
                                int param_dtype, const float* mean, const float* rstd, void* dx, float* dgamma,
                                float* dbeta, void* stream);

// ---- pooling (generic strides, flattened h*W+w indices) -------------------------------------
typedef struct B200PoolParams {
  int N, C, H, W, P, Q;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  long long in_s[4];    // element strides of N, C, H, W
  long long out_s[4];   // element strides of N, C, P, Q
  int channels_last;    // iterate with C fastest
  int dtype;
  int count_include_pad;
  int divisor_override; // 0 = none
} B200PoolParams;
B200_API int b200_maxpool2d_fwd(const B200PoolParams* p, const void* x, void* y, long long* indices, void* stream);
B200_API int b200_maxpool2d_bwd(const B200PoolParams* p, const void* dy, const long long* indices, void* dx, void* stream);
B200_API int b200_avgpool2d_fwd(const B200PoolParams* p, const void* x, void* y, void* stream);
B200_API int b200_avgpool2d_bwd(const B200PoolParams* p, const void* dy, void* dx, void* stream);
// adaptive average pooling: windows [floor(i*H/P), ceil((i+1)*H/P))
B200_API int b200_adaptive_avgpool2d_fwd(const B200PoolParams* p, const void* x, void* y, void* stream);
B200_API int b200_adaptive_avgpool2d_bwd(const B200PoolParams* p, const void* dy, void* dx, void* stream);

// ---- pooling over three spatial dimensions (pooling3d.cu) ------------------------------------
// One parameter block for max / average / adaptive-average / adaptive-max pooling of a 5-D tensor
// (N, C, D, H, W); 2-D adaptive max pooling uses it with D = 1.  Indices are flattened (d*H + h)*W + w.
typedef struct B200Pool3Params {
  int N, C;
  int in[3], out[3];      // D, H, W and their pooled extents
  int k[3], s[3], p[3], dil[3];
  long long in_s[5];      // element strides of N, C, D, H, W
  long long out_s[5];
  int channels_last;      // iterate with C fastest
  int dtype;
  int is_max;             // 1 = max (with indices), 0 = average
  int adaptive;           // windows [floor(o*I/O), ceil((o+1)*I/O)) instead of kernel / stride / padding
  int count_include_pad;
  int divisor_override;   // 0 = none
} B200Pool3Params;
B200_API int b200_pool3d_fwd(const B200Pool3Params* p, const void* x, void* y, long long* indices /* max only */, void* stream);
B200_API int b200_pool3d_bwd(const B200Pool3Params* p, const void* dy, const long long* indices /* max only */, void* dx,
                             void* stream);

// ---- softmax / losses over contiguous rows ---------------------------------------------------
B200_API int b200_softmax_fwd(const void* x, int in_dtype, void* y, int out_dtype, long long rows, int cols, int log_mode,
                              void* stream);
// grad_in = softmax: y*(dy - sum(dy*y)) ; log_softmax: dy - exp(y)*sum(dy)
B200_API int b200_softmax_bwd(const void* dy, const void* y, int dtype, void* dx, int dx_dtype, long long rows, int cols,
                              int log_mode, void* stream);
// NLL loss on log-probabilities [rows, cols]; reduction 0 none, 1 mean, 2 sum.  `out` is fp32-computed,
// stored in `dtype`; total_weight (same dtype) receives the sum of weights of non-ignored rows.
B200_API int b200_nll_loss_fwd(const void* logp, int dtype, const long long* target, const void* weight, long long rows,
                               int cols, int reduction, long long ignore_index, void* out, void* total_weight,
                               void* stream);
B200_API int b200_nll_loss_bwd(const void* grad_out, int dtype, const long long* target, const void* weight,
                               const void* total_weight, long long rows, int cols, int reduction, long long ignore_index,
                               void* grad_in, void* stream);
// Fused softmax + cross entropy (mean reduction over non-ignored rows): writes the
// per-row loss (fp32), and d(logits) scaled by grad_scale / n_valid in `dlogits` when non-null.
B200_API int b200_softmax_xent(const void* logits, int dtype, const long long* target, long long rows, int cols,
                               long long ignore_index, float label_smoothing, float* row_loss, float* n_valid,
                               void* dlogits, int dl_dtype, float grad_scale, void* stream);

// ---- reductions ----------------------------------------------------------------------------------
enum B200ReduceOp { RED_SUM = 0, RED_MEAN, RED_PROD, RED_MAX, RED_MIN, RED_ANY, RED_ALL, RED_NORM1, RED_NORM2,
                    RED_NORM_INF, RED_ARGMAX, RED_ARGMIN, RED_SUMSQ };
#define B200_RED_MAX_DIMS 6
typedef struct B200ReduceParams {
  int op;
  int in_dtype, out_dtype;          // out for ARG* is int64
  long long n_out, n_red;
  int n_kept, n_reduced;
  long long kept_size[B200_RED_MAX_DIMS], kept_in_stride[B200_RED_MAX_DIMS];
  long long red_size[B200_RED_MAX_DIMS], red_in_stride[B200_RED_MAX_DIMS];
  const void* in;
  void* out;                        // contiguous over the kept dims (in order)
  long long* out_index;             // optional (max/min with indices); flat index along the single reduced dim
  float* workspace;                 // n_out * splits * 2 floats when splits > 1
  int splits;                       // filled by b200_reduce_plan
  int outer;                        // filled by b200_reduce_plan: sum / mean over the leading rows of a dense [rows, cols] view
  int per_thread;                   // filled by b200_reduce_plan: short reductions with many outputs, one thread per output
} B200ReduceParams;
B200_API int b200_reduce_plan(B200ReduceParams* p);   // chooses splits; returns workspace floats needed
B200_API int b200_reduce(const B200ReduceParams* p, void* stream);

// ---- fused multi-tensor optimizers ------------------------------------------------------------------
#define B200_OPT_MAX_TENSORS 48
typedef struct B200OptTensors {
  int count;
  void* param[B200_OPT_MAX_TENSORS];      // fp32 master parameters
  const void* grad[B200_OPT_MAX_TENSORS];
  void* state1[B200_OPT_MAX_TENSORS];     // momentum buffer / exp_avg
  void* state2[B200_OPT_MAX_TENSORS];     // exp_avg_sq (AdamW)
  void* lowp[B200_OPT_MAX_TENSORS];       // optional 16-bit copy of the parameter to refresh
  long long numel[B200_OPT_MAX_TENSORS];
  int grad_dtype, lowp_dtype;
} B200OptTensors;
// SGD: g = grad*grad_scale + wd*p; buf = first ? g : mu*buf + (1-dampening)*g; g = nesterov ? g + mu*buf : buf; p -= lr*g
B200_API int b200_sgd_step(const B200OptTensors* t, float lr, float momentum, float dampening, float weight_decay,
                           int nesterov, int first_step, float grad_scale, void* stream);
// AdamW (decoupled weight decay), bias corrections computed from `step`.
B200_API int b200_adamw_step(const B200OptTensors* t, float lr, float beta1, float beta2, float eps, float weight_decay,
                             long long step, float grad_scale, int adam_l2_mode, void* stream);

// ---- embedding / index ---------------------------------------------------------------------------------
B200_API int b200_embedding_fwd(const void* weight, int dtype, const long long* idx, long long n_idx, int dim,
                                long long padding_idx, void* out, void* stream);
// dweight (fp32 or same dtype, zeroed by caller) += scatter of dy rows
B200_API int b200_embedding_bwd(const void* dy, int dtype, const long long* idx, long long n_idx, int dim,
                                long long padding_idx, void* dweight, int dw_dtype, void* stream);
// out[i, :] = src[index[i], :] for a [n, row_elems] view (index_select along dim 0 of a 2-D view)
B200_API int b200_index_select_rows(const void* src, int elem_bytes, const long long* idx, long long n_idx,
                                    long long row_elems, long long n_src_rows, void* out, void* stream);

// ---- random numbers (Philox 4x32-10) ----------------------------------------------------------------------
B200_API int b200_rng_uniform(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                              double lo, double hi, void* stream);
B200_API int b200_rng_normal(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                             double mean, double std, void* stream);
B200_API int b200_rng_bernoulli(void* out, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                                double p, void* stream);
// y = x * mask / (1-p); mask is uint8 (bool)
B200_API int b200_dropout_fwd(const void* x, int dtype, long long n, unsigned long long seed, unsigned long long offset,
                              float p, void* y, unsigned char* mask, void* stream);

// dx = dy * mask * scale (mask: one byte per element)
B200_API int b200_dropout_bwd(const void* dy, const unsigned char* mask, int dtype, long long n, float scale, void* dx,
                              void* stream);
// Fused transformer residual block (fused_norm.cu): s = residual + dropout(h); y = LayerNorm(s) * gamma + beta.
// mask holds one byte per vector of four elements (bit k = element k kept); cols % 4 == 0 and
// cols <= b200_dropout_add_layernorm_max_cols().  Backward: ds (gradient of s, i.e. of the residual) and
// dh = ds * keep / (1 - p); dgamma / dbeta (fp32, zeroed by the caller) are accumulated with atomics.
B200_API int b200_dropout_add_layernorm_max_cols(void);
B200_API int b200_dropout_add_layernorm_fwd(const void* h, const void* residual, int dtype, long long rows, int cols, float p,
                                            unsigned long long seed, unsigned long long offset, const void* gamma,
                                            const void* beta, int param_dtype, float eps, void* y, void* s_out,
                                            unsigned char* mask, float* mean, float* rstd, void* stream);
B200_API int b200_dropout_add_layernorm_bwd(const void* dy, const void* s, const unsigned char* mask, int dtype, long long rows,
                                            int cols, float p, const void* gamma, int param_dtype, const float* mean,
                                            const float* rstd, void* ds, void* dh, float* dgamma, float* dbeta, void* stream);

// ---- debug dump kernel ---------------------------------------------------------------------------------------
// Prints up to `count` elements of a device tensor with device-side printf.
B200_API int b200_dump_device(const void* x, int dtype, long long count, void* stream);

// ---- collectives over peer-mapped memory (NVLink / NVSwitch) ------------------------------------
// Every rank owns an "arena" (staging bytes followed by a flag block) that all peers map
// through CUDA IPC.  Kernels signal and wait on monotonically increasing sequence numbers
// in the flag blocks with system-scope release / acquire accesses; every wait is bounded
// and reports through `status` (host-mapped): 0 ok, else B200_COMM_TIMEOUT | (peer << 8).
#define B200_COMM_MAX_RANKS 16
#define B200_COMM_TIMEOUT 1
#define B200_COMM_FLAG_BYTES 4096
#define B200_COMM_COUNTER_SLOT 64   // 64-bit slot of the flag block that counts CTAs arriving at the end barrier
typedef struct B200CommCtx {
  int rank, world;
  void* arena[B200_COMM_MAX_RANKS];                 // peer staging bases (arena[rank] is local)
  unsigned long long* flags[B200_COMM_MAX_RANKS];   // peer flag blocks: ready[16], done[16], p2p ready[16], p2p done[16], counter
  int* status;                                      // host-mapped status word
  unsigned long long timeout_ns;                    // wait limit (0 = 10 s)
  void* mc;                                         // multicast address of the arena (null without NVLS): a
                                                    // multimem access at mc + off reaches arena[r] + off on every rank
} B200CommCtx;
enum B200CommOp { COMM_SUM = 0, COMM_PROD = 1, COMM_MIN = 2, COMM_MAX = 3, COMM_AVG = 4 };

// In-place all-reduce of `n` elements of `dtype` stored at arena + offset on every rank
// (two-shot: each rank reduces one shard reading all peers, then writes the result to all
// peers).  result = op(...) * scale.  `no_signal` (tests only) skips this rank's "ready"
// signal so peers run into their bounded wait.
B200_API int b200_comm_allreduce(const B200CommCtx* ctx, size_t offset, long long n, int dtype, int op, float scale,
                                 unsigned long long seq, int no_signal, void* stream);
// Fused DDP step for one gradient bucket: reduce-scatter of the gradients in the arena
// (dtype grad_dtype) * scale, SGD-momentum / AdamW update of this rank's shard of the
// fp32 master parameters (which live in every rank's arena at param_offset), then the
// updated shard is written to every peer's parameter region (all-gather of parameters
// instead of gradients).  state1/state2 are this rank's local optimizer-state shards.
typedef struct B200FusedOptArgs {
  int kind;                  // 0 = SGD momentum, 1 = AdamW
  float lr, momentum, dampening, weight_decay, beta1, beta2, eps, bc1, bc2_sqrt;
  int nesterov, first_step;
  float* state1;             // momentum / exp_avg shard (shard_elems floats)
  float* state2;             // exp_avg_sq shard
  size_t lowp_offset;        // optional 16-bit parameter copy region in the arena (0 = none)
  int lowp_dtype;
  float* cast_src;           // optional: this rank's local fp32 gradients; the kernel converts them into the
                             // grad_dtype exchange region at grad_offset before the ranks exchange anything
  int zero_grads;            // clear the gradients for the next backward pass (cast_src if given, else the
                             // exchange region once every peer has finished reading it)
} B200FusedOptArgs;
B200_API long long b200_comm_shard_elems(long long n, int world, int dtype);
B200_API long long b200_comm_nvls_min_bytes(void);  // messages at least this large use multimem when ctx->mc is set
B200_API int b200_comm_allreduce_opt(const B200CommCtx* ctx, size_t grad_offset, size_t param_offset, long long n,
                                     int grad_dtype, float scale, const B200FusedOptArgs* opt, unsigned long long seq,
                                     void* stream);
// out[i - e0] = op over ranks of the element i of the message at arena + offset, for i in [e0, e1)
// (`out` is local memory).  Every rank of the group must call it, ranks with e0 >= e1 only synchronise.
B200_API int b200_comm_reduce_range(const B200CommCtx* ctx, size_t offset, long long e0, long long e1, void* out,
                                    int dtype, int op, unsigned long long seq, void* stream);
// Building blocks for broadcast / all-gather / reduce / send / recv.
B200_API int b200_comm_signal(const B200CommCtx* ctx, int which /*0 ready, 1 done, 2 p2p ready, 3 p2p done*/, int peer /*-1 = all*/,
                              unsigned long long seq, void* stream);
B200_API int b200_comm_wait(const B200CommCtx* ctx, int which, int peer /*-1 = all*/, unsigned long long seq,
                            void* stream);
B200_API int b200_comm_copy(void* dst, const void* src, size_t bytes, void* stream);
// dst[i] = op(dst[i], src[i]) for n elements (used by reduce / reduce_scatter pulls)
B200_API int b200_comm_accumulate(void* dst, const void* src, long long n, int dtype, int op, void* stream);

// ---- int8 quantisation -------------------------------------------------------------------------
// q[i] = clamp(round_half_even(x[i] * scale), -127, 127) as int8 (per-tensor scale)
B200_API int b200_quantize_int8(const void* x, int x_dtype, long long n, float scale, void* q, void* stream);
// per-row (output-channel) symmetric weight quantisation of a dense [rows, cols] matrix:
// scale[r] = 127 / max|w[r, :]| (1 if the row is all zero), q = round(w * scale[r])
B200_API int b200_quantize_int8_rows(const void* w, int w_dtype, long long rows, long long cols, void* q, float* scale,
                                     void* stream);
// abs-max of a tensor into *out (fp32, must be zero-initialised; uses an atomic max on the bit pattern)
B200_API int b200_absmax(const void* x, int x_dtype, long long n, float* out, void* stream);

// ---- indexing, sorting, resampling, NMS, depthwise convolution (indexing.cu) ------------
// Gather / scatter along dimension `dim`.  `sizes` is the shape of the (contiguous) index tensor;
// a = the indexed tensor, b = the tensor shaped like the index, both addressed with element strides.
// mode 0: b[i] = a[index[i]]; 1: a[index[i]] = b[i]; 2: a[index[i]] += b[i] (fp32).  An index out of
// range sets *bad_flag (device int) and is skipped.
B200_API int b200_dim_index(void* a, void* b, int elem_bytes, const long long* index, int ndim, int dim,
                            const long long* sizes, const long long* a_strides, const long long* b_strides,
                            long long dim_size, int mode, int* bad_flag, void* stream);
// out[o][n][:] = src[o][idx[n]][:] for src of shape [outer][n_src][row_bytes]
B200_API int b200_take_rows(const void* src, const long long* idx, long long outer, long long n_src, long long n_idx,
                            long long row_bytes, void* out, int* bad_flag, void* stream);
// dst[o][idx[n]][:] = (or += for fp32 when accumulate) values[o][n][:]
B200_API int b200_put_rows(void* dst, const long long* idx, long long outer, long long n_dst, long long n_idx,
                           long long row_elems, int elem_bytes, const void* values, int accumulate, int* bad_flag,
                           void* stream);
// nonzero in two passes over a contiguous tensor of n elements; workspace holds
// b200_nonzero_workspace_elems(n) int64 values, the last of which receives the count after pass 1.
B200_API long long b200_nonzero_workspace_elems(long long n);
B200_API int b200_nonzero_count(const void* x, int elem_bytes, int is_float, long long n, long long* workspace, void* stream);
B200_API int b200_nonzero_write(const void* x, int elem_bytes, int is_float, long long n, const long long* workspace,
                                int ndim, const long long* sizes, long long* out, void* stream);
B200_API int b200_arange(void* out, int dtype, long long n, double start, double step, void* stream);
B200_API int b200_tri(const void* in, void* out, int elem_bytes, long long batch, long long rows, long long cols,
                      long long k, int upper, void* stream);
B200_API int b200_sort_rows_max_len(void);
B200_API int b200_sort_rows(const void* x, int dtype, int elem_bytes, long long rows, int len, int descending, int k,
                            void* values, long long* indices, void* stream);
// Rows of any length and any orderable dtype (sort_scan.cu): `workspace` holds b200_sort_long_workspace_bytes
// bytes; values / indices may be null; equal keys keep their order; NaN sorts as the largest value.
B200_API long long b200_sort_long_workspace_bytes(long long rows, long long len);
B200_API int b200_sort_long(const void* x, int dtype, int elem_bytes, long long rows, long long len, int descending,
                            long long k, void* values, long long* indices, void* workspace, void* stream);
// out[i] = in[0] + ... + in[i] over int64; workspace: b200_scan_workspace_elems(n) int64 values
B200_API long long b200_scan_workspace_elems(long long n);
B200_API int b200_inclusive_scan_i64(const long long* in, long long* out, long long n, long long* workspace, void* stream);
// dst[o][idx[j]][:] = fill for dst of shape [outer][n_dst][inner] (elements of elem_bytes <= 8 bytes, value given as
// its bit pattern); an index out of range sets *bad_flag and is skipped
B200_API int b200_index_fill(void* dst, int elem_bytes, const long long* idx, long long outer, long long n_dst,
                             long long n_idx, long long inner, unsigned long long fill_bits, int* bad_flag, void* stream);
// mode 0 nearest, 1 bilinear; backward: `out` holds the output gradient and the input gradient is
// accumulated into in_acc (zeroed fp32, contiguous NCHW).  sizes = {N, C, H, W, OH, OW}.
B200_API int b200_resample2d(const void* in, void* out, int dtype, const long long* sizes, const long long* in_strides,
                             const long long* out_strides, double scale_h, double scale_w, int align_corners, int mode,
                             int backward, float* in_acc, void* stream);
// boxes (x1, y1, x2, y2) fp32 sorted by descending score; mask is [n][ceil(n/64)] words
B200_API int b200_nms_mask(const float* sorted_boxes, int n, float iou_threshold, unsigned long long* mask, void* stream);
// dims = {N, C, H, W, K, P, Q}; conv = {R, S, stride_h, stride_w, pad_h, pad_w}; weight contiguous [K][1][R][S].
// pass 0: y = conv(x, w).  pass 1: x is the input-gradient buffer to fill, y the output gradient.
// pass 2: w is the fp32 [K][R][S] weight-gradient buffer to fill, y the output gradient, x the input.
B200_API int b200_depthwise_conv(int pass, const void* x, const void* w, void* y, int dtype, const long long* dims,
                                 const int* conv, const long long* x_strides, const long long* y_strides, void* stream);

#ifdef __cplusplus
}
#endif
