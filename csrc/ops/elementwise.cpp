// Element-wise operators of the b200 device: arithmetic with broadcasting and
// type promotion, comparisons, logical / bitwise ops, unary math, activations
// and their gradients, fill / where / masked_fill / addcmul / addcdiv / lerp.
//
// Parity: torch_mlu/csrc/aten/operators/cnnl/{add,sub,mul,div,activation,logic,
// abs,ceil,floor,round,exp,log,neg,sqrt,reciprocal,pow,clamp,remainder,max,min,
// bitwise_operator,isfinite,fill,masked_fill}.cpp.  Shape / dtype semantics come
// from at::TensorIterator (the reference also routes add/sub/mul/div through
// the TensorIterator, add.cpp:49-93); the math runs in the element-wise kernel
// family of the device layer.
#include <ATen/native/TensorIterator.h>
#include <ATen/ScalarOps.h>
#include <cmath>
#include <limits>

#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Scalar;
using at::Tensor;
using at::TensorIterator;

void run(TensorIterator& iter, int op, double s0 = 0, double s1 = 0,
         std::optional<at::ScalarType> compute = std::nullopt) {
  OpScope scope("elementwise", iter.device(0).index());
  launch_ew(iter, op, s0, s1, scope.stream(), compute);
}

enum class Kind { Plain, Float, Compare };

TensorIterator make_binary(const Tensor& out, const Tensor& a, const Tensor& b, Kind k) {
  switch (k) {
    case Kind::Float: return TensorIterator::binary_float_op(const_cast<Tensor&>(out), a, b);
    case Kind::Compare: return TensorIterator::comparison_op(const_cast<Tensor&>(out), a, b);
    default: return TensorIterator::binary_op(const_cast<Tensor&>(out), a, b);
  }
}

Tensor binary(const Tensor& a, const Tensor& b, int op, Kind k, double s0 = 1.0) {
  Tensor out;
  auto iter = make_binary(out, a, b, k);
  run(iter, op, s0);
  return iter.output();
}
Tensor& binary_(Tensor& a, const Tensor& b, int op, Kind k, double s0 = 1.0) {
  auto iter = make_binary(a, a, b, k);
  run(iter, op, s0);
  return a;
}
Tensor& binary_out(const Tensor& a, const Tensor& b, Tensor& out, int op, Kind k, double s0 = 1.0) {
  auto iter = make_binary(out, a, b, k);
  run(iter, op, s0);
  return out;
}

Tensor wrap(const Scalar& s) { return at::native::wrapped_scalar_tensor(s); }

TensorIterator make_unary(const Tensor& out, const Tensor& a, bool float_op) {
  return float_op ? TensorIterator::unary_float_op(const_cast<Tensor&>(out), a)
                  : TensorIterator::unary_op(const_cast<Tensor&>(out), a);
}
Tensor unary(const Tensor& a, int op, bool float_op, double s0 = 0, double s1 = 0) {
  Tensor out;
  auto iter = make_unary(out, a, float_op);
  run(iter, op, s0, s1);
  return iter.output();
}
Tensor& unary_(Tensor& a, int op, bool float_op, double s0 = 0, double s1 = 0) {
  auto iter = make_unary(a, a, float_op);
  run(iter, op, s0, s1);
  return a;
}
Tensor& unary_out(const Tensor& a, Tensor& out, int op, bool float_op, double s0 = 0, double s1 = 0) {
  auto iter = make_unary(out, a, float_op);
  run(iter, op, s0, s1);
  return out;
}
// bool-valued unary (isnan, logical_not ...)
Tensor unary_bool(const Tensor& a, int op) {
  Tensor out = empty_b200(a.sizes(), at::kBool, a.device().index());
  auto iter = at::TensorIteratorConfig().add_output(out).add_const_input(a).check_all_same_dtype(false).build();
  run(iter, op, 0, 0, a.scalar_type());
  return out;
}

constexpr double kNaN = std::numeric_limits<double>::quiet_NaN();

// ----------------------------------------------------------------------- macros
#define B200_BINARY(NAME, OP, KIND)                                                                   \
  Tensor NAME##_tensor(const Tensor& a, const Tensor& b) { return binary(a, b, OP, KIND); }           \
  Tensor& NAME##_tensor_(Tensor& a, const Tensor& b) { return binary_(a, b, OP, KIND); }              \
  Tensor& NAME##_out(const Tensor& a, const Tensor& b, Tensor& out) { return binary_out(a, b, out, OP, KIND); }

#define B200_COMPARE(NAME, OP)                                                                              \
  B200_BINARY(NAME, OP, Kind::Compare)                                                                      \
  Tensor NAME##_scalar(const Tensor& a, const Scalar& b) { return binary(a, wrap(b), OP, Kind::Compare); }  \
  Tensor& NAME##_scalar_(Tensor& a, const Scalar& b) { return binary_(a, wrap(b), OP, Kind::Compare); }     \
  Tensor& NAME##_scalar_out(const Tensor& a, const Scalar& b, Tensor& out) {                                \
    return binary_out(a, wrap(b), out, OP, Kind::Compare);                                                  \
  }

#define B200_UNARY(NAME, OP, FLOAT)                                                          \
  Tensor NAME(const Tensor& a) { return unary(a, OP, FLOAT); }                               \
  Tensor& NAME##_(Tensor& a) { return unary_(a, OP, FLOAT); }                                \
  Tensor& NAME##_out(const Tensor& a, Tensor& out) { return unary_out(a, out, OP, FLOAT); }

// add / sub carry alpha
Tensor add_tensor(const Tensor& a, const Tensor& b, const Scalar& alpha) {
  return binary(a, b, EW_ADD, Kind::Plain, alpha.toDouble());
}
Tensor& add_tensor_(Tensor& a, const Tensor& b, const Scalar& alpha) {
  return binary_(a, b, EW_ADD, Kind::Plain, alpha.toDouble());
}
Tensor& add_out(const Tensor& a, const Tensor& b, const Scalar& alpha, Tensor& out) {
  return binary_out(a, b, out, EW_ADD, Kind::Plain, alpha.toDouble());
}
Tensor sub_tensor(const Tensor& a, const Tensor& b, const Scalar& alpha) {
  return binary(a, b, EW_SUB, Kind::Plain, alpha.toDouble());
}
Tensor& sub_tensor_(Tensor& a, const Tensor& b, const Scalar& alpha) {
  return binary_(a, b, EW_SUB, Kind::Plain, alpha.toDouble());
}
Tensor& sub_out(const Tensor& a, const Tensor& b, const Scalar& alpha, Tensor& out) {
  return binary_out(a, b, out, EW_SUB, Kind::Plain, alpha.toDouble());
}
Tensor rsub_tensor(const Tensor& a, const Tensor& b, const Scalar& alpha) {
  return binary(b, a, EW_SUB, Kind::Plain, alpha.toDouble());
}

B200_BINARY(mul, EW_MUL, Kind::Plain)
B200_BINARY(div, EW_DIV, Kind::Float)
B200_BINARY(maximum, EW_MAXIMUM, Kind::Plain)
B200_BINARY(minimum, EW_MINIMUM, Kind::Plain)
B200_BINARY(remainder, EW_REMAINDER, Kind::Plain)
B200_BINARY(fmod, EW_FMOD, Kind::Plain)
B200_BINARY(pow_tt, EW_POW, Kind::Plain)
B200_BINARY(atan2, EW_ATAN2, Kind::Float)
B200_BINARY(logical_and, EW_LOGICAL_AND, Kind::Compare)
B200_BINARY(logical_or, EW_LOGICAL_OR, Kind::Compare)
B200_BINARY(logical_xor, EW_LOGICAL_XOR, Kind::Compare)
B200_BINARY(bitwise_and, EW_BIT_AND, Kind::Plain)
B200_BINARY(bitwise_or, EW_BIT_OR, Kind::Plain)
B200_BINARY(bitwise_xor, EW_BIT_XOR, Kind::Plain)
B200_COMPARE(eq, EW_EQ)
B200_COMPARE(ne, EW_NE)
B200_COMPARE(lt, EW_LT)
B200_COMPARE(le, EW_LE)
B200_COMPARE(gt, EW_GT)
B200_COMPARE(ge, EW_GE)

int div_mode_op(std::optional<c10::string_view> mode, Kind* k) {
  *k = Kind::Float;
  if (!mode.has_value()) return EW_DIV;
  *k = Kind::Plain;
  if (*mode == "trunc") return EW_DIV_TRUNC;
  if (*mode == "floor") return EW_DIV_FLOOR;
  TORCH_CHECK(false, "div expected rounding_mode to be one of None, 'trunc', or 'floor' but found '", *mode, "'");
}
Tensor div_mode(const Tensor& a, const Tensor& b, std::optional<c10::string_view> mode) {
  Kind k;
  int op = div_mode_op(mode, &k);
  return binary(a, b, op, k);
}
Tensor& div_mode_(Tensor& a, const Tensor& b, std::optional<c10::string_view> mode) {
  Kind k;
  int op = div_mode_op(mode, &k);
  return binary_(a, b, op, k);
}
Tensor& div_mode_out(const Tensor& a, const Tensor& b, std::optional<c10::string_view> mode, Tensor& out) {
  Kind k;
  int op = div_mode_op(mode, &k);
  return binary_out(a, b, out, op, k);
}

B200_UNARY(neg, EW_NEG, false)
B200_UNARY(abs, EW_ABS, false)
B200_UNARY(sqrt, EW_SQRT, true)
B200_UNARY(rsqrt, EW_RSQRT, true)
B200_UNARY(reciprocal, EW_RECIPROCAL, true)
B200_UNARY(exp, EW_EXP, true)
B200_UNARY(log, EW_LOG, true)
B200_UNARY(log2, EW_LOG2, true)
B200_UNARY(log10, EW_LOG10, true)
B200_UNARY(log1p, EW_LOG1P, true)
B200_UNARY(expm1, EW_EXPM1, true)
B200_UNARY(sin, EW_SIN, true)
B200_UNARY(cos, EW_COS, true)
B200_UNARY(tanh, EW_TANH, true)
B200_UNARY(sigmoid, EW_SIGMOID, true)
B200_UNARY(relu, EW_RELU, false)
B200_UNARY(silu, EW_SILU, true)
B200_UNARY(ceil, EW_CEIL, false)
B200_UNARY(floor, EW_FLOOR, false)
B200_UNARY(round, EW_ROUND, false)
B200_UNARY(trunc, EW_TRUNC, false)
B200_UNARY(sign, EW_SIGN, false)
B200_UNARY(sgn, EW_SIGN, false)  // real types only: identical to sign
B200_UNARY(erf, EW_ERF, true)
B200_UNARY(bitwise_not, EW_BIT_NOT, false)
B200_UNARY(hardswish, EW_HARDSWISH, true)
B200_UNARY(hardsigmoid, EW_HARDSIGMOID, true)

Tensor isnan(const Tensor& a) { return unary_bool(a, EW_ISNAN); }
Tensor logical_not(const Tensor& a) { return unary_bool(a, EW_LOGICAL_NOT); }
Tensor& logical_not_out(const Tensor& a, Tensor& out) {
  auto iter = at::TensorIteratorConfig().add_output(out).add_const_input(a).check_all_same_dtype(false).build();
  run(iter, EW_LOGICAL_NOT, 0, 0, a.scalar_type());
  return out;
}

// gelu(approximate)
int gelu_op(c10::string_view approx, bool bwd) {
  if (approx == "tanh") return bwd ? EW_GELU_TANH_BWD : EW_GELU_TANH;
  return bwd ? EW_GELU_BWD : EW_GELU;
}
Tensor gelu(const Tensor& a, c10::string_view approx) { return unary(a, gelu_op(approx, false), true); }
Tensor& gelu_(Tensor& a, c10::string_view approx) { return unary_(a, gelu_op(approx, false), true); }
Tensor& gelu_out(const Tensor& a, c10::string_view approx, Tensor& out) {
  return unary_out(a, out, gelu_op(approx, false), true);
}
Tensor gelu_backward(const Tensor& grad, const Tensor& self, c10::string_view approx) {
  return binary(grad, self, gelu_op(approx, true), Kind::Plain);
}

// parametrised activations
Tensor leaky_relu(const Tensor& a, const Scalar& slope) { return unary(a, EW_LEAKY_RELU, false, slope.toDouble()); }
Tensor& leaky_relu_(Tensor& a, const Scalar& slope) { return unary_(a, EW_LEAKY_RELU, false, slope.toDouble()); }
Tensor leaky_relu_backward(const Tensor& grad, const Tensor& self, const Scalar& slope, bool) {
  return binary(grad, self, EW_LEAKY_RELU_BWD, Kind::Plain, slope.toDouble());
}
Tensor softplus(const Tensor& a, const Scalar& beta, const Scalar& thr) {
  return unary(a, EW_SOFTPLUS, true, beta.toDouble(), thr.toDouble());
}
Tensor softplus_backward(const Tensor& grad, const Tensor& self, const Scalar& beta, const Scalar& thr) {
  Tensor out;
  auto iter = TensorIterator::binary_op(out, grad, self);
  run(iter, EW_SOFTPLUS_BWD, beta.toDouble(), thr.toDouble());
  return iter.output();
}
Tensor threshold(const Tensor& a, const Scalar& thr, const Scalar& value) {
  return unary(a, EW_THRESHOLD, false, thr.toDouble(), value.toDouble());
}
Tensor& threshold_(Tensor& a, const Scalar& thr, const Scalar& value) {
  return unary_(a, EW_THRESHOLD, false, thr.toDouble(), value.toDouble());
}
Tensor threshold_backward(const Tensor& grad, const Tensor& self, const Scalar& thr) {
  return binary(grad, self, EW_THRESHOLD_BWD, Kind::Plain, thr.toDouble());
}
Tensor hardtanh(const Tensor& a, const Scalar& lo, const Scalar& hi) {
  return unary(a, EW_CLAMP, false, lo.toDouble(), hi.toDouble());
}
Tensor& hardtanh_(Tensor& a, const Scalar& lo, const Scalar& hi) {
  return unary_(a, EW_CLAMP, false, lo.toDouble(), hi.toDouble());
}
Tensor hardtanh_backward(const Tensor& grad, const Tensor& self, const Scalar& lo, const Scalar& hi) {
  Tensor out;
  auto iter = TensorIterator::binary_op(out, grad, self);
  run(iter, EW_HARDTANH_BWD, lo.toDouble(), hi.toDouble());
  return iter.output();
}
Tensor elu_any(const Tensor& a, const Scalar& alpha, const Scalar& scale, const Scalar& input_scale) {
  if (scale.toDouble() == 1.0 && input_scale.toDouble() == 1.0) return unary(a, EW_ELU, true, alpha.toDouble());
  // selu / celu: scale * (x > 0 ? x : alpha * (exp(x * input_scale) - 1)), from element-wise device kernels, in fp32
  TORCH_CHECK(a.scalar_type() == at::kFloat || a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf,
              "b200 elu: unsupported dtype ", a.scalar_type());
  Tensor x = a.scalar_type() == at::kFloat ? a : a.to(at::kFloat);
  Tensor neg = at::sub(at::exp(at::mul(x, input_scale)), Scalar(1.0)).mul_(Scalar(alpha.toDouble() * scale.toDouble()));
  Tensor r = at::where(at::gt(x, Scalar(0.0)), at::mul(x, scale), neg);
  return r.scalar_type() == a.scalar_type() ? r : r.to(a.scalar_type());
}
Tensor& elu_(Tensor& a, const Scalar& alpha, const Scalar& scale, const Scalar& input_scale) {
  a.copy_(elu_any(a, alpha, scale, input_scale));
  return a;
}
Tensor sigmoid_backward(const Tensor& grad, const Tensor& out) { return binary(grad, out, EW_SIGMOID_BWD, Kind::Plain); }
Tensor tanh_backward(const Tensor& grad, const Tensor& out) { return binary(grad, out, EW_TANH_BWD, Kind::Plain); }
Tensor silu_backward(const Tensor& grad, const Tensor& self) { return binary(grad, self, EW_SILU_BWD, Kind::Plain); }

double lim(const std::optional<Scalar>& s, const Tensor& a, bool lower) {
  if (s.has_value()) return s->toDouble();
  if (c10::isFloatingType(a.scalar_type())) return kNaN;
  return lower ? -9.2e18 : 9.2e18;
}
Tensor clamp(const Tensor& a, const std::optional<Scalar>& lo, const std::optional<Scalar>& hi) {
  TORCH_CHECK(lo.has_value() || hi.has_value(), "torch.clamp: At least one of 'min' or 'max' must not be None");
  return unary(a, EW_CLAMP, false, lim(lo, a, true), lim(hi, a, false));
}
Tensor& clamp_(Tensor& a, const std::optional<Scalar>& lo, const std::optional<Scalar>& hi) {
  TORCH_CHECK(lo.has_value() || hi.has_value(), "torch.clamp: At least one of 'min' or 'max' must not be None");
  return unary_(a, EW_CLAMP, false, lim(lo, a, true), lim(hi, a, false));
}
Tensor& clamp_out(const Tensor& a, const std::optional<Scalar>& lo, const std::optional<Scalar>& hi, Tensor& out) {
  return unary_out(a, out, EW_CLAMP, false, lim(lo, a, true), lim(hi, a, false));
}
Tensor clamp_min(const Tensor& a, const Scalar& lo) { return unary(a, EW_CLAMP, false, lo.toDouble(), lim({}, a, false)); }
Tensor& clamp_min_(Tensor& a, const Scalar& lo) { return unary_(a, EW_CLAMP, false, lo.toDouble(), lim({}, a, false)); }
Tensor clamp_max(const Tensor& a, const Scalar& hi) { return unary(a, EW_CLAMP, false, lim({}, a, true), hi.toDouble()); }
Tensor& clamp_max_(Tensor& a, const Scalar& hi) { return unary_(a, EW_CLAMP, false, lim({}, a, true), hi.toDouble()); }

Tensor pow_tensor_scalar(const Tensor& a, const Scalar& e) {
  // integer tensors with a float exponent promote to float
  Tensor out;
  auto iter = TensorIterator::binary_op(out, a, wrap(e));
  run(iter, EW_POW);
  return iter.output();
}
Tensor& pow_tensor_scalar_out(const Tensor& a, const Scalar& e, Tensor& out) {
  auto iter = TensorIterator::binary_op(out, a, wrap(e));
  run(iter, EW_POW);
  return out;
}
Tensor pow_scalar_tensor(const Scalar& b, const Tensor& e) {
  Tensor out;
  auto iter = TensorIterator::binary_op(out, wrap(b).to(e.device()), e);
  run(iter, EW_POW);
  return iter.output();
}

// fill / zero
Tensor& fill_scalar_(Tensor& self, const Scalar& v) {
  if (self.numel() == 0) return self;
  OpScope scope("fill_", self);
  const double val = v.isBoolean() ? double(v.toBool()) : v.toDouble();
  if (val == 0.0 && self.is_non_overlapping_and_dense()) {
    backend().memset_async(self.data_ptr(), 0, self.nbytes(), scope.stream());
    return self;
  }
  launch_fill(self, val, scope.stream());
  return self;
}
Tensor& fill_tensor_(Tensor& self, const Tensor& v) {
  TORCH_CHECK(v.dim() == 0, "fill_ only supports 0-dimension value tensor but got tensor with ", v.dim(), " dimensions.");
  return fill_scalar_(self, v.item());
}
Tensor& zero_(Tensor& self) { return fill_scalar_(self, 0); }

// ternary
Tensor where_self(const Tensor& cond, const Tensor& a, const Tensor& b) {
  TORCH_CHECK(cond.scalar_type() == at::kBool || cond.scalar_type() == at::kByte, "where expected condition to be a boolean tensor");
  at::ScalarType rt = at::result_type(a, b);
  Tensor a2 = a.scalar_type() == rt ? a : a.to(rt);
  Tensor b2 = b.scalar_type() == rt ? b : b.to(rt);
  if (!is_b200(a2)) a2 = a2.to(cond.device());
  if (!is_b200(b2)) b2 = b2.to(cond.device());
  auto shape = at::infer_size(at::infer_size(cond.sizes(), a2.sizes()), b2.sizes());
  Tensor out = empty_b200(shape, rt, cond.device().index());
  auto iter = at::TensorIteratorConfig()
                  .check_all_same_dtype(false)
                  .resize_outputs(false)
                  .add_output(out)
                  .add_const_input(cond)
                  .add_const_input(a2)
                  .add_const_input(b2)
                  .build();
  run(iter, EW_WHERE, 0, 0, rt);
  return out;
}
Tensor& masked_fill_scalar_(Tensor& self, const Tensor& mask, const Scalar& value) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ", mask.scalar_type());
  auto iter = at::TensorIteratorConfig()
                  .set_check_mem_overlap(false)
                  .check_all_same_dtype(false)
                  .resize_outputs(false)
                  .add_output(self)
                  .add_const_input(self)
                  .add_const_input(mask)
                  .build();
  run(iter, EW_MASKED_FILL, value.isBoolean() ? double(value.toBool()) : value.toDouble(), 0, self.scalar_type());
  return self;
}
Tensor& masked_fill_tensor_(Tensor& self, const Tensor& mask, const Tensor& value) {
  TORCH_CHECK(value.dim() == 0, "masked_fill_ only supports a 0-dimensional value tensor");
  return masked_fill_scalar_(self, mask, value.item());
}
Tensor& addc_impl(const Tensor& self, const Tensor& t1, const Tensor& t2, const Scalar& value, Tensor& out, int op) {
  auto iter = at::TensorIteratorConfig()
                  .set_check_mem_overlap(false)
                  .promote_inputs_to_common_dtype(true)
                  .cast_common_dtype_to_outputs(true)
                  .enforce_safe_casting_to_output(true)
                  .add_output(out)
                  .add_const_input(self)
                  .add_const_input(t1)
                  .add_const_input(t2)
                  .build();
  run(iter, op, value.toDouble());
  if (!out.defined()) out = iter.output();
  return out;
}
Tensor addcmul(const Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v) {
  Tensor out;
  return addc_impl(s, a, b, v, out, EW_ADDCMUL);
}
Tensor& addcmul_(Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v) { return addc_impl(s, a, b, v, s, EW_ADDCMUL); }
Tensor& addcmul_out(const Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v, Tensor& out) {
  return addc_impl(s, a, b, v, out, EW_ADDCMUL);
}
Tensor addcdiv(const Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v) {
  Tensor out;
  return addc_impl(s, a, b, v, out, EW_ADDCDIV);
}
Tensor& addcdiv_(Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v) { return addc_impl(s, a, b, v, s, EW_ADDCDIV); }
Tensor& addcdiv_out(const Tensor& s, const Tensor& a, const Tensor& b, const Scalar& v, Tensor& out) {
  return addc_impl(s, a, b, v, out, EW_ADDCDIV);
}
Tensor& lerp_scalar_(Tensor& self, const Tensor& end, const Scalar& w) {
  auto iter = TensorIterator::binary_op(self, self, end);
  run(iter, EW_LERP_SCALAR, w.toDouble());
  return self;
}
Tensor lerp_scalar(const Tensor& self, const Tensor& end, const Scalar& w) {
  Tensor out;
  auto iter = TensorIterator::binary_op(out, self, end);
  run(iter, EW_LERP_SCALAR, w.toDouble());
  return iter.output();
}

}  // namespace

#define REG3(NAME, FN)                                  \
  m.impl(#NAME ".Tensor", TORCH_FN(FN##_tensor));       \
  m.impl(#NAME "_.Tensor", TORCH_FN(FN##_tensor_));     \
  m.impl(#NAME ".out", TORCH_FN(FN##_out));
#define REG3_PLAIN(NAME, FN)                    \
  m.impl(#NAME, TORCH_FN(FN##_tensor));         \
  m.impl(#NAME "_", TORCH_FN(FN##_tensor_));    \
  m.impl(#NAME ".out", TORCH_FN(FN##_out));
#define REG_CMP(NAME)                                       \
  m.impl(#NAME ".Tensor", TORCH_FN(NAME##_tensor));         \
  m.impl(#NAME "_.Tensor", TORCH_FN(NAME##_tensor_));       \
  m.impl(#NAME ".Tensor_out", TORCH_FN(NAME##_out));        \
  m.impl(#NAME ".Scalar", TORCH_FN(NAME##_scalar));         \
  m.impl(#NAME "_.Scalar", TORCH_FN(NAME##_scalar_));       \
  m.impl(#NAME ".Scalar_out", TORCH_FN(NAME##_scalar_out));
#define REG_UNARY(NAME)                      \
  m.impl(#NAME, TORCH_FN(NAME));             \
  m.impl(#NAME "_", TORCH_FN(NAME##_));      \
  m.impl(#NAME ".out", TORCH_FN(NAME##_out));

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  if (!device_kernels_enabled()) return;
  REG3(add, add)
  REG3(sub, sub)
  m.impl("rsub.Tensor", TORCH_FN(rsub_tensor));
  REG3(mul, mul)
  REG3(div, div)
  m.impl("div.Tensor_mode", TORCH_FN(div_mode));
  m.impl("div_.Tensor_mode", TORCH_FN(div_mode_));
  m.impl("div.out_mode", TORCH_FN(div_mode_out));
  REG3_PLAIN(maximum, maximum)
  REG3_PLAIN(minimum, minimum)
  REG3(remainder, remainder)
  m.impl("remainder.Tensor_out", TORCH_FN(remainder_out));
  REG3(fmod, fmod)
  m.impl("fmod.Tensor_out", TORCH_FN(fmod_out));
  m.impl("pow.Tensor_Tensor", TORCH_FN(pow_tt_tensor));
  m.impl("pow_.Tensor", TORCH_FN(pow_tt_tensor_));
  m.impl("pow.Tensor_Tensor_out", TORCH_FN(pow_tt_out));
  m.impl("pow.Tensor_Scalar", TORCH_FN(pow_tensor_scalar));
  m.impl("pow.Tensor_Scalar_out", TORCH_FN(pow_tensor_scalar_out));
  m.impl("pow.Scalar", TORCH_FN(pow_scalar_tensor));
  REG3_PLAIN(atan2, atan2)
  REG3_PLAIN(logical_and, logical_and)
  REG3_PLAIN(logical_or, logical_or)
  REG3_PLAIN(logical_xor, logical_xor)
  m.impl("bitwise_and.Tensor", TORCH_FN(bitwise_and_tensor));
  m.impl("bitwise_and_.Tensor", TORCH_FN(bitwise_and_tensor_));
  m.impl("bitwise_and.Tensor_out", TORCH_FN(bitwise_and_out));
  m.impl("bitwise_or.Tensor", TORCH_FN(bitwise_or_tensor));
  m.impl("bitwise_or_.Tensor", TORCH_FN(bitwise_or_tensor_));
  m.impl("bitwise_or.Tensor_out", TORCH_FN(bitwise_or_out));
  m.impl("bitwise_xor.Tensor", TORCH_FN(bitwise_xor_tensor));
  m.impl("bitwise_xor_.Tensor", TORCH_FN(bitwise_xor_tensor_));
  m.impl("bitwise_xor.Tensor_out", TORCH_FN(bitwise_xor_out));
  REG_CMP(eq) REG_CMP(ne) REG_CMP(lt) REG_CMP(le) REG_CMP(gt) REG_CMP(ge)
  REG_UNARY(neg) REG_UNARY(abs) REG_UNARY(sqrt) REG_UNARY(rsqrt) REG_UNARY(reciprocal) REG_UNARY(exp)
  REG_UNARY(log) REG_UNARY(log2) REG_UNARY(log10) REG_UNARY(log1p) REG_UNARY(expm1) REG_UNARY(sin) REG_UNARY(cos)
  REG_UNARY(tanh) REG_UNARY(sigmoid) REG_UNARY(silu) REG_UNARY(ceil) REG_UNARY(floor) REG_UNARY(trunc)
  REG_UNARY(sign) REG_UNARY(sgn) REG_UNARY(erf) REG_UNARY(bitwise_not) REG_UNARY(hardswish) REG_UNARY(hardsigmoid)
  m.impl("round", TORCH_FN(round));
  m.impl("round_", TORCH_FN(round_));
  m.impl("round.out", TORCH_FN(round_out));
  m.impl("relu", TORCH_FN(relu));
  m.impl("relu_", TORCH_FN(relu_));
  m.impl("isnan", TORCH_FN(isnan));
  m.impl("logical_not", TORCH_FN(logical_not));
  m.impl("logical_not.out", TORCH_FN(logical_not_out));
  m.impl("gelu", TORCH_FN(gelu));
  m.impl("gelu_", TORCH_FN(gelu_));
  m.impl("gelu.out", TORCH_FN(gelu_out));
  m.impl("gelu_backward", TORCH_FN(gelu_backward));
  m.impl("leaky_relu", TORCH_FN(leaky_relu));
  m.impl("leaky_relu_", TORCH_FN(leaky_relu_));
  m.impl("leaky_relu_backward", TORCH_FN(leaky_relu_backward));
  m.impl("softplus", TORCH_FN(softplus));
  m.impl("softplus_backward", TORCH_FN(softplus_backward));
  m.impl("threshold", TORCH_FN(threshold));
  m.impl("threshold_", TORCH_FN(threshold_));
  m.impl("threshold_backward", TORCH_FN(threshold_backward));
  m.impl("hardtanh", TORCH_FN(hardtanh));
  m.impl("hardtanh_", TORCH_FN(hardtanh_));
  m.impl("hardtanh_backward", TORCH_FN(hardtanh_backward));
  m.impl("elu", TORCH_FN(elu_any));
  m.impl("elu_", TORCH_FN(elu_));
  m.impl("sigmoid_backward", TORCH_FN(sigmoid_backward));
  m.impl("tanh_backward", TORCH_FN(tanh_backward));
  m.impl("silu_backward", TORCH_FN(silu_backward));
  m.impl("clamp", TORCH_FN(clamp));
  m.impl("clamp_", TORCH_FN(clamp_));
  m.impl("clamp.out", TORCH_FN(clamp_out));
  m.impl("clamp_min", TORCH_FN(clamp_min));
  m.impl("clamp_min_", TORCH_FN(clamp_min_));
  m.impl("clamp_max", TORCH_FN(clamp_max));
  m.impl("clamp_max_", TORCH_FN(clamp_max_));
  m.impl("fill_.Scalar", TORCH_FN(fill_scalar_));
  m.impl("fill_.Tensor", TORCH_FN(fill_tensor_));
  m.impl("zero_", TORCH_FN(zero_));
  m.impl("where.self", TORCH_FN(where_self));
  m.impl("masked_fill_.Scalar", TORCH_FN(masked_fill_scalar_));
  m.impl("masked_fill_.Tensor", TORCH_FN(masked_fill_tensor_));
  m.impl("addcmul", TORCH_FN(addcmul));
  m.impl("addcmul_", TORCH_FN(addcmul_));
  m.impl("addcmul.out", TORCH_FN(addcmul_out));
  m.impl("addcdiv", TORCH_FN(addcdiv));
  m.impl("addcdiv_", TORCH_FN(addcdiv_));
  m.impl("addcdiv.out", TORCH_FN(addcdiv_out));
  m.impl("lerp.Scalar", TORCH_FN(lerp_scalar));
  m.impl("lerp_.Scalar", TORCH_FN(lerp_scalar_));
}

}  // namespace ops
}  // namespace catch_b200
