// Quantized convolution / linear custom ops (int8 tcgen05 kernels).
//
// Same argument order as the reference's custom ops
//   torch_mlu::conv2d(input, weight, bias, padding, stride, dilation, groups, q_scale, q_mode)
//   torch_mlu::linear(input, weight, bias, q_scale, q_mode)
// (torch_mlu/core/quantized/modules/conv.py:182-190, linear.py:44-48;
//  torch_mlu/csrc/aten/operators/cnnl/quantify_conv_forward.cpp:56-147, linear.cpp:171).
// q_scale = [input_scale, weight_scale] with scale = 127 / absmax (per tensor);
// q_mode 1 = int8 per-tensor weights, 3 = int8 per-channel weights (the int16 modes 2 / 4
// of the reference are computed as per-channel int8 here: the tensor cores have no int16
// path), 0 / missing scale = no quantization.
// The activation is quantized per tensor with input_scale; weights per output channel on
// the fly (cached per weight tensor); the int32 accumulator is de-quantized in the kernel
// epilogue with 1 / (input_scale * weight_scale[c]) and the bias is added in floating point.
#include <torch/library.h>

#include <mutex>
#include <unordered_map>

#include "../runtime/caching_allocator.h"
#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

struct QWeight {
  Tensor q;        // int8, same memory layout as the dense source
  Tensor inv;      // fp32 [rows]: 1 / (input_scale * row_scale) for the input scale `inv_s_in`
  double inv_s_in = 0.0;
  Tensor scale;    // fp32 [rows]: 127 / absmax(row)
  uint32_t version = 0;
  const void* ptr = nullptr;
  Tensor keep;     // the source weight: keeps its storage (and so the cache key) from being reused
};

std::mutex g_mu;
std::unordered_map<const void*, QWeight> g_cache;

// Host copies of the small scale / mode tensors.  Reading them from the device costs a synchronisation,
// so the values are cached per (storage address, version) and re-read only when the tensor changes.
struct HostVals {
  std::vector<double> v;
  uint32_t version = 0;
  int64_t numel = 0;
  Tensor keep;  // keeps the storage alive so that its address cannot be handed to another tensor while cached
};
std::unordered_map<const void*, HostVals> g_host_vals;

// torch.blackwell.empty_cache() also empties these caches (they keep device tensors alive)
const bool g_dropper_registered = [] {
  registerCacheDropper([] {
    std::lock_guard<std::mutex> g(g_mu);
    g_cache.clear();
    g_host_vals.clear();
  });
  return true;
}();
std::vector<double> host_values(const Tensor& t) {
  if (!t.defined() || t.numel() == 0) return {};
  if (t.device().is_cpu()) {  // nothing to synchronise with: read it directly
    Tensor h = t.detach().to(at::kDouble).contiguous().view({-1});
    return std::vector<double>(h.data_ptr<double>(), h.data_ptr<double>() + h.numel());
  }
  const void* key = t.data_ptr();
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_host_vals.find(key);
    if (it != g_host_vals.end() && it->second.version == t._version() && it->second.numel == t.numel()) return it->second.v;
  }
  Tensor h = t.detach().cpu().to(at::kDouble).contiguous().view({-1});
  HostVals hv;
  hv.v.assign(h.data_ptr<double>(), h.data_ptr<double>() + h.numel());
  hv.version = t._version();
  hv.numel = t.numel();
  hv.keep = t.detach();
  std::lock_guard<std::mutex> g(g_mu);
  if (g_host_vals.size() > 8192) g_host_vals.clear();
  g_host_vals[key] = hv;
  return hv.v;
}

// `w2d`: dense [rows, cols] view of the weight in the memory order the kernel reads.
QWeight quantize_weight(const Tensor& weight, const Tensor& w2d, bool per_channel, double tensor_scale,
                        const OpScope& scope) {
  const void* key = weight.data_ptr();
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_cache.find(key);
    if (it != g_cache.end() && it->second.version == weight._version() && it->second.q.numel() == w2d.numel())
      return it->second;
  }
  QWeight qw;
  qw.ptr = key;
  qw.version = weight._version();
  qw.keep = weight.detach();
  qw.q = empty_b200(w2d.sizes(), at::kChar, weight.device().index());
  qw.scale = empty_b200({w2d.size(0)}, at::kFloat, weight.device().index());
  if (per_channel) {
    B200_KERNEL_CHECK(b200_quantize_int8_rows(w2d.data_ptr(), to_b200_dtype(w2d.scalar_type()), w2d.size(0), w2d.size(1),
                                              qw.q.data_ptr(), qw.scale.data_ptr<float>(), scope.stream()));
  } else {
    B200_KERNEL_CHECK(b200_quantize_int8(w2d.data_ptr(), to_b200_dtype(w2d.scalar_type()), w2d.numel(),
                                         (float)tensor_scale, qw.q.data_ptr(), scope.stream()));
    qw.scale.fill_(tensor_scale);
  }
  std::lock_guard<std::mutex> g(g_mu);
  if (g_cache.size() > 4096) g_cache.clear();
  g_cache[key] = qw;
  return qw;
}

// 1 / (input scale * weight row scale): computed once per (weight, input scale)
Tensor dequant_scale(const Tensor& weight, QWeight& qw, double s_in) {
  if (qw.inv.defined() && qw.inv_s_in == s_in) return qw.inv;
  qw.inv = at::reciprocal(qw.scale * s_in);
  qw.inv_s_in = s_in;
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_cache.find(weight.data_ptr());
  if (it != g_cache.end() && it->second.version == qw.version) { it->second.inv = qw.inv; it->second.inv_s_in = s_in; }
  return qw.inv;
}

bool quant_active(const std::optional<Tensor>& q_scale, const std::optional<Tensor>& q_mode) {
  if (!q_scale.has_value() || !q_scale->defined() || q_scale->numel() == 0) return false;
  if (q_mode.has_value() && q_mode->defined() && q_mode->numel() > 0 && (int64_t)host_values(*q_mode)[0] == 0) return false;
  return true;
}

// input: floating point (quantized here with q_scale[0]) or int8 that a producer already quantized with that scale.
// residual / act: added / applied to the de-quantized result in the epilogue.  out_scale > 0: the result leaves the
// kernel as int8, quantized with out_scale (the input scale of the consumer), instead of as a 16-bit tensor.
Tensor qconv2d_device(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias,
                      at::IntArrayRef padding, at::IntArrayRef stride, at::IntArrayRef dilation, int64_t groups,
                      const Tensor& q_scale, int64_t mode, const std::optional<Tensor>& residual = std::nullopt,
                      int64_t act = 0, double out_scale = 0.0) {
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 4 && groups == 1 && dilation[0] == 1 && dilation[1] == 1,
              "b200 quantized conv2d: only dense 2-D convolutions");
  TORCH_CHECK(stride[0] >= 1 && stride[0] <= 2 && stride[1] >= 1 && stride[1] <= 2, "b200 quantized conv2d: stride 1 or 2");
  const int64_t N = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3);
  const int64_t K = weight.size(0), R = weight.size(2), S = weight.size(3);
  TORCH_CHECK(C % 16 == 0 && K % 8 == 0, "b200 quantized conv2d: channels must be multiples of 16 (in) and 8 (out)");
  const bool pre_quantized = input.scalar_type() == at::kChar;
  const at::ScalarType ft = pre_quantized ? weight.scalar_type() : input.scalar_type();
  TORCH_CHECK(ft == at::kHalf || ft == at::kBFloat16 || ft == at::kFloat, "b200 quantized conv2d: unsupported dtype ", ft);
  const std::vector<double> sc = host_values(q_scale);
  const double s_in = sc[0];
  const double s_w = sc.size() > 1 ? sc[1] : 1.0;
  OpScope scope("quantized_conv2d", input);
  const int64_t P = (H + 2 * padding[0] - R) / stride[0] + 1, Q = (W + 2 * padding[1] - S) / stride[1] + 1;
  Tensor x = input.contiguous(at::MemoryFormat::ChannelsLast);
  if (C == 1 || (H == 1 && W == 1)) x = empty_b200(input.sizes(), input.scalar_type(), input.device().index(), at::MemoryFormat::ChannelsLast).copy_(input);
  Tensor xq = x;
  if (!pre_quantized) {
    xq = empty_b200(x.sizes(), at::kChar, input.device().index(), at::MemoryFormat::ChannelsLast);
    B200_KERNEL_CHECK(b200_quantize_int8(x.data_ptr(), to_b200_dtype(ft), x.numel(), (float)s_in, xq.data_ptr(), scope.stream()));
  }
  Tensor wcl = weight.contiguous(at::MemoryFormat::ChannelsLast);
  if (R == 1 && S == 1) wcl = empty_b200(weight.sizes(), weight.scalar_type(), weight.device().index(), at::MemoryFormat::ChannelsLast).copy_(weight);
  Tensor w2d = wcl.permute({0, 2, 3, 1}).reshape({K, R * S * C});  // a view: memory is [K][R][S][C]
  QWeight qw = quantize_weight(weight, w2d, mode != 1, s_w, scope);
  Tensor inv = dequant_scale(weight, qw, s_in);
  const at::ScalarType ot = out_scale > 0 ? at::kChar : ft == at::kFloat ? at::kHalf : ft;
  Tensor out = empty_b200({N, K, P, Q}, ot, input.device().index(), at::MemoryFormat::ChannelsLast);
  B200ConvParams p;
  std::memset(&p, 0, sizeof(p));
  p.N = (int)N; p.P = (int)P; p.Q = (int)Q; p.Cin = (int)C; p.Cout = (int)K;
  p.ab_dtype = B200_I8;
  const int64_t sh = stride[0], sw = stride[1], ph = padding[0], pw = padding[1];
  const int64_t x_sn = xq.stride(0), x_sh = xq.stride(2), x_sw = xq.stride(3);
  p.num_views = (int)(sh * sw);
  bool view_ok[4] = {false, false, false, false};
  for (int64_t a = 0; a < sh; ++a)
    for (int64_t b = 0; b < sw; ++b) {
      const int idx = (int)(a * sw + b);
      const int64_t hv = (H - a + sh - 1) / sh, wv = (W - b + sw - 1) / sw;
      view_ok[idx] = hv > 0 && wv > 0;
      p.views[idx].base = static_cast<const char*>(xq.data_ptr()) + (a * x_sh + b * x_sw);
      p.views[idx].dims[0] = C; p.views[idx].dims[1] = std::max<int64_t>(wv, 1);
      p.views[idx].dims[2] = std::max<int64_t>(hv, 1); p.views[idx].dims[3] = N;
      p.views[idx].strides[0] = sw * x_sw; p.views[idx].strides[1] = sh * x_sh; p.views[idx].strides[2] = x_sn;
    }
  for (int64_t r = 0; r < R; ++r)
    for (int64_t s = 0; s < S; ++s) {
      const int64_t oh = r - ph, ow = s - pw;
      const int64_t a = ((oh % sh) + sh) % sh, b = ((ow % sw) + sw) % sw;
      const int idx = (int)(a * sw + b);
      if (!view_ok[idx]) continue;
      TORCH_CHECK(p.ntaps < B200_CONV_MAX_TAPS, "b200 quantized conv2d: filter too large");
      B200ConvTap& t = p.taps[p.ntaps++];
      t.dh = (short)((oh - a) / sh); t.dw = (short)((ow - b) / sw); t.map = (short)idx; t.wtap = (short)(r * S + s);
    }
  p.weight = qw.q.data_ptr();
  p.w_stride_k = 1; p.w_stride_n = R * S * C; p.w_stride_tap = C;
  p.wtaps = (int)(R * S);
  p.out = out.data_ptr(); p.out_dtype = to_b200_dtype(ot);
  p.o_sn = out.stride(0); p.o_sh = out.stride(2); p.o_sw = out.stride(3);
  p.o_mul_h = 1; p.o_mul_w = 1;
  p.scale = inv.data_ptr<float>();
  Tensor b;
  if (bias.has_value() && bias->defined()) {
    b = bias->to(at::kFloat).contiguous();
    p.bias = b.data_ptr();
    p.bias_dtype = B200_F32;
  }
  Tensor res;
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->sizes() == out.sizes(), "b200 quantized conv2d: the residual must have the output's shape");
    res = residual->scalar_type() == at::kFloat || residual->scalar_type() == at::kHalf || residual->scalar_type() == at::kBFloat16
              ? *residual : residual->to(ft == at::kFloat ? at::kHalf : ft);
    res = res.contiguous(at::MemoryFormat::ChannelsLast);  // addressed with the output's element offsets
    p.residual = res.data_ptr();
    p.res_dtype = to_b200_dtype(res.scalar_type());
  }
  p.act = (int)act;
  p.out_qscale = (float)out_scale;
  B200_KERNEL_CHECK(b200_conv_fprop(&p, scope.stream()));
  return ft == at::kFloat && out_scale <= 0 ? out.to(at::kFloat) : out;
}

Tensor qlinear_device(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, const Tensor& q_scale,
                      int64_t mode) {
  const at::ScalarType ft = input.scalar_type();
  TORCH_CHECK(ft == at::kHalf || ft == at::kBFloat16 || ft == at::kFloat, "b200 quantized linear: unsupported dtype ", ft);
  const int64_t K = input.size(-1), Nout = weight.size(0);
  TORCH_CHECK(weight.dim() == 2 && weight.size(1) == K && K % 16 == 0, "b200 quantized linear: in_features must be a multiple of 16");
  const std::vector<double> sc = host_values(q_scale);
  const double s_in = sc[0];
  const double s_w = sc.size() > 1 ? sc[1] : 1.0;
  OpScope scope("quantized_linear", input);
  Tensor x = input.reshape({-1, K}).contiguous();
  const int64_t M = x.size(0);
  Tensor xq = empty_b200({M, K}, at::kChar, input.device().index());
  B200_KERNEL_CHECK(b200_quantize_int8(x.data_ptr(), to_b200_dtype(ft), x.numel(), (float)s_in, xq.data_ptr(), scope.stream()));
  Tensor w = weight.contiguous();
  QWeight qw = quantize_weight(weight, w, mode != 1, s_w, scope);
  Tensor inv = dequant_scale(weight, qw, s_in);
  const at::ScalarType ot = ft;
  Tensor out = empty_b200({M, Nout}, ot, input.device().index());
  B200GemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.M = (int)M; p.N = (int)Nout; p.K = (int)K; p.batch = 1;
  p.A = xq.data_ptr(); p.B = qw.q.data_ptr(); p.D = out.data_ptr();
  p.lda = K; p.ldb = K; p.ldd = Nout;
  p.ab_dtype = B200_I8; p.d_dtype = to_b200_dtype(ot);
  p.alpha = 1.f; p.beta = 0.f;
  p.col_scale = inv.data_ptr<float>();
  Tensor b;
  if (bias.has_value() && bias->defined()) {
    b = bias->to(at::kFloat).contiguous();
    p.bias = b.data_ptr();
    p.bias_dtype = B200_F32;
  }
  if (M > 0) B200_KERNEL_CHECK(b200_gemm(&p, scope.stream()));
  std::vector<int64_t> osz(input.sizes().begin(), input.sizes().end());
  osz.back() = Nout;
  return out.reshape(osz);
}

int64_t mode_of(const std::optional<Tensor>& q_mode) {
  if (!q_mode.has_value() || !q_mode->defined() || q_mode->numel() == 0) return 1;
  return (int64_t)host_values(*q_mode)[0];
}

// Fake-quantized reference used on the CPU path and when the device kernel rejects a shape.
Tensor fake_quant(const Tensor& t, double scale) { return at::clamp(at::round(t * scale), -127, 127) / scale; }
Tensor fake_quant_rows(const Tensor& w) {
  Tensor flat = w.reshape({w.size(0), -1});
  Tensor amax = std::get<0>(flat.abs().max(1, true)).clamp_min(1e-30);
  Tensor s = 127.0 / amax;
  return (at::clamp(at::round(flat * s), -127, 127) / s).reshape(w.sizes());
}

Tensor qconv2d(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, at::IntArrayRef padding,
               at::IntArrayRef stride, at::IntArrayRef dilation, int64_t groups, const std::optional<Tensor>& q_scale,
               const std::optional<Tensor>& q_mode) {
  check_same_device("qconv2d", input, weight, bias);
  if (!quant_active(q_scale, q_mode)) return at::conv2d(input, weight, bias, stride, padding, dilation, groups);
  const int64_t mode = mode_of(q_mode);
  auto reference = [&]() {
    Tensor sc = q_scale->cpu().to(at::kDouble);
    Tensor xf = input.to(at::kFloat), wf = weight.to(at::kFloat);
    Tensor xq = fake_quant(xf, sc[0].item<double>());
    Tensor wq = mode == 1 && sc.numel() > 1 ? fake_quant(wf, sc[1].item<double>()) : fake_quant_rows(wf);
    std::optional<Tensor> b;
    if (bias.has_value() && bias->defined()) b = bias->to(at::kFloat);
    return at::conv2d(xq, wq, b, stride, padding, dilation, groups).to(input.scalar_type());
  };
  if (use_cpu_path() || !is_b200(input)) return reference();
  try {
    return qconv2d_device(input, weight, bias, padding, stride, dilation, groups, *q_scale, mode);
  } catch (const c10::OutOfMemoryError&) {
    throw;
  } catch (const std::exception& e) {
    if (!flags().op_trycatch) throw;
    B200LOG(DBG) << "quantized conv2d: device kernel rejected the configuration (" << e.what() << "); emulating.";
    return reference();
  }
}

// conv2d (quantized or not) + residual + ReLU + optional re-quantization for the next quantized layer: what the
// fusion pass makes of catch_b200::conv2d -> add -> relu chains (the reference folds the same chain into one
// quantized convolution node: torch_mlu/csrc/jit/codegen/convertion/ops/conv.cpp:180-216).
Tensor qconv_act(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, at::IntArrayRef padding,
                 at::IntArrayRef stride, at::IntArrayRef dilation, int64_t groups, const std::optional<Tensor>& q_scale,
                 const std::optional<Tensor>& q_mode, const std::optional<Tensor>& residual, int64_t act, double out_scale) {
  check_same_device("qconv_act", input, weight, bias, residual);
  const bool pre_quantized = input.scalar_type() == at::kChar;
  const bool quant = quant_active(q_scale, q_mode);
  TORCH_CHECK(quant || !pre_quantized, "catch_b200::qconv_act: an int8 input needs the layer's quantization scale");
  const at::ScalarType ft = pre_quantized ? weight.scalar_type() : input.scalar_type();
  auto finish = [&](Tensor y) {
    if (residual.has_value() && residual->defined()) y = y + residual->to(y.scalar_type());
    if (act == 1) y = at::relu(y);
    if (out_scale > 0) return at::clamp(at::round(y.to(at::kFloat) * out_scale), -127, 127).to(at::kChar);
    return y;
  };
  if (!quant) return finish(at::conv2d(input, weight, bias, stride, padding, dilation, groups));
  const int64_t mode = mode_of(q_mode);
  auto reference = [&]() {
    Tensor sc = q_scale->cpu().to(at::kDouble);
    const double s_in = sc[0].item<double>();
    Tensor xq = pre_quantized ? input.to(at::kFloat) / s_in : fake_quant(input.to(at::kFloat), s_in);
    Tensor wf = weight.to(at::kFloat);
    Tensor wq = mode == 1 && sc.numel() > 1 ? fake_quant(wf, sc[1].item<double>()) : fake_quant_rows(wf);
    std::optional<Tensor> b;
    if (bias.has_value() && bias->defined()) b = bias->to(at::kFloat);
    return finish(at::conv2d(xq, wq, b, stride, padding, dilation, groups).to(ft));
  };
  if (use_cpu_path() || !is_b200(input)) return reference();
  try {
    return qconv2d_device(input, weight, bias, padding, stride, dilation, groups, *q_scale, mode, residual, act, out_scale);
  } catch (const c10::OutOfMemoryError&) {
    throw;
  } catch (const std::exception& e) {
    if (!flags().op_trycatch) throw;
    B200LOG(DBG) << "qconv_act: device kernel rejected the configuration (" << e.what() << "); emulating.";
    return reference();
  }
}

Tensor qlinear(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias,
               const std::optional<Tensor>& q_scale, const std::optional<Tensor>& q_mode) {
  check_same_device("qlinear", input, weight, bias);
  if (!quant_active(q_scale, q_mode)) return at::linear(input, weight, bias);
  const int64_t mode = mode_of(q_mode);
  auto reference = [&]() {
    Tensor sc = q_scale->cpu().to(at::kDouble);
    Tensor xq = fake_quant(input.to(at::kFloat), sc[0].item<double>());
    Tensor wf = weight.to(at::kFloat);
    Tensor wq = mode == 1 && sc.numel() > 1 ? fake_quant(wf, sc[1].item<double>()) : fake_quant_rows(wf);
    std::optional<Tensor> b;
    if (bias.has_value() && bias->defined()) b = bias->to(at::kFloat);
    return at::linear(xq, wq, b).to(input.scalar_type());
  };
  if (use_cpu_path() || !is_b200(input)) return reference();
  try {
    return qlinear_device(input, weight, bias, *q_scale, mode);
  } catch (const c10::OutOfMemoryError&) {
    throw;
  } catch (const std::exception& e) {
    if (!flags().op_trycatch) throw;
    B200LOG(DBG) << "quantized linear: device kernel rejected the configuration (" << e.what() << "); emulating.";
    return reference();
  }
}

// abs-max on the device (observers use it during on-device calibration)
Tensor absmax(const Tensor& t) {
  if (use_cpu_path() || !is_b200(t) || (t.scalar_type() != at::kFloat && t.scalar_type() != at::kHalf && t.scalar_type() != at::kBFloat16))
    return t.abs().max().to(at::kFloat);
  OpScope scope("absmax", t);
  Tensor x = t.is_non_overlapping_and_dense() ? t : t.contiguous();
  Tensor out = at::zeros({}, t.options().dtype(at::kFloat));
  B200_KERNEL_CHECK(b200_absmax(x.data_ptr(), to_b200_dtype(x.scalar_type()), x.numel(), out.data_ptr<float>(), scope.stream()));
  return out;
}

// conv1d: the same kernels through a [N, C, 1, L] view.
Tensor qconv1d(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, at::IntArrayRef padding,
               at::IntArrayRef stride, at::IntArrayRef dilation, int64_t groups, const std::optional<Tensor>& q_scale,
               const std::optional<Tensor>& q_mode) {
  TORCH_CHECK(input.dim() == 3 && weight.dim() == 3, "catch_b200::conv1d expects [N, C, L] input and [K, C, S] weight");
  const int64_t p[2] = {0, padding.empty() ? 0 : padding[0]}, st[2] = {1, stride.empty() ? 1 : stride[0]};
  const int64_t d[2] = {1, dilation.empty() ? 1 : dilation[0]};
  Tensor out = qconv2d(input.unsqueeze(2), weight.unsqueeze(2), bias, at::IntArrayRef(p, 2), at::IntArrayRef(st, 2),
                       at::IntArrayRef(d, 2), groups, q_scale, q_mode);
  return out.squeeze(2);
}

// conv3d: no int8 device kernel; quantized calls compute with fake-quantized operands (same rounding as
// the int8 path) through the floating-point convolution.
Tensor qconv3d(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, at::IntArrayRef padding,
               at::IntArrayRef stride, at::IntArrayRef dilation, int64_t groups, const std::optional<Tensor>& q_scale,
               const std::optional<Tensor>& q_mode) {
  if (!quant_active(q_scale, q_mode)) return at::conv3d(input, weight, bias, stride, padding, dilation, groups);
  const int64_t mode = mode_of(q_mode);
  const std::vector<double> sc = host_values(*q_scale);
  Tensor xf = input.to(at::kFloat), wf = weight.to(at::kFloat);
  Tensor xq = fake_quant(xf, sc[0]);
  Tensor wq = mode == 1 && sc.size() > 1 ? fake_quant(wf, sc[1]) : fake_quant_rows(wf);
  std::optional<Tensor> b;
  if (bias.has_value() && bias->defined()) b = bias->to(at::kFloat);
  return at::conv3d(xq, wq, b, stride, padding, dilation, groups).to(input.scalar_type());
}

// view as a named op, so that fusion graphs can keep shape changes inside a fusion group
Tensor view_op(const Tensor& self, at::IntArrayRef size) { return self.view(size); }

}  // namespace

TORCH_LIBRARY_FRAGMENT(catch_b200, m) {
  m.def("conv1d(Tensor input, Tensor weight, Tensor? bias, int[] padding, int[] stride, int[] dilation, int groups, "
        "Tensor? q_scale, Tensor? q_mode) -> Tensor");
  m.def("conv3d(Tensor input, Tensor weight, Tensor? bias, int[] padding, int[] stride, int[] dilation, int groups, "
        "Tensor? q_scale, Tensor? q_mode) -> Tensor");
  m.def("view(Tensor(a) self, int[] size) -> Tensor(a)");
  m.def("conv2d(Tensor input, Tensor weight, Tensor? bias, int[] padding, int[] stride, int[] dilation, int groups, "
        "Tensor? q_scale, Tensor? q_mode) -> Tensor");
  m.def("linear(Tensor input, Tensor weight, Tensor? bias, Tensor? q_scale, Tensor? q_mode) -> Tensor");
  m.def("absmax(Tensor t) -> Tensor");
  m.def("qconv_act(Tensor input, Tensor weight, Tensor? bias, int[] padding, int[] stride, int[] dilation, int groups, "
        "Tensor? q_scale, Tensor? q_mode, Tensor? residual, int act, float out_scale) -> Tensor");
}
TORCH_LIBRARY_IMPL(catch_b200, CompositeExplicitAutograd, m) {
  m.impl("conv2d", TORCH_FN(qconv2d));
  m.impl("qconv_act", TORCH_FN(qconv_act));
  m.impl("conv1d", TORCH_FN(qconv1d));
  m.impl("conv3d", TORCH_FN(qconv3d));
  m.impl("view", TORCH_FN(view_op));
  m.impl("linear", TORCH_FN(qlinear));
  m.impl("absmax", TORCH_FN(absmax));
}

}  // namespace ops
}  // namespace catch_b200
