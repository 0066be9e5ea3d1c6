// Host drivers of the tcgen05 convolution kernels: layout normalisation (NHWC),
// per-parity input views for strided convolutions, tap tables, the first-layer
// "row window" formulation for tiny channel counts, data and weight gradients.
//
// Behavioural parity: cnnl_convolution_overrideable / _backward_overrideable
// (torch_mlu/csrc/aten/operators/cnnl/convolution_overrideable.cpp:241-297) make
// inputs channels-last, pick a dense or depthwise kernel and return channels-last
// results; configurations the device kernels do not cover raise, and the caller
// (conv.cpp) reruns them on the CPU.
#include "conv_impl.h"

#include "common.h"
#include "kernels.h"

namespace catch_b200 {
namespace ops {
namespace {

using at::Tensor;

struct ConvGeom {
  int64_t N, C, H, W, K, R, S, P, Q;
  int64_t sh, sw, ph, pw;
  int64_t dlh = 1, dlw = 1;  // dilation
};

inline int64_t floordiv(int64_t a, int64_t b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }
inline int64_t ceildiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Tensor-core operand type: 16-bit inputs run as they are.  fp32 inputs are split into two bf16 terms
// (x = hi + lo, hi = bf16(x), lo = bf16(x - hi)) and a convolution becomes three tensor-core passes
// hi*hi + lo*hi + hi*lo accumulated in fp32: bf16 has fp32's exponent range, so values above 65504 or below
// 1e-7 survive, and the two terms carry 16 mantissa bits (more than a TF32 path would).
at::ScalarType compute_dtype(at::ScalarType t) { return t == at::kHalf ? at::kHalf : at::kBFloat16; }
struct Split {
  Tensor hi, lo;  // lo is undefined for 16-bit sources
};
Split split_operand(const Tensor& x) {
  Split s;
  if (x.scalar_type() != at::kFloat) {
    s.hi = x;
    return s;
  }
  s.hi = x.to(at::kBFloat16);
  s.lo = (x - s.hi.to(at::kFloat)).to(at::kBFloat16);
  return s;
}
// The (a, b) operand pairs of the passes, the full-precision one last (it carries bias / activation).
std::vector<std::pair<Tensor, Tensor>> split_passes(const Split& a, const Split& b) {
  std::vector<std::pair<Tensor, Tensor>> v;
  if (a.lo.defined()) v.emplace_back(a.lo, b.hi);
  if (b.lo.defined()) v.emplace_back(a.hi, b.lo);
  v.emplace_back(a.hi, b.hi);
  return v;
}

// channels-last (dense NHWC) tensor of dtype `dt`
Tensor to_nhwc(const Tensor& x, at::ScalarType dt) {
  Tensor t = x.scalar_type() == dt ? x : x.to(dt);
  if (t.size(1) == 1 || (t.size(2) == 1 && t.size(3) == 1)) {
    // stride ambiguity: force a fresh channels-last copy
    Tensor o = empty_b200(t.sizes(), dt, t.device().index(), at::MemoryFormat::ChannelsLast);
    o.copy_(t);
    return o;
  }
  return t.contiguous(at::MemoryFormat::ChannelsLast);
}

void check_supported(const Tensor& input, const Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding,
                     at::IntArrayRef dilation, bool transposed, int64_t groups) {
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "b200 conv: only 2-D convolutions run on the device");
  TORCH_CHECK(!transposed, "b200 conv: transposed convolution has no device kernel");
  TORCH_CHECK(groups == 1, "b200 conv: grouped convolution has no device kernel");
  TORCH_CHECK(dilation[0] >= 1 && dilation[1] >= 1, "b200 conv: invalid dilation");
  TORCH_CHECK(stride[0] >= 1 && stride[0] <= 4 && stride[1] >= 1 && stride[1] <= 4, "b200 conv: strides above 4 have no device kernel");
  TORCH_CHECK(weight.size(2) * weight.size(3) <= B200_CONV_MAX_TAPS, "b200 conv: filters with more than ", B200_CONV_MAX_TAPS,
              " taps have no device kernel");
  const auto t = input.scalar_type();
  TORCH_CHECK(t == at::kBFloat16 || t == at::kHalf || t == at::kFloat, "b200 conv: unsupported dtype ", t);
  TORCH_CHECK(weight.size(0) % 8 == 0, "b200 conv: output channels must be a multiple of 8");
  const int64_t C = input.size(1);
  TORCH_CHECK(C % 8 == 0 || (C <= 8 && weight.size(3) <= 8 && dilation[0] == 1 && dilation[1] == 1 && stride[0] <= 2 && stride[1] <= 2),
              "b200 conv: input channels must be a multiple of 8 (or <= 8 with an undilated filter of width <= 8 and stride <= 2)");
}

ConvGeom geom(const Tensor& input, const Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding,
              at::IntArrayRef dilation = {}) {
  ConvGeom g;
  g.N = input.size(0); g.C = input.size(1); g.H = input.size(2); g.W = input.size(3);
  g.K = weight.size(0); g.R = weight.size(2); g.S = weight.size(3);
  g.sh = stride[0]; g.sw = stride[1]; g.ph = padding[0]; g.pw = padding[1];
  if (dilation.size() == 2) { g.dlh = dilation[0]; g.dlw = dilation[1]; }
  g.P = (g.H + 2 * g.ph - g.dlh * (g.R - 1) - 1) / g.sh + 1;
  g.Q = (g.W + 2 * g.pw - g.dlw * (g.S - 1) - 1) / g.sw + 1;
  return g;
}

// Per-parity views of an NHWC tensor x for a convolution with stride (sh, sw):
// view (a, b) holds the pixels (a + i*sh, b + j*sw).  Fills views / taps for the
// forward problem (also used by wgrad).  Returns number of taps.
template <typename Params>
void build_forward_taps(Params& p, const Tensor& x, const ConvGeom& g) {
  const int64_t x_sn = x.stride(0), x_sh = x.stride(2), x_sw = x.stride(3);
  const char* base = static_cast<const char*>(x.data_ptr());
  p.num_views = (int)(g.sh * g.sw);
  TORCH_CHECK(p.num_views <= B200_CONV_MAX_MAPS, "b200 conv: stride ", g.sh, "x", g.sw, " needs more input views than the kernel has");
  bool view_ok[B200_CONV_MAX_MAPS];
  std::fill(view_ok, view_ok + B200_CONV_MAX_MAPS, false);
  for (int64_t a = 0; a < g.sh; ++a) {
    for (int64_t b = 0; b < g.sw; ++b) {
      const int idx = (int)(a * g.sw + b);
      B200ConvView& v = p.views[idx];
      const int64_t hv = ceildiv(g.H - a, g.sh), wv = ceildiv(g.W - b, g.sw);
      view_ok[idx] = hv > 0 && wv > 0;
      v.base = base + (a * x_sh + b * x_sw) * x.element_size();
      v.dims[0] = g.C; v.dims[1] = std::max<int64_t>(wv, 1); v.dims[2] = std::max<int64_t>(hv, 1); v.dims[3] = g.N;
      v.strides[0] = g.sw * x_sw; v.strides[1] = g.sh * x_sh; v.strides[2] = x_sn;
    }
  }
  p.ntaps = 0;
  for (int64_t r = 0; r < g.R; ++r) {
    for (int64_t s = 0; s < g.S; ++s) {
      const int64_t oh = r * g.dlh - g.ph, ow = s * g.dlw - g.pw;
      const int64_t a = ((oh % g.sh) + g.sh) % g.sh, b = ((ow % g.sw) + g.sw) % g.sw;
      const int idx = (int)(a * g.sw + b);
      if (!view_ok[idx]) continue;
      B200ConvTap& t = p.taps[p.ntaps++];
      t.dh = (short)((oh - a) / g.sh);
      t.dw = (short)((ow - b) / g.sw);
      t.map = (short)idx;
      t.wtap = (short)(r * g.S + s);
    }
  }
}

// ---- first layer (C <= 8): rows of the padded NHWC8 image are the K dimension ----
struct StemPack {
  Tensor xp;       // [N][Hp][Wp][8]
  int64_t Hp, Wp;
};
StemPack pack_stem_input(const Tensor& input, const ConvGeom& g, at::ScalarType dt, const OpScope& scope) {
  StemPack sp;
  sp.Hp = g.H + 2 * g.ph;
  // every window of 8 pixels must stay inside its row
  sp.Wp = std::max<int64_t>(g.W + 2 * g.pw, (g.Q - 1) * g.sw + 8);
  sp.xp = empty_b200({g.N, sp.Hp, sp.Wp, 8}, dt, input.device().index());
  B200_KERNEL_CHECK(b200_pack_nhwc8(input.data_ptr(), to_b200_dtype(input.scalar_type()), input.stride(0),
                                    input.stride(1), input.stride(2), input.stride(3), (int)g.N, (int)g.C, (int)g.H,
                                    (int)g.W, sp.xp.data_ptr(), to_b200_dtype(dt), (int)sp.Hp, (int)sp.Wp, (int)g.ph,
                                    (int)g.pw, scope.stream()));
  return sp;
}
template <typename Params>
void build_stem_taps(Params& p, const StemPack& sp, const ConvGeom& g) {
  // view a (row parity): rows a, a+sh, ...; each "pixel" of the view is a window of
  // 8 packed pixels (64 elements) starting at packed column q*sw.
  const char* base = static_cast<const char*>(sp.xp.data_ptr());
  p.num_views = (int)g.sh;
  for (int64_t a = 0; a < g.sh; ++a) {
    B200ConvView& v = p.views[a];
    v.base = base + a * sp.Wp * 8 * 2;
    v.dims[0] = 64; v.dims[1] = g.Q; v.dims[2] = ceildiv(sp.Hp - a, g.sh); v.dims[3] = g.N;
    v.strides[0] = g.sw * 8; v.strides[1] = g.sh * sp.Wp * 8; v.strides[2] = sp.Hp * sp.Wp * 8;
  }
  p.ntaps = 0;
  for (int64_t r = 0; r < g.R; ++r) {
    B200ConvTap& t = p.taps[p.ntaps++];
    t.dh = (short)(r / g.sh);
    t.dw = 0;
    t.map = (short)(r % g.sh);
    t.wtap = (short)r;
  }
}
// weight [K, C, R, S] -> [R][K][8(s)][8(c)] zero padded
Tensor pack_stem_weight(const Tensor& weight, const ConvGeom& g, at::ScalarType dt) {
  Tensor wp = at::zeros({g.R, g.K, 8, 8}, weight.options().dtype(dt));
  wp.narrow(2, 0, g.S).narrow(3, 0, g.C).copy_(weight.permute({2, 0, 3, 1}));
  return wp;
}

// One tensor-core pass: out = act((x * w) * scale + bias + residual); x and w are 16-bit tensors of one dtype.
void forward_pass(const Tensor& input, const Tensor& weight, const Tensor* bias, const ConvGeom& g, const float* scale,
                  const Tensor* residual, int act, Tensor& out, double* stats, const OpScope& scope) {
  const at::ScalarType dt = input.scalar_type();
  B200ConvParams p;
  std::memset(&p, 0, sizeof(p));
  Tensor x, w;
  StemPack sp;
  if (g.C % 8 != 0 || g.C < 8) {
    sp = pack_stem_input(input, g, dt, scope);
    w = pack_stem_weight(weight, g, dt);
    build_stem_taps(p, sp, g);
    p.Cin = 64;
    p.weight = w.data_ptr();
    p.w_stride_k = 1; p.w_stride_n = 64; p.w_stride_tap = g.K * 64;
    p.wtaps = (int)g.R;
  } else {
    x = to_nhwc(input, dt);
    w = to_nhwc(weight, dt);  // memory [K][R][S][C]
    build_forward_taps(p, x, g);
    p.Cin = (int)g.C;
    p.weight = w.data_ptr();
    p.w_stride_k = 1; p.w_stride_n = g.R * g.S * g.C; p.w_stride_tap = g.C;
    p.wtaps = (int)(g.R * g.S);
  }
  p.N = (int)g.N; p.P = (int)g.P; p.Q = (int)g.Q; p.Cout = (int)g.K;
  p.ab_dtype = to_b200_dtype(dt);
  p.out = out.data_ptr(); p.out_dtype = to_b200_dtype(out.scalar_type());
  p.o_sn = out.stride(0); p.o_sh = out.stride(2); p.o_sw = out.stride(3);
  p.o_mul_h = 1; p.o_mul_w = 1;
  p.scale = scale;
  Tensor b;
  if (bias) {
    b = bias->contiguous();
    p.bias = b.data_ptr();
    p.bias_dtype = to_b200_dtype(b.scalar_type());
  }
  if (residual) {
    TORCH_CHECK(residual->sizes() == out.sizes() && residual->strides() == out.strides(), "conv residual layout mismatch");
    p.residual = residual->data_ptr();
    p.res_dtype = to_b200_dtype(residual->scalar_type());
  }
  p.act = act;
  p.stats = stats;
  TORCH_CHECK(p.ntaps > 0, "b200 conv: empty tap list");
  B200_KERNEL_CHECK(b200_conv_fprop(&p, scope.stream()));
}

Tensor forward_impl(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, const ConvGeom& g,
                    const float* scale, const Tensor* residual, int act, at::ScalarType out_dtype,
                    double* stats = nullptr) {
  OpScope scope("conv_fprop", input);
  Tensor out = empty_b200({g.N, g.K, g.P, g.Q}, out_dtype, input.device().index(), at::MemoryFormat::ChannelsLast);
  if (out.numel() == 0) return out;
  const at::ScalarType dt = compute_dtype(input.scalar_type());
  Tensor res;
  if (residual) {
    res = to_nhwc(*residual, residual->scalar_type());
    TORCH_CHECK(res.sizes() == out.sizes(), "conv residual shape mismatch");
  }
  const Tensor* bptr = (bias.has_value() && bias->defined()) ? &*bias : nullptr;
  if (input.scalar_type() != at::kFloat) {
    Tensor w = weight.scalar_type() == dt ? weight : weight.to(dt);
    forward_pass(input, w, bptr, g, scale, residual ? &res : nullptr, act, out, stats, scope);
    return out;
  }
  // fp32: three bf16 passes accumulated through the epilogue's residual input; the per-channel scale applies to
  // every partial sum, bias / activation (and a caller's residual, added first) only once
  TORCH_CHECK(!stats && out_dtype == at::kFloat, "b200 conv: fp32 inputs produce fp32 outputs without channel statistics");
  auto passes = split_passes(split_operand(input), split_operand(weight.to(at::kFloat)));
  for (size_t i = 0; i < passes.size(); ++i) {
    const bool first = i == 0, last = i + 1 == passes.size();
    const Tensor* r = first ? (residual ? &res : nullptr) : &out;
    forward_pass(passes[i].first, passes[i].second, last ? bptr : nullptr, g, scale, r, last ? act : 0, out, nullptr, scope);
  }
  return out;
}

// add_to: a gradient of the same input that arrived over another path (the skip connection of a residual block);
// it is added in the epilogue of the kernel instead of by a separate element-wise kernel afterwards.
Tensor dgrad_impl(const Tensor& grad_in, const Tensor& weight, const ConvGeom& g, at::ScalarType out_dtype,
                  const Tensor* add_to = nullptr) {
  OpScope scope("conv_dgrad", grad_in);
  Tensor dx = empty_b200({g.N, g.C, g.H, g.W}, out_dtype, grad_in.device().index(), at::MemoryFormat::ChannelsLast);
  if (dx.numel() == 0) return dx;
  Tensor extra;
  if (add_to && add_to->defined()) {
    TORCH_CHECK(add_to->sizes() == dx.sizes(), "b200 conv dgrad: the gradient to add must have the input's shape");
    extra = add_to->scalar_type() == out_dtype ? *add_to : add_to->to(out_dtype);
    extra = extra.contiguous(at::MemoryFormat::ChannelsLast);
  }
  // the epilogue can add it when every input element is written by exactly one launch of the first pass
  const bool fuse_extra = extra.defined() && g.sh == 1 && g.sw == 1 && out_dtype != at::kFloat;
  const bool fp32 = grad_in.scalar_type() == at::kFloat;
  const at::ScalarType dt = compute_dtype(grad_in.scalar_type());
  TORCH_CHECK(!fp32 || out_dtype == at::kFloat, "b200 conv dgrad: fp32 gradients produce fp32 input gradients");
  auto passes = fp32 ? split_passes(split_operand(grad_in), split_operand(weight.to(at::kFloat)))
                     : std::vector<std::pair<Tensor, Tensor>>{{grad_in, weight.scalar_type() == dt ? weight : weight.to(dt)}};
  bool zeroed = false;
  for (size_t pass = 0; pass < passes.size(); ++pass) {
    Tensor dy = to_nhwc(passes[pass].first, dt);
    Tensor w = to_nhwc(passes[pass].second, dt);
    bool need_zero = false;
    std::vector<B200ConvParams> launches;
    for (int64_t a = 0; a < g.sh; ++a) {
      for (int64_t b = 0; b < g.sw; ++b) {
        const int64_t Pa = ceildiv(g.H - a, g.sh), Qb = ceildiv(g.W - b, g.sw);
        if (Pa <= 0 || Qb <= 0) continue;
        B200ConvParams p;
        std::memset(&p, 0, sizeof(p));
        p.ntaps = 0;
        for (int64_t r = 0; r < g.R; ++r) {
          if ((a + g.ph - r * g.dlh) % g.sh != 0) continue;
          for (int64_t s = 0; s < g.S; ++s) {
            if ((b + g.pw - s * g.dlw) % g.sw != 0) continue;
            B200ConvTap& t = p.taps[p.ntaps++];
            t.dh = (short)floordiv(a + g.ph - r * g.dlh, g.sh);
            t.dw = (short)floordiv(b + g.pw - s * g.dlw, g.sw);
            t.map = 0;
            t.wtap = (short)(r * g.S + s);
          }
        }
        if (p.ntaps == 0) { need_zero = true; continue; }
        p.N = (int)g.N; p.P = (int)Pa; p.Q = (int)Qb;
        p.Cin = (int)g.K; p.Cout = (int)g.C;
        p.ab_dtype = to_b200_dtype(dt);
        p.num_views = 1;
        p.views[0].base = dy.data_ptr();
        p.views[0].dims[0] = g.K; p.views[0].dims[1] = g.Q; p.views[0].dims[2] = g.P; p.views[0].dims[3] = g.N;
        p.views[0].strides[0] = dy.stride(3); p.views[0].strides[1] = dy.stride(2); p.views[0].strides[2] = dy.stride(0);
        p.weight = w.data_ptr();
        // element (tap, n = ci, k = co) of the channels-last filter [K][R][S][C]
        p.w_stride_n = 1; p.w_stride_k = g.R * g.S * g.C; p.w_stride_tap = g.C;
        p.wtaps = (int)(g.R * g.S);
        p.out = dx.data_ptr(); p.out_dtype = to_b200_dtype(out_dtype);
        p.o_sn = dx.stride(0); p.o_sh = dx.stride(2); p.o_sw = dx.stride(3);
        p.o_mul_h = (int)g.sh; p.o_off_h = (int)a; p.o_mul_w = (int)g.sw; p.o_off_w = (int)b;
        p.alpha = 1.f;
        if (pass > 0) {  // later passes add to what the earlier ones wrote
          p.residual = dx.data_ptr();
          p.res_dtype = to_b200_dtype(out_dtype);
        } else if (fuse_extra) {
          p.residual = extra.data_ptr();
          p.res_dtype = to_b200_dtype(out_dtype);
        }
        launches.push_back(p);
      }
    }
    if (need_zero && !zeroed) { dx.zero_(); zeroed = true; }
    for (auto& p : launches) B200_KERNEL_CHECK(b200_conv_fprop(&p, scope.stream()));
  }
  if (extra.defined() && !fuse_extra) dx.add_(extra);
  return dx;
}

// fp32_result: hand back the fp32 accumulation buffer itself (viewed as [K, C, R, S] in channels-last
// memory) instead of a copy in the weight's dtype -- for callers that accumulate into fp32 master gradients.
// accum_into: an fp32 tensor holding [K][R][S][C] (the channels-last memory of the weight gradient) that the
// kernel adds its result to, e.g. a view of a flat gradient bucket; nothing is returned then.
Tensor wgrad_impl(const Tensor& grad_in, const Tensor& input, const Tensor& weight, const ConvGeom& g,
                  bool fp32_result = false, const Tensor* accum_into = nullptr) {
  OpScope scope("conv_wgrad", grad_in);
  const bool fp32 = grad_in.scalar_type() == at::kFloat || input.scalar_type() == at::kFloat;
  const at::ScalarType dt = compute_dtype(fp32 ? at::kFloat : grad_in.scalar_type());
  const bool stem = g.C % 8 != 0 || g.C < 8;
  const int64_t cin_k = stem ? 64 : g.C, wtaps = stem ? g.R : g.R * g.S;
  const bool direct = accum_into && !stem;
  Tensor acc;
  if (direct) {
    TORCH_CHECK(accum_into->scalar_type() == at::kFloat && accum_into->numel() == g.K * wtaps * cin_k,
                "conv wgrad: the accumulation target must be fp32 with the weight's number of elements");
    acc = *accum_into;
  } else {
    acc = at::zeros({g.K, wtaps * cin_k}, grad_in.options().dtype(at::kFloat));
  }
  auto passes = fp32 ? split_passes(split_operand(grad_in.to(at::kFloat)), split_operand(input.to(at::kFloat)))
                     : std::vector<std::pair<Tensor, Tensor>>{{grad_in, input.scalar_type() == dt ? input : input.to(dt)}};
  for (auto& pr : passes) {
    Tensor dy = to_nhwc(pr.first, dt);
    B200ConvWgradParams p;
    std::memset(&p, 0, sizeof(p));
    Tensor x;
    StemPack sp;
    if (stem) {
      sp = pack_stem_input(pr.second, g, dt, scope);
      build_stem_taps(p, sp, g);
    } else {
      x = to_nhwc(pr.second, dt);
      build_forward_taps(p, x, g);
    }
    p.N = (int)g.N; p.P = (int)g.P; p.Q = (int)g.Q; p.Cin = (int)cin_k; p.Cout = (int)g.K;
    p.ab_dtype = to_b200_dtype(dt);
    p.dy = dy.data_ptr();
    p.dy_sn = dy.stride(0); p.dy_sh = dy.stride(2); p.dy_sw = dy.stride(3);
    p.dw_acc = acc.data_ptr<float>();
    p.wtaps = (int)wtaps;
    if (p.ntaps > 0) B200_KERNEL_CHECK(b200_conv_wgrad(&p, scope.stream()));
  }
  if (direct) return Tensor();
  Tensor dw;
  if (stem) {
    // acc [K][R][8(s)][8(c)] -> [K, C, R, S]
    dw = acc.view({g.K, g.R, 8, 8}).narrow(2, 0, g.S).narrow(3, 0, g.C).permute({0, 3, 1, 2});
  } else {
    // acc [K][R][S][C] is the channels-last memory of a [K, C, R, S] tensor
    dw = acc.view({g.K, g.R, g.S, g.C}).permute({0, 3, 1, 2});
  }
  if (accum_into) {  // the first-layer packing cannot add in place
    at::Tensor target = accum_into->dim() == 4 ? *accum_into : accum_into->view({g.K, g.R, g.S, g.C}).permute({0, 3, 1, 2});
    target.add_(dw);
    return Tensor();
  }
  if (fp32_result) return dw;
  Tensor out = at::empty_like(weight, weight.options(), weight.suggest_memory_format());
  out.copy_(dw);
  return out;
}


// ---- depthwise (groups == Cin, one filter per output channel): direct CUDA-core kernels ----
bool is_depthwise(const Tensor& input, const Tensor& weight, int64_t groups) {
  return groups > 1 && groups == input.size(1) && weight.size(1) == 1 && weight.size(0) % groups == 0;
}
void check_depthwise(const Tensor& input, at::IntArrayRef dilation, bool transposed) {
  TORCH_CHECK(!transposed && dilation[0] == 1 && dilation[1] == 1, "b200 depthwise conv: no dilation / transposition on the device");
  const auto t = input.scalar_type();
  TORCH_CHECK(t == at::kFloat || t == at::kBFloat16 || t == at::kHalf, "b200 depthwise conv: unsupported dtype ", t);
  TORCH_CHECK(input.dim() == 4, "b200 depthwise conv: 4-D input expected");
}
struct DwCall {
  long long dims[7];
  int conv[6];
  std::vector<long long> xs, ys;
};
DwCall dw_call(const ConvGeom& g, const Tensor& x_like, const Tensor& y_like) {
  DwCall c;
  const long long d[7] = {g.N, g.C, g.H, g.W, g.K, g.P, g.Q};
  std::copy(d, d + 7, c.dims);
  const int cv[6] = {(int)g.R, (int)g.S, (int)g.sh, (int)g.sw, (int)g.ph, (int)g.pw};
  std::copy(cv, cv + 6, c.conv);
  c.xs.assign(x_like.strides().begin(), x_like.strides().end());
  c.ys.assign(y_like.strides().begin(), y_like.strides().end());
  return c;
}
Tensor depthwise_forward(const Tensor& input, const Tensor& weight, const std::optional<Tensor>& bias, const ConvGeom& g) {
  OpScope scope("depthwise_conv", input);
  Tensor out = empty_b200({g.N, g.K, g.P, g.Q}, input.scalar_type(), input.device().index(), input.suggest_memory_format());
  Tensor w = weight.to(input.scalar_type()).contiguous();
  DwCall c = dw_call(g, input, out);
  B200_KERNEL_CHECK(b200_depthwise_conv(0, input.data_ptr(), w.data_ptr(), out.data_ptr(), to_b200_dtype(input.scalar_type()), c.dims,
                                        c.conv, c.xs.data(), c.ys.data(), scope.stream()));
  if (bias.has_value() && bias->defined()) out.add_(bias->view({1, -1, 1, 1}));
  return out;
}
std::tuple<Tensor, Tensor, Tensor> depthwise_backward(const Tensor& grad_in, const Tensor& input, const Tensor& weight,
                                                      const ConvGeom& g, std::array<bool, 3> mask) {
  OpScope scope("depthwise_conv_backward", grad_in);
  Tensor grad = grad_in.to(input.scalar_type());
  Tensor dx, dw, db;
  const int dt = to_b200_dtype(input.scalar_type());
  if (mask[0]) {
    dx = at::empty_strided(input.sizes(), input.strides(), input.options());
    if (!dx.is_non_overlapping_and_dense()) dx = at::empty_like(input, at::MemoryFormat::Contiguous);
    Tensor w = weight.to(input.scalar_type()).contiguous();
    DwCall c = dw_call(g, dx, grad);
    B200_KERNEL_CHECK(b200_depthwise_conv(1, dx.data_ptr(), w.data_ptr(), grad.data_ptr(), dt, c.dims, c.conv, c.xs.data(),
                                          c.ys.data(), scope.stream()));
  }
  if (mask[1]) {
    Tensor acc = at::empty({g.K, 1, g.R, g.S}, input.options().dtype(at::kFloat));
    DwCall c = dw_call(g, input, grad);
    B200_KERNEL_CHECK(b200_depthwise_conv(2, input.data_ptr(), acc.data_ptr(), grad.data_ptr(), dt, c.dims, c.conv, c.xs.data(),
                                          c.ys.data(), scope.stream()));
    dw = acc.to(weight.scalar_type());
  }
  if (mask[2]) db = grad_in.sum({0, 2, 3});
  return {dx, dw, db};
}

// ---- transposed convolution = the data gradient of the matching forward convolution ----
ConvGeom transposed_geom(const Tensor& input, const Tensor& weight, at::IntArrayRef stride, at::IntArrayRef padding,
                         at::IntArrayRef output_padding, at::IntArrayRef dilation) {
  // weight [Cin, Cout, R, S]; the matching forward convolution maps [N, Cout, Hout, Wout] -> [N, Cin, H, W]
  ConvGeom g;
  g.N = input.size(0); g.K = weight.size(0); g.C = weight.size(1); g.R = weight.size(2); g.S = weight.size(3);
  g.sh = stride[0]; g.sw = stride[1]; g.ph = padding[0]; g.pw = padding[1];
  g.P = input.size(2); g.Q = input.size(3);
  if (dilation.size() == 2) { g.dlh = dilation[0]; g.dlw = dilation[1]; }
  g.H = (g.P - 1) * g.sh - 2 * g.ph + g.dlh * (g.R - 1) + 1 + (output_padding.empty() ? 0 : output_padding[0]);
  g.W = (g.Q - 1) * g.sw - 2 * g.pw + g.dlw * (g.S - 1) + 1 + (output_padding.empty() ? 0 : output_padding[1]);
  return g;
}

}  // namespace

at::Tensor conv_forward_device(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& bias,
                               at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                               bool transposed, at::IntArrayRef output_padding, int64_t groups) {
  if (transposed) {
    TORCH_CHECK(groups == 1 && input.dim() == 4 && weight.dim() == 4,
                "b200 transposed conv: only dense 2-D transposed convolutions run on the device");
    TORCH_CHECK(stride[0] >= 1 && stride[0] <= 4 && stride[1] >= 1 && stride[1] <= 4, "b200 conv: strides above 4 have no device kernel");
    TORCH_CHECK(weight.size(2) * weight.size(3) <= B200_CONV_MAX_TAPS, "b200 conv: too many filter taps for the device kernel");
    TORCH_CHECK(input.size(1) == weight.size(0), "conv_transpose: channel mismatch");
    TORCH_CHECK(weight.size(0) % 8 == 0 && weight.size(1) % 8 == 0, "b200 transposed conv: channel counts must be multiples of 8");
    ConvGeom g = transposed_geom(input, weight, stride, padding, output_padding, dilation);
    TORCH_CHECK(g.H > 0 && g.W > 0, "conv_transpose: output size is too small");
    at::Tensor out = dgrad_impl(input, weight, g, input.scalar_type());
    if (bias.has_value() && bias->defined()) out.add_(bias->view({1, -1, 1, 1}));
    return out;
  }
  if (is_depthwise(input, weight, groups)) {
    check_depthwise(input, dilation, transposed);
    ConvGeom g = geom(input, weight, stride, padding);
    TORCH_CHECK(g.P > 0 && g.Q > 0, "conv: output size is too small");
    return depthwise_forward(input, weight, bias, g);
  }
  if (groups > 1) {
    // grouped: one dense convolution per group on channel slices
    TORCH_CHECK(input.size(1) % groups == 0 && weight.size(0) % groups == 0, "conv: channels not divisible by groups");
    const int64_t cg = input.size(1) / groups, kg = weight.size(0) / groups;
    std::vector<at::Tensor> outs;
    for (int64_t i = 0; i < groups; ++i) {
      std::optional<at::Tensor> bg;
      if (bias.has_value() && bias->defined()) bg = bias->narrow(0, i * kg, kg);
      outs.push_back(conv_forward_device(input.narrow(1, i * cg, cg), weight.narrow(0, i * kg, kg), bg, stride, padding, dilation,
                                         false, output_padding, 1));
    }
    return at::cat(outs, 1);
  }
  check_supported(input, weight, stride, padding, dilation, transposed, groups);
  TORCH_CHECK(input.size(1) == weight.size(1), "conv: channel mismatch");
  ConvGeom g = geom(input, weight, stride, padding, dilation);
  TORCH_CHECK(g.P > 0 && g.Q > 0, "conv: output size is too small");
  return forward_impl(input, weight, bias, g, nullptr, nullptr, 0, input.scalar_type());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> conv_backward_device(
    const at::Tensor& grad, const at::Tensor& input, const at::Tensor& weight, at::IntArrayRef stride,
    at::IntArrayRef padding, at::IntArrayRef dilation, bool transposed, at::IntArrayRef output_padding, int64_t groups,
    std::array<bool, 3> mask) {
  if (transposed) {
    TORCH_CHECK(groups == 1 && input.dim() == 4,
                "b200 transposed conv backward: only dense 2-D transposed convolutions run on the device");
    TORCH_CHECK(stride[0] <= 4 && stride[1] <= 4 && weight.size(2) * weight.size(3) <= B200_CONV_MAX_TAPS,
                "b200 transposed conv backward: stride / filter size has no device kernel");
    TORCH_CHECK(weight.size(0) % 8 == 0 && weight.size(1) % 8 == 0, "b200 transposed conv: channel counts must be multiples of 8");
    ConvGeom g = transposed_geom(input, weight, stride, padding, output_padding, dilation);
    TORCH_CHECK(g.H == grad.size(2) && g.W == grad.size(3), "conv_transpose backward: gradient shape mismatch");
    at::Tensor dx, dw, db;
    // d(input) is the forward convolution of the output gradient; d(weight) is the weight gradient of
    // that convolution with the roles of activation and gradient exchanged
    if (mask[0]) dx = forward_impl(grad, weight, std::nullopt, g, nullptr, nullptr, 0, input.scalar_type());
    if (mask[1]) dw = wgrad_impl(input, grad, weight, g);
    if (mask[2]) db = grad.sum({0, 2, 3});
    return {dx, dw, db};
  }
  if (is_depthwise(input, weight, groups)) {
    check_depthwise(input, dilation, transposed);
    return depthwise_backward(grad, input, weight, geom(input, weight, stride, padding), mask);
  }
  if (groups > 1) {
    const int64_t cg = input.size(1) / groups, kg = weight.size(0) / groups;
    std::vector<at::Tensor> dxs, dws;
    for (int64_t i = 0; i < groups; ++i) {
      auto r = conv_backward_device(grad.narrow(1, i * kg, kg), input.narrow(1, i * cg, cg), weight.narrow(0, i * kg, kg), stride,
                                    padding, dilation, false, output_padding, 1, {mask[0], mask[1], false});
      if (mask[0]) dxs.push_back(std::get<0>(r));
      if (mask[1]) dws.push_back(std::get<1>(r));
    }
    at::Tensor dx, dw, db;
    if (mask[0]) dx = at::cat(dxs, 1);
    if (mask[1]) dw = at::cat(dws, 0);
    if (mask[2]) db = grad.sum({0, 2, 3});
    return {dx, dw, db};
  }
  check_supported(input, weight, stride, padding, dilation, transposed, groups);
  ConvGeom g = geom(input, weight, stride, padding, dilation);
  at::Tensor dx, dw, db;
  if (mask[0]) {
    TORCH_CHECK(g.C % 8 == 0, "b200 conv dgrad: input channels must be a multiple of 8");
    dx = dgrad_impl(grad, weight, g, input.scalar_type());
  }
  if (mask[1]) dw = wgrad_impl(grad, input, weight, g);
  if (mask[2]) db = grad.sum({0, 2, 3});
  return {dx, dw, db};
}

// Fused inference convolution used by the fusion pass and the quantization-free
// fast path: act(conv(x, w) * scale + bias + residual).
at::Tensor conv_bn_act_device(const at::Tensor& input, const at::Tensor& weight, const std::optional<at::Tensor>& scale,
                              const std::optional<at::Tensor>& bias, const std::optional<at::Tensor>& residual,
                              at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
                              int64_t act) {
  check_supported(input, weight, stride, padding, dilation, false, groups);
  ConvGeom g = geom(input, weight, stride, padding, dilation);
  at::Tensor sc;
  const float* scp = nullptr;
  if (scale.has_value() && scale->defined()) {
    sc = scale->to(at::kFloat).contiguous();
    scp = sc.data_ptr<float>();
  }
  const at::Tensor* res = (residual.has_value() && residual->defined()) ? &*residual : nullptr;
  return forward_impl(input, weight, bias, g, scp, res, (int)act, input.scalar_type());
}

// Backward of a dense 16-bit convolution whose weight gradient is returned in fp32 (the accumulation
// buffer of the weight-gradient kernel, no rounding to the activation dtype): used when the parameter
// and its gradient are fp32 and only the compute copy of the weight is 16-bit.
// With `accum`, the weight gradient is added straight into that fp32 buffer (a flat view of memory laid out
// [K][R][S][C]) and the second result is undefined: no temporary, no separate accumulation kernel.
std::tuple<at::Tensor, at::Tensor> conv_backward_fp32w_device(const at::Tensor& grad, const at::Tensor& input,
                                                              const at::Tensor& weight, at::IntArrayRef stride,
                                                              at::IntArrayRef padding, bool need_dx, bool need_dw,
                                                              const std::optional<at::Tensor>& accum,
                                                              const std::optional<at::Tensor>& dx_add) {
  const int64_t ones[2] = {1, 1};
  if (use_cpu_path()) {
    // Host path (host simulation, force-CPU mode): the same results from the stock convolution gradient in fp32.
    const int64_t zeros[2] = {0, 0};
    std::vector<int64_t> no_bias;
    auto r = at::convolution_backward(grad.to(at::kFloat), input.to(at::kFloat), weight.to(at::kFloat), at::OptionalIntArrayRef(), stride,
                                      padding, at::IntArrayRef(ones, 2), false, at::IntArrayRef(zeros, 2), 1,
                                      {need_dx, need_dw, false});
    at::Tensor dx, dw;
    if (need_dx) {
      dx = std::get<0>(r);
      if (dx_add.has_value() && dx_add->defined()) dx = dx + dx_add->to(at::kFloat);
      dx = dx.to(input.scalar_type()).contiguous(at::MemoryFormat::ChannelsLast);
    }
    if (need_dw) {
      dw = std::get<1>(r);
      if (accum.has_value() && accum->defined()) {  // flat fp32 in the memory order [K][R][S][C]
        accum->view({dw.size(0), dw.size(2), dw.size(3), dw.size(1)}).add_(dw.permute({0, 2, 3, 1}));
        dw = at::Tensor();
      } else {
        dw = dw.contiguous(at::MemoryFormat::ChannelsLast);
      }
    }
    return {dx, dw};
  }
  check_supported(input, weight, stride, padding, at::IntArrayRef(ones, 2), false, 1);
  ConvGeom g = geom(input, weight, stride, padding);
  at::Tensor dx, dw;
  if (need_dx) {
    TORCH_CHECK(g.C % 8 == 0, "b200 conv dgrad: input channels must be a multiple of 8");
    const bool has_add = dx_add.has_value() && dx_add->defined();
    dx = dgrad_impl(grad, weight, g, input.scalar_type(), has_add ? &*dx_add : nullptr);
  }
  if (need_dw) {
    const bool has_acc = accum.has_value() && accum->defined();
    at::Tensor flat;
    if (has_acc) {
      TORCH_CHECK(is_b200(*accum) && accum->is_contiguous() && accum->dim() == 1, "conv2d_backward_fp32w: accum must be a flat device tensor");
      flat = *accum;
    }
    dw = wgrad_impl(grad, input, weight, g, /*fp32_result=*/true, has_acc ? &flat : nullptr);
  }
  return {dx, dw};
}

// Convolution that also returns the per-channel sum / sum of squares of its output
// ([2 * Cout] fp64), accumulated in the epilogue, for the batch norm that follows it.
std::tuple<at::Tensor, at::Tensor> conv_stats_device(const at::Tensor& input, const at::Tensor& weight,
                                                     at::IntArrayRef stride, at::IntArrayRef padding) {
  check_same_device("conv2d_stats", input, weight);
  const int64_t ones[2] = {1, 1};
  if (use_cpu_path()) {
    // Host path: the stock convolution, then the sums of the (rounded) result as the epilogue would have produced them
    at::Tensor y = at::conv2d(input, weight, std::nullopt, stride, padding).contiguous(at::MemoryFormat::ChannelsLast);
    at::Tensor yd = y.to(at::kDouble);
    const std::vector<int64_t> rdims{0, 2, 3};
    return {y, at::cat({yd.sum(rdims), (yd * yd).sum(rdims)})};
  }
  check_supported(input, weight, stride, padding, at::IntArrayRef(ones, 2), false, 1);
  TORCH_CHECK(input.scalar_type() != at::kFloat, "conv2d_stats: 16-bit activations only");
  TORCH_CHECK(input.size(1) == weight.size(1), "conv: channel mismatch");
  ConvGeom g = geom(input, weight, stride, padding);
  TORCH_CHECK(g.P > 0 && g.Q > 0, "conv: output size is too small");
  TORCH_CHECK(g.K % 64 == 0, "conv2d_stats: output channels must be a multiple of 64");
  at::Tensor sums = at::zeros({2 * g.K}, input.options().dtype(at::kDouble));
  at::Tensor out = forward_impl(input, weight, std::nullopt, g, nullptr, nullptr, 0, input.scalar_type(), sums.data_ptr<double>());
  return {out, sums};
}

}  // namespace ops
}  // namespace catch_b200
