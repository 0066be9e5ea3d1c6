#include <torch/csrc/jit/ir/alias_analysis.h>
#include <torch/csrc/jit/passes/common_subexpression_elimination.h>
#include <torch/csrc/jit/passes/constant_propagation.h>
#include <torch/csrc/jit/passes/dead_code_elimination.h>
#include <torch/csrc/jit/passes/inliner.h>
#include <torch/csrc/jit/passes/lower_tuples.h>
#include <torch/csrc/jit/passes/pass_manager.h>
#include <torch/csrc/jit/passes/remove_dropout.h>
#include <torch/csrc/jit/passes/remove_mutation.h>
#include <torch/csrc/jit/ir/subgraph_matcher.h>
#include <torch/csrc/jit/passes/subgraph_rewrite.h>
#include <torch/csrc/jit/passes/utils/subgraph_utils.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <sstream>
#include <unordered_set>

#include "../runtime/log.h"
#include "fusion.h"

namespace catch_b200 {
namespace jit {

using namespace torch::jit;

namespace {
std::atomic<bool> g_enabled{true};
}
bool fusion_enabled() { return g_enabled.load(); }
void set_fusion_enabled(bool on) { g_enabled.store(on); }

// ------------------------------------------------------------------------ lowering
namespace {

// prim::If whose taken branch only raises: keep the other branch's effects.
bool block_only_raises(Block* b) {
  bool raises = false;
  for (Node* n : b->nodes()) {
    if (n->kind() == prim::RaiseException) raises = true;
    else if (n->kind() != prim::Constant && n->kind() != aten::format && n->kind() != prim::ListConstruct &&
             n->kind() != aten::str)
      return false;
  }
  return raises;
}

void eliminate_exception_ifs(Block* block) {
  for (auto it = block->nodes().begin(); it != block->nodes().end();) {
    Node* n = *it;
    ++it;
    for (Block* b : n->blocks()) eliminate_exception_ifs(b);
    if (n->kind() != prim::If || n->outputs().size() != 0) continue;
    Block* t = n->blocks()[0];
    Block* f = n->blocks()[1];
    const bool t_raises = block_only_raises(t), f_raises = block_only_raises(f);
    const bool t_empty = t->nodes().begin() == t->nodes().end(), f_empty = f->nodes().begin() == f->nodes().end();
    if ((t_raises && f_empty) || (f_raises && t_empty) || (t_raises && f_raises)) n->destroy();
  }
}

// Does anything downstream of `v` depend on v's strides?  view() and its relatives do, and so does whoever receives
// a graph output; operators that write a fresh dense result (convolutions, GEMMs, reductions, pooling, cat, reshape ...)
// cut the dependence; everything else (element-wise operators keep their input's strides, transpose / slice / chunk
// build their strides from it) passes it on.
bool strides_matter(Value* v, std::unordered_set<Value*>& seen) {
  if (!seen.insert(v).second) return false;
  static const std::unordered_set<std::string> sensitive = {
      "aten::view", "aten::view_as", "aten::as_strided", "aten::unflatten", "aten::stride", "aten::is_contiguous",
      "aten::unfold", "aten::_unsafe_view", "aten::resize_", "aten::set_"};
  static const std::unordered_set<std::string> fresh = {
      "aten::conv2d", "aten::_convolution", "aten::convolution", "aten::linear", "aten::matmul", "aten::mm", "aten::bmm",
      "aten::addmm", "aten::cat", "aten::stack", "aten::max_pool2d", "aten::avg_pool2d", "aten::adaptive_avg_pool2d",
      "aten::adaptive_max_pool2d", "aten::mean", "aten::sum", "aten::softmax", "aten::log_softmax", "aten::layer_norm",
      "aten::batch_norm", "aten::reshape", "aten::flatten", "aten::contiguous", "aten::upsample_nearest2d", "aten::size",
      "aten::embedding", "aten::argmax", "aten::max", "aten::min", "aten::topk", "aten::sort",
      "catch_b200::conv_bn_act", "catch_b200::linear_act", "catch_b200::qconv_act", "catch_b200::conv2d", "catch_b200::linear"};
  for (const Use& u : v->uses()) {
    Node* user = u.user;
    if (user->kind() == prim::Return) return true;
    const std::string kind = user->kind().toQualString();
    if (sensitive.count(kind)) return true;
    if (fresh.count(kind)) continue;
    for (Value* out : user->outputs())
      if (strides_matter(out, seen)) return true;
  }
  return false;
}

// x.contiguous() is dropped where nothing downstream can tell the difference (the copy it may make is pure cost
// there); in front of a view() -- the channel shuffle of ShuffleNet -- or of a graph output it stays.
void remove_contiguous(Block* block) {
  for (auto it = block->nodes().begin(); it != block->nodes().end();) {
    Node* n = *it;
    ++it;
    for (Block* b : n->blocks()) remove_contiguous(b);
    if (n->kind() == aten::contiguous) {
      std::unordered_set<Value*> seen;
      if (strides_matter(n->output(), seen)) continue;
      n->output()->replaceAllUsesWith(n->input(0));
      n->destroy();
    }
  }
}

// Tracing records convolutions as the 13-argument aten::_convolution; the fusion patterns
// are written against aten::conv2d, so non-transposed 2-D instances are rewritten to it.
void canonicalize_convolution(std::shared_ptr<Graph>& graph) {
  const std::string traced = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %t, %op, %g, %bm, %det, %cud, %tf32):
      %y = aten::_convolution(%x, %w, %b, %s, %p, %d, %t, %op, %g, %bm, %det, %cud, %tf32)
      return (%y))IR";
  const std::string plain = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %t, %op, %g, %bm, %det, %cud, %tf32):
      %y = aten::conv2d(%x, %w, %b, %s, %p, %d, %g)
      return (%y))IR";
  auto is_plain_2d = [](const Match& m, const std::unordered_map<std::string, Value*>& vmap) {
    auto t = toIValue(m.values_map.at(vmap.at("t")));
    auto s = toIValue(m.values_map.at(vmap.at("s")));
    auto p = toIValue(m.values_map.at(vmap.at("p")));
    auto d = toIValue(m.values_map.at(vmap.at("d")));
    return t.has_value() && t->isBool() && !t->toBool() && s.has_value() && s->isIntList() && s->toIntList().size() == 2 &&
           p.has_value() && p->isIntList() && p->toIntList().size() == 2 && d.has_value() && d->isIntList() &&
           d->toIntList().size() == 2;
  };
  SubgraphRewriter rw;
  rw.RegisterRewritePattern(traced, plain);
  rw.runOnGraph(graph, is_plain_2d);
}

}  // namespace

void LowerGraph(std::shared_ptr<Graph>& graph) {
  if (!fusion_enabled()) return;
  Inline(*graph);
  LowerSimpleTuples(graph);
  canonicalize_convolution(graph);
  eliminate_exception_ifs(graph->block());
  removeDropout(graph);
  RemoveTensorMutation(graph);
  remove_contiguous(graph->block());
  ConstantPropagation(graph);
  EliminateCommonSubexpression(graph);
  EliminateDeadCode(graph);
}

// -------------------------------------------------------------------- kernel fusion
namespace {

// Input scale of a quantized convolution node when it is known at pass time (frozen module: the scale and mode
// tensors are constants) and the layer is active; 0 otherwise.
double constant_input_scale(Node* n) {
  static const Symbol qconv = Symbol::fromQualString("catch_b200::qconv_act");
  if (n->kind() != qconv) return 0.0;
  auto qs = toIValue(n->input(7));
  auto qm = toIValue(n->input(8));
  if (!qs.has_value() || !qs->isTensor() || qs->toTensor().numel() == 0) return 0.0;
  if (qm.has_value() && qm->isTensor() && qm->toTensor().numel() > 0 &&
      qm->toTensor().cpu().to(at::kDouble).view({-1})[0].item<double>() == 0.0) return 0.0;
  if (qm.has_value() && !qm->isTensor() && !qm->isNone()) return 0.0;
  if (!qm.has_value()) return 0.0;  // mode decided at run time
  return qs->toTensor().cpu().to(at::kDouble).view({-1})[0].item<double>();
}

// A quantized convolution whose result is consumed only as the input of quantized convolutions that share one
// input scale emits int8 quantized with that scale: the consumers skip their quantization pass and the
// activation crosses memory at one byte per element.
void chain_quantized(Block* block) {
  static const Symbol qconv = Symbol::fromQualString("catch_b200::qconv_act");
  for (Node* n : block->nodes()) {
    for (Block* b : n->blocks()) chain_quantized(b);
    if (n->kind() != qconv) continue;
    auto os = toIValue(n->input(11));
    if (!os.has_value() || !os->isDouble() || os->toDouble() != 0.0) continue;
    if (constant_input_scale(n) == 0.0) continue;  // an unquantized producer keeps its floating-point result
    const auto& uses = n->output()->uses();
    if (uses.empty()) continue;
    double scale = 0.0;
    bool ok = true;
    for (const Use& u : uses) {
      const double s = u.offset == 0 ? constant_input_scale(u.user) : 0.0;
      if (s == 0.0 || (scale != 0.0 && s != scale)) { ok = false; break; }
      scale = s;
    }
    if (!ok) continue;
    WithInsertPoint guard(n);
    n->replaceInput(11, block->owningGraph()->insertConstant(scale));
    n->output()->setType(TensorType::get());
  }
}

}  // namespace

void FuseKernels(std::shared_ptr<Graph>& graph) {
  if (!fusion_enabled()) return;
  // Longest chains first.  `%none` placeholders are created inside the replacement.
  const std::string conv_add_relu = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g, %res, %alpha):
      %y = aten::conv2d(%x, %w, %b, %s, %p, %d, %g)
      %z = aten::add(%y, %res, %alpha)
      %r = aten::relu(%z)
      return (%r))IR";
  const std::string conv_add_relu_fused = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g, %res, %alpha):
      %none : NoneType = prim::Constant()
      %act : int = prim::Constant[value=1]()
      %r = catch_b200::conv_bn_act(%x, %w, %none, %b, %res, %s, %p, %d, %g, %act)
      return (%r))IR";
  const std::string conv_relu = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g):
      %y = aten::conv2d(%x, %w, %b, %s, %p, %d, %g)
      %r = aten::relu(%y)
      return (%r))IR";
  const std::string conv_relu_fused = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g):
      %none : NoneType = prim::Constant()
      %act : int = prim::Constant[value=1]()
      %r = catch_b200::conv_bn_act(%x, %w, %none, %b, %none, %s, %p, %d, %g, %act)
      return (%r))IR";
  const std::string conv_only = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g):
      %y = aten::conv2d(%x, %w, %b, %s, %p, %d, %g)
      return (%y))IR";
  const std::string conv_only_fused = R"IR(
    graph(%x, %w, %b, %s, %p, %d, %g):
      %none : NoneType = prim::Constant()
      %act : int = prim::Constant[value=0]()
      %y = catch_b200::conv_bn_act(%x, %w, %none, %b, %none, %s, %p, %d, %g, %act)
      return (%y))IR";
  const std::string linear_relu = R"IR(
    graph(%x, %w, %b):
      %y = aten::linear(%x, %w, %b)
      %r = aten::relu(%y)
      return (%r))IR";
  const std::string linear_relu_fused = R"IR(
    graph(%x, %w, %b):
      %act : int = prim::Constant[value=1]()
      %r = catch_b200::linear_act(%x, %w, %b, %act)
      return (%r))IR";
  const std::string linear_gelu = R"IR(
    graph(%x, %w, %b, %approx):
      %y = aten::linear(%x, %w, %b)
      %r = aten::gelu(%y, %approx)
      return (%r))IR";
  const std::string linear_gelu_fused = R"IR(
    graph(%x, %w, %b, %approx):
      %act : int = prim::Constant[value=2]()
      %r = catch_b200::linear_act(%x, %w, %b, %act)
      return (%r))IR";
  const std::string linear_only = R"IR(
    graph(%x, %w, %b):
      %y = aten::linear(%x, %w, %b)
      return (%y))IR";
  const std::string linear_only_fused = R"IR(
    graph(%x, %w, %b):
      %act : int = prim::Constant[value=0]()
      %y = catch_b200::linear_act(%x, %w, %b, %act)
      return (%y))IR";

  // Quantized convolutions (catch_b200::conv2d carries the calibrated scales): the same three chains.
  const std::string qconv_args = "%x, %w, %b, %p, %s, %d, %g, %qs, %qm";
  const std::string qconv_add_relu = "graph(" + qconv_args + R"IR(, %res, %alpha):
      %y = catch_b200::conv2d()IR" + qconv_args + R"IR()
      %z = aten::add(%y, %res, %alpha)
      %r = aten::relu(%z)
      return (%r))IR";
  const std::string qconv_add_relu_fused = "graph(" + qconv_args + R"IR(, %res, %alpha):
      %act : int = prim::Constant[value=1]()
      %os : float = prim::Constant[value=0.]()
      %r = catch_b200::qconv_act()IR" + qconv_args + R"IR(, %res, %act, %os)
      return (%r))IR";
  const std::string qconv_relu = "graph(" + qconv_args + R"IR():
      %y = catch_b200::conv2d()IR" + qconv_args + R"IR()
      %r = aten::relu(%y)
      return (%r))IR";
  const std::string qconv_relu_fused = "graph(" + qconv_args + R"IR():
      %none : NoneType = prim::Constant()
      %act : int = prim::Constant[value=1]()
      %os : float = prim::Constant[value=0.]()
      %r = catch_b200::qconv_act()IR" + qconv_args + R"IR(, %none, %act, %os)
      return (%r))IR";
  const std::string qconv_only = "graph(" + qconv_args + R"IR():
      %y = catch_b200::conv2d()IR" + qconv_args + R"IR()
      return (%y))IR";
  const std::string qconv_only_fused = "graph(" + qconv_args + R"IR():
      %none : NoneType = prim::Constant()
      %act : int = prim::Constant[value=0]()
      %os : float = prim::Constant[value=0.]()
      %y = catch_b200::qconv_act()IR" + qconv_args + R"IR(, %none, %act, %os)
      return (%y))IR";

  // the residual pattern only applies when alpha == 1
  auto alpha_is_one = [](const Match& m, const std::unordered_map<std::string, Value*>& vmap) {
    Value* a = m.values_map.at(vmap.at("alpha"));
    auto v = toIValue(a);
    return v.has_value() && ((v->isInt() && v->toInt() == 1) || (v->isDouble() && v->toDouble() == 1.0));
  };
  auto gelu_exact = [](const Match& m, const std::unordered_map<std::string, Value*>& vmap) {
    Value* a = m.values_map.at(vmap.at("approx"));
    auto v = toIValue(a);
    return v.has_value() && v->isString() && v->toStringRef() == "none";
  };
  {
    SubgraphRewriter rw;
    rw.RegisterRewritePattern(conv_add_relu, conv_add_relu_fused);
    rw.RegisterRewritePattern(qconv_add_relu, qconv_add_relu_fused);
    rw.runOnGraph(graph, alpha_is_one);
  }
  {
    SubgraphRewriter rw;
    rw.RegisterRewritePattern(conv_relu, conv_relu_fused);
    rw.RegisterRewritePattern(qconv_relu, qconv_relu_fused);
    rw.RegisterRewritePattern(linear_relu, linear_relu_fused);
    rw.runOnGraph(graph);
  }
  {
    SubgraphRewriter rw;
    rw.RegisterRewritePattern(linear_gelu, linear_gelu_fused);
    rw.runOnGraph(graph, gelu_exact);
  }
  {
    SubgraphRewriter rw;
    rw.RegisterRewritePattern(conv_only, conv_only_fused);
    rw.RegisterRewritePattern(qconv_only, qconv_only_fused);
    rw.RegisterRewritePattern(linear_only, linear_only_fused);
    rw.runOnGraph(graph);
  }
  chain_quantized(graph->block());
  EliminateDeadCode(graph);
}

// --------------------------------------------------------------------- partitioner
namespace {

const Symbol& fusion_kind() {
  static Symbol s = Symbol::fromQualString("catch_b200::FusionGroup");
  return s;
}

std::unordered_set<std::string> forced_fallback_ops() {
  std::unordered_set<std::string> out;
  const char* env = std::getenv("CATCH_B200_FORCED_FALLBACK_OPS");
  if (!env) return out;
  std::stringstream ss(env);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    if (!tok.empty()) out.insert(tok);
  }
  return out;
}

const std::unordered_set<std::string>& supported_ops() {
  static const std::unordered_set<std::string> ops = {
      "catch_b200::conv_bn_act", "catch_b200::linear_act", "catch_b200::qconv_act", "catch_b200::conv2d",
      "catch_b200::linear", "aten::relu", "aten::relu_", "aten::hardtanh",
      "aten::hardtanh_", "aten::batch_norm", "aten::cat", "aten::conv2d", "aten::_convolution", "aten::add",
      "aten::sub", "aten::mul", "aten::div", "aten::floor", "aten::addmm", "aten::linear", "aten::matmul",
      "aten::max_pool2d", "aten::avg_pool2d", "aten::adaptive_avg_pool2d", "aten::reshape", "aten::view",
      "aten::transpose", "aten::t", "aten::flatten", "aten::permute", "aten::stack", "aten::to",
      "aten::upsample_nearest2d", "aten::sigmoid", "aten::tanh", "aten::gelu", "aten::softmax", "aten::layer_norm",
      "aten::mean", "aten::size", "aten::Int", "prim::ListConstruct", "prim::NumToTensor", "aten::contiguous",
      "aten::dropout", "aten::clamp", "aten::leaky_relu", "aten::silu"};
  return ops;
}

}  // namespace

bool isSupported(const Node* n) {
  static const auto blacklist = forced_fallback_ops();
  const std::string name = n->kind().toQualString();
  if (blacklist.count(name)) return false;
  if (n->kind() == prim::Constant || n->kind() == prim::GetAttr) return false;  // stay outside, become inputs
  if (!n->blocks().empty()) return false;                                      // no control flow inside groups
  return supported_ops().count(name) > 0;
}

namespace {

bool produces_tensor(const Node* n) {
  for (const Value* v : n->outputs())
    if (v->type()->isSubtypeOf(*TensorType::get())) return true;
  return false;
}

// Non-tensor outputs (ints, lists) may only be consumed inside the group.
bool non_tensor_outputs_stay_inside(Node* producer, Node* group) {
  for (Value* v : producer->outputs()) {
    if (v->type()->isSubtypeOf(*TensorType::get())) continue;
    for (const Use& u : v->uses())
      if (u.user != group) return false;
  }
  return true;
}

std::optional<Node*> try_fuse(Node* consumer, Value* producer_value, AliasDb& db) {
  Node* producer = producer_value->node();
  if (producer->owningBlock() != consumer->owningBlock()) return std::nullopt;
  const bool group_producer = producer->kind() == fusion_kind();
  if (!group_producer && !isSupported(producer)) return std::nullopt;
  if (!db.moveBeforeTopologicallyValid(producer, consumer)) return std::nullopt;
  // every refusal comes before the consumer is wrapped: wrapping destroys the consumer node, and the caller goes on
  // to its next input with the same pointer when this returns nothing
  if (!group_producer && !non_tensor_outputs_stay_inside(producer, consumer)) return std::nullopt;
  Node* group = consumer;
  if (consumer->kind() != fusion_kind()) {
    if (!produces_tensor(consumer)) return std::nullopt;
    group = SubgraphUtils::createSingletonSubgraphAndUpdateAliasing(consumer, fusion_kind(), db);
  }
  SubgraphUtils::mergeNodeIntoSubgraphAndUpdateAliasing(producer, group, db);
  return group;
}

std::pair<graph_node_list::iterator, bool> scan_node(Node* consumer, AliasDb& db) {
  if (consumer->kind() == fusion_kind() || isSupported(consumer)) {
    // visit inputs in reverse topological order so producers closest to the consumer merge first
    std::vector<Value*> inputs(consumer->inputs().begin(), consumer->inputs().end());
    std::sort(inputs.begin(), inputs.end(), [](Value* a, Value* b) { return a->node()->isAfter(b->node()); });
    for (Value* in : inputs) {
      if (in->node()->kind() == prim::Param) continue;
      auto group = try_fuse(consumer, in, db);
      if (group) return {(*group)->reverseIterator(), true};
    }
  }
  return {++consumer->reverseIterator(), false};
}

void fuse_block(Block* block, std::shared_ptr<Graph>& graph) {
  bool any = true;
  while (any) {
    any = false;
    AliasDb db(graph);
    for (auto it = block->nodes().rbegin(); it != block->nodes().rend();) {
      bool changed;
      std::tie(it, changed) = scan_node(*it, db);
      any |= changed;
    }
  }
  // a lone supported tensor op still becomes a (singleton) group when it is a fused kernel
  {
    AliasDb db(graph);
    for (auto it = block->nodes().begin(); it != block->nodes().end();) {
      Node* n = *it;
      ++it;
      const std::string name = n->kind().toQualString();
      if (name == "catch_b200::conv_bn_act" || name == "catch_b200::linear_act")
        SubgraphUtils::createSingletonSubgraphAndUpdateAliasing(n, fusion_kind(), db);
    }
  }
  for (Node* n : block->nodes())
    for (Block* b : n->blocks()) fuse_block(b, graph);
}

}  // namespace

void SegmentGraph(std::shared_ptr<Graph>& graph) {
  if (!fusion_enabled()) return;
  fuse_block(graph->block(), graph);
  EliminateCommonSubexpression(graph);
  EliminateDeadCode(graph);
}

// Inverse of SegmentGraph: the nodes of every fusion group go back into the surrounding graph.  A module
// has to be in this form to be serialised (a subgraph attribute has no textual form in a saved module).
void UnfuseGraph(std::shared_ptr<Graph>& graph) {
  std::function<void(Block*)> walk = [&](Block* block) {
    for (auto it = block->nodes().begin(); it != block->nodes().end();) {
      Node* n = *it;
      ++it;
      for (Block* b : n->blocks()) walk(b);
      if (n->kind() == fusion_kind()) SubgraphUtils::unmergeSubgraph(n);
    }
  };
  walk(graph->block());
  EliminateDeadCode(graph);
}

void register_passes() {
  static std::once_flag once;
  std::call_once(once, [] {
    registerPrePass([](std::shared_ptr<Graph>& g) { LowerGraph(g); });
    registerPrePass([](std::shared_ptr<Graph>& g) { FuseKernels(g); });
    registerPrePass([](std::shared_ptr<Graph>& g) { SegmentGraph(g); });
  });
}

}  // namespace jit
}  // namespace catch_b200
