// C++ tests of the fusion passes and the fusion-group runner cache on plain IR (no Python):
// lowering, the partitioner's grouping and alias safety, un-fusing, runner sharing, execution of a
// group through the graph executor, and the shared checking helpers.
// Reference suites: torch_mlu/csrc/test/jit/{fuser_test,codegen_test,runtime_test}.cpp,
// torch_mlu/csrc/test/common/test_assert_tensor.cpp.
#include <torch/csrc/jit/ir/irparser.h>
#include <torch/csrc/jit/runtime/graph_executor.h>

#include <cstdio>

#include "../jit/fusion.h"
#include "../runtime/check_util.h"

using namespace torch::jit;
using namespace catch_b200;

extern int g_failures, g_checks;
#define CHECK_J(cond)                                                              \
  do {                                                                             \
    ++g_checks;                                                                    \
    if (!(cond)) {                                                                 \
      ++g_failures;                                                                \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
    }                                                                              \
  } while (0)

namespace {

int count_kind(const std::shared_ptr<Graph>& g, const char* kind) {
  int n = 0;
  for (Node* node : g->nodes()) n += node->kind().toQualString() == std::string(kind) ? 1 : 0;
  return n;
}

std::shared_ptr<Graph> parse(const char* ir) {
  auto g = std::make_shared<Graph>();
  parseIR(ir, g.get());
  return g;
}

}  // namespace

void test_jit_lowering() {
  auto g = parse(R"IR(
    graph(%x : Tensor):
      %p : float = prim::Constant[value=0.5]()
      %f : bool = prim::Constant[value=0]()
      %one : int = prim::Constant[value=1]()
      %none : NoneType = prim::Constant()
      %d : Tensor = aten::dropout(%x, %p, %f)
      %c : Tensor = aten::contiguous(%d, %one)
      %r : Tensor = aten::relu(%c)
      %y : Tensor = aten::mean(%r, %none)
      return (%y))IR");
  jit::LowerGraph(g);
  CHECK_J(count_kind(g, "aten::dropout") == 0);
  CHECK_J(count_kind(g, "aten::contiguous") == 0);  // nothing after it depends on strides (the reduction writes a fresh result)
  CHECK_J(count_kind(g, "aten::relu") == 1);
  // ... but in front of a view, or when the result leaves the graph, it stays
  auto g2 = parse(R"IR(
    graph(%x : Tensor):
      %one : int = prim::Constant[value=1]()
      %zero : int = prim::Constant[value=0]()
      %m1 : int = prim::Constant[value=-1]()
      %t : Tensor = aten::transpose(%x, %zero, %one)
      %c : Tensor = aten::contiguous(%t, %zero)
      %r : Tensor = aten::relu(%c)
      %shape : int[] = prim::ListConstruct(%m1)
      %v : Tensor = aten::view(%r, %shape)
      %c2 : Tensor = aten::contiguous(%t, %zero)
      return (%v, %c2))IR");
  jit::LowerGraph(g2);
  CHECK_J(count_kind(g2, "aten::contiguous") == 2);
}

void test_jit_partitioner() {
  // supported chain -> one group; the unsupported op in the middle splits it
  auto g = parse(R"IR(
    graph(%x : Tensor, %y : Tensor):
      %one : int = prim::Constant[value=1]()
      %a : Tensor = aten::add(%x, %y, %one)
      %b : Tensor = aten::relu(%a)
      %c : Tensor = aten::mul(%b, %y)
      %d : Tensor = aten::erfinv(%c)
      %e : Tensor = aten::sigmoid(%d)
      %f : Tensor = aten::tanh(%e)
      return (%f))IR");
  jit::SegmentGraph(g);
  CHECK_J(count_kind(g, "catch_b200::FusionGroup") == 2);
  CHECK_J(count_kind(g, "aten::erfinv") == 1);
  CHECK_J(count_kind(g, "aten::relu") == 0 && count_kind(g, "aten::tanh") == 0);
  // groups execute: same numbers as the plain graph
  auto plain = parse(R"IR(
    graph(%x : Tensor, %y : Tensor):
      %one : int = prim::Constant[value=1]()
      %a : Tensor = aten::add(%x, %y, %one)
      %b : Tensor = aten::relu(%a)
      %c : Tensor = aten::mul(%b, %y)
      %d : Tensor = aten::erfinv(%c)
      %e : Tensor = aten::sigmoid(%d)
      %f : Tensor = aten::tanh(%e)
      return (%f))IR");
  at::Tensor x = at::rand({4, 5}) * 0.5, y = at::rand({4, 5}) * 0.5;
  Stack s1{x, y}, s2{x, y};
  GraphExecutor(g, "grouped").run(s1);
  GraphExecutor(plain, "plain").run(s2);
  assertTensorsEqual(s1.back().toTensor(), s2.back().toTensor(), 1e-6);
  ++g_checks;
  // dissolving the groups gives the original operators back
  jit::UnfuseGraph(g);
  CHECK_J(count_kind(g, "catch_b200::FusionGroup") == 0);
  CHECK_J(count_kind(g, "aten::relu") == 1 && count_kind(g, "aten::sigmoid") == 1 && count_kind(g, "aten::tanh") == 1);
}

void test_jit_alias_safety() {
  // relu_ writes its input in place: the earlier read of %x by aten::neg (unsupported, stays outside) must not
  // move behind the group that holds the write
  auto g = parse(R"IR(
    graph(%x : Tensor):
      %one : int = prim::Constant[value=1]()
      %n : Tensor = aten::neg(%x)
      %r : Tensor = aten::relu_(%x)
      %s : Tensor = aten::add(%r, %n, %one)
      %t : Tensor = aten::sigmoid(%s)
      return (%t))IR");
  jit::SegmentGraph(g);
  at::Tensor x = at::randn({16});
  at::Tensor expect = at::sigmoid(at::relu(x) + at::neg(x));
  Stack s{x.clone()};
  GraphExecutor(g, "alias").run(s);
  assertTensorsEqual(s.back().toTensor(), expect, 1e-6);
  ++g_checks;
}

void test_jit_runner_cache() {
  const char* ir = R"IR(
    graph(%x : Tensor):
      %a : Tensor = aten::relu(%x)
      %b : Tensor = aten::sigmoid(%a)
      %c : Tensor = aten::tanh(%b)
      return (%c))IR";
  jit::fusion_cache_clear();
  const int64_t compiles0 = jit::fusion_compile_count();
  {
    auto g1 = parse(ir), g2 = parse(ir);
    jit::SegmentGraph(g1);
    jit::SegmentGraph(g2);
    GraphExecutor e1(g1, "one"), e2(g2, "two");
    Stack s1{at::randn({3, 3})}, s2{at::randn({3, 3})};
    e1.run(s1);
    e2.run(s2);
    CHECK_J(jit::fusion_cache_size() == 1);  // identical groups share one runner
    CHECK_J(jit::fusion_compile_count() == compiles0 + 1);
    Stack s3{at::randn({7})};  // another shape: a new plan of the same runner
    e1.run(s3);
    CHECK_J(jit::fusion_cache_size() == 1);
    CHECK_J(jit::fusion_compile_count() == compiles0 + 2);
  }
  // the executors are gone: the cache only observed their runner
  CHECK_J(jit::fusion_cache_size() == 0);
}

void test_check_util() {
  at::Tensor a = at::ones({4, 4});
  at::Tensor b = a + 0.01;
  assertTensorsEqual(a, b, 0.011);
  assertTensorsEqual(a, b, 0.011, /*use_MSE=*/true);
  assertTensorsEqual(a, b, 0.011, false, /*use_RAE=*/true);
  assertTensorsEqual(a, b, 0.0, false, false, /*use_RMA=*/true);  // b's mean is larger: the signed measure is negative
  bool threw = false;
  try {
    assertTensorsEqual(a, b, 0.001);
  } catch (const c10::Error& e) {
    threw = std::string(e.what()).find("maximum absolute error") != std::string::npos;
  }
  CHECK_J(threw);
  threw = false;
  try {
    assertTensorsEqual(a, at::ones({2, 2}), 1.0);
  } catch (const c10::Error&) {
    threw = true;
  }
  CHECK_J(threw);
  const TensorDiff d = tensorDiff(at::zeros({8}), at::zeros({8}));
  CHECK_J(d.max_abs == 0 && d.rel_rms == 0 && d.rel_abs == 0 && d.rel_mean == 0);
  at::Tensor infos = at::tensor({0, 2, 0, -1}, at::kInt);
  CHECK_J(batchCheckErrors(infos, "cholesky") == 2);
  CHECK_J(batchCheckErrors(infos, "lu", /*allow_singular=*/true) == 1);
  CHECK_J(batchCheckErrors(at::zeros({3}, at::kInt), "svd") == 0);
}
