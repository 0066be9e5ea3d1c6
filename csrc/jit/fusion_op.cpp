// The catch_b200::FusionGroup operator: runner cache keyed by the canonical graph
// text, per-runner plans keyed by argument dtypes / shapes / device, interpreter
// fallback, and the debug mode that also runs the group on the CPU.
// Reference: torch_mlu/csrc/jit/partition/customer_partition_manager.cpp:51-72,
// runtime/runner_cache.cpp:44-85, runtime/graph_runner.cpp:55-238.
#include <torch/csrc/jit/passes/canonicalize.h>
#include <torch/csrc/jit/runtime/custom_operator.h>
#include <torch/csrc/jit/runtime/interpreter.h>
#include <torch/csrc/jit/serialization/pickle.h>

#include <atomic>
#include <fstream>
#include <mutex>
#include <sstream>
#include <unordered_map>

#include "../runtime/backend.h"
#include "../runtime/device.h"
#include "../runtime/graph.h"
#include "../runtime/log.h"
#include "../runtime/notifier.h"
#include "../runtime/queue.h"
#include "../runtime/tensor_impl.h"
#include "fusion.h"

namespace catch_b200 {
namespace jit {

using namespace torch::jit;

namespace {

std::atomic<int64_t> g_compiles{0}, g_fallbacks{0}, g_graph_captures{0}, g_graph_replays{0};

// A compiled group plus, once the same argument shapes have been seen a few times, its captured device graph:
// the group then costs one submission instead of one per kernel.  CATCH_B200_JIT_GRAPHS=0 keeps the interpreter.
struct Plan {
  std::shared_ptr<Code> code;
  std::mutex mu;                 // the static buffers of a captured plan serve one call at a time
  int eager_runs = 0;
  int graph_state = 0;           // 0 undecided, 1 captured, -1 cannot be captured
  std::unique_ptr<DeviceGraph> graph;
  std::vector<at::Tensor> static_in, static_out;
};

bool graphs_wanted() {
  static const bool on = [] {
    const char* e = std::getenv("CATCH_B200_JIT_GRAPHS");
    return !(e && std::string(e) == "0");
  }();
  return on && backend().supports_graphs();
}

std::string arg_spec(const Stack& stack, size_t n_inputs) {
  std::ostringstream os;
  for (size_t i = stack.size() - n_inputs; i < stack.size(); ++i) {
    const IValue& v = stack[i];
    if (v.isTensor()) {
      const at::Tensor& t = v.toTensor();
      if (!t.defined()) { os << "U;"; continue; }
      os << static_cast<int>(t.scalar_type()) << t.sizes() << "@" << t.device() << (t.is_contiguous() ? "c" : "s") << ";";
    } else {
      os << "_;";
    }
  }
  return os.str();
}

class FusedRunner {
 public:
  explicit FusedRunner(std::shared_ptr<Graph> g) : graph_(std::move(g)), fallback_(graph_, "b200_fusion_fallback") {}

  void run(Stack& stack) {
    const size_t n_in = graph_->inputs().size();
    const std::string spec = arg_spec(stack, n_in);
    std::shared_ptr<Plan> plan;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = plans_.find(spec);
      if (it != plans_.end()) plan = it->second;
    }
    // The interpreter consumes the group's inputs from the stack, so they are kept aside: the
    // op-by-op fallback (and the debug comparison) start again from them.
    const Stack saved(stack.end() - n_in, stack.end());
    const size_t base = stack.size() - n_in;
    const char* dbg = std::getenv("CATCH_B200_FUSED_KERNEL_DEBUG");
    try {
      if (!plan) plan = compile(spec, stack, n_in);
      if (!dbg && graphs_wanted() && run_graphed(*plan, stack, saved, base)) return;
      InterpreterState(*plan->code).run(stack);
      plan->eager_runs++;
    } catch (const c10::OutOfMemoryError&) {
      throw;
    } catch (const std::exception& e) {
      TORCH_WARN("b200 fusion group failed (", e.what(), "); running it op by op instead.");
      g_fallbacks++;
      stack.resize(base);  // drop whatever the failed plan left behind
      run_fallback(stack, saved);
      return;
    }
    if (dbg) debug_compare(dbg, saved, stack);
  }

  size_t plan_count() {
    std::lock_guard<std::mutex> g(mu_);
    return plans_.size();
  }

 private:
  // Replays (after capturing, on the third call with these shapes) the plan's device graph.  Returns false when
  // this call has to go through the interpreter; the stack is untouched then.
  bool run_graphed(Plan& plan, Stack& stack, const Stack& inputs, size_t base) {
    if (plan.graph_state < 0 || (plan.graph_state == 0 && plan.eager_runs < 2)) return false;
    int device = -1;
    for (const IValue& v : inputs) {
      if (!v.isTensor() || !v.toTensor().defined()) return false;  // scalars would be baked into the graph
      const at::Tensor& t = v.toTensor();
      if (!is_b200(t) || (device >= 0 && t.device().index() != device)) return false;
      if (t.requires_grad() && at::GradMode::is_enabled()) return false;
      device = t.device().index();
    }
    if (device < 0) return false;
    std::lock_guard<std::mutex> lk(plan.mu);
    if (plan.graph_state == 0 && !capture(plan, inputs, device)) return false;
    if (plan.graph_state != 1) return false;
    for (size_t i = 0; i < inputs.size(); ++i) {
      const at::Tensor& src = inputs[i].toTensor();
      if (src.data_ptr() != plan.static_in[i].data_ptr()) plan.static_in[i].copy_(src, /*non_blocking=*/true);
    }
    plan.graph->replay();
    g_graph_replays++;
    stack.resize(base);
    // the static outputs are overwritten by the next call: hand out copies
    for (const at::Tensor& o : plan.static_out) stack.emplace_back(o.clone());
    return true;
  }

  bool capture(Plan& plan, const Stack& inputs, int device) {
    plan.graph_state = -1;  // until proven otherwise
    DeviceSwitch sw(device);
    std::vector<at::Tensor> statics;
    for (const IValue& v : inputs) statics.push_back(v.toTensor().clone());
    const Queue main = getCurrentQueue(device), side = getQueueFromPool(device);
    {
      Notifier ready(false);
      ready.place(main);
      ready.wait(side);
    }
    auto graph = std::make_unique<DeviceGraph>();
    Stack st;
    bool ok = false;
    {
      QueueGuard qg(side);
      try {
        graph->capture_begin();
        for (const at::Tensor& t : statics) st.emplace_back(t);
        InterpreterState(*plan.code).run(st);
        ok = graph->capture_end();
      } catch (const std::exception& e) {
        graph->capture_abort();
        B200LOG(DBG) << "fusion group not captured as a device graph: " << e.what();
        ok = false;
      }
    }
    {
      Notifier done(false);
      done.place(side);
      done.wait(main);
    }
    if (!ok) return false;
    std::vector<at::Tensor> outs;
    for (const IValue& v : st) {
      if (!v.isTensor() || !v.toTensor().defined()) return false;  // graph dropped with `graph`
      outs.push_back(v.toTensor());
    }
    plan.graph = std::move(graph);
    plan.static_in = std::move(statics);
    plan.static_out = std::move(outs);
    plan.graph_state = 1;
    g_graph_captures++;
    B200LOG(DBG) << "fusion group captured as a device graph with " << plan.graph->num_nodes() << " nodes";
    return true;
  }

  std::shared_ptr<Plan> compile(const std::string& spec, const Stack& stack, size_t n_in) {
    // specialise a copy of the subgraph: concrete input types, fused kernels
    std::shared_ptr<Graph> g = graph_->copy();
    for (size_t i = 0; i < n_in; ++i) {
      const IValue& v = stack[stack.size() - n_in + i];
      if (v.isTensor() && v.toTensor().defined()) g->inputs()[i]->setType(TensorType::create(v.toTensor()));
    }
    FuseKernels(g);
    auto plan = std::make_shared<Plan>();
    plan->code = std::make_shared<Code>(g, "b200_fusion_group");
    g_compiles++;
    std::lock_guard<std::mutex> lk(mu_);
    plans_[spec] = plan;
    return plan;
  }

  void run_fallback(Stack& stack, const Stack& saved) {
    stack.insert(stack.end(), saved.begin(), saved.end());
    InterpreterState(fallback_).run(stack);
  }

  void debug_compare(const std::string& mode, const Stack& inputs, const Stack& stack) {
    // mode "cpu": run the same subgraph on CPU copies and write both results next to each other
    if (mode != "cpu") return;
    Stack cpu_stack;
    for (const IValue& v : inputs) cpu_stack.push_back(v.isTensor() && v.toTensor().defined() ? IValue(v.toTensor().cpu()) : v);
    try {
      InterpreterState(fallback_).run(cpu_stack);
    } catch (const std::exception& e) {
      TORCH_WARN("b200 fusion debug: CPU run failed: ", e.what());
      return;
    }
    static std::atomic<int> counter{0};
    const int id = counter++;
    const size_t n_out = graph_->outputs().size();
    c10::List<at::Tensor> dev_out, cpu_out;
    for (size_t i = 0; i < n_out; ++i) {
      const IValue& d = stack[stack.size() - n_out + i];
      const IValue& c = cpu_stack[cpu_stack.size() - n_out + i];
      if (d.isTensor()) dev_out.push_back(d.toTensor().cpu());
      if (c.isTensor()) cpu_out.push_back(c.toTensor());
    }
    auto write = [&](const std::string& name, const c10::List<at::Tensor>& l) {
      auto bytes = torch::jit::pickle_save(IValue(l));
      std::ofstream f(name, std::ios::binary);
      f.write(bytes.data(), static_cast<std::streamsize>(bytes.size()));
    };
    write("fused_kernel_" + std::to_string(id) + "_device.pt", dev_out);
    write("fused_kernel_" + std::to_string(id) + "_cpu.pt", cpu_out);
  }

  std::shared_ptr<Graph> graph_;
  Code fallback_;
  std::mutex mu_;
  std::unordered_map<std::string, std::shared_ptr<Plan>> plans_;
};

class RunnerCache {
 public:
  static RunnerCache& get() {
    static RunnerCache c;
    return c;
  }
  std::shared_ptr<FusedRunner> registerFusion(const Node* node) {
    std::shared_ptr<Graph> g = node->g(attr::Subgraph)->copy();
    std::shared_ptr<Graph> canon = Canonicalize(g, /*keep_unique_names=*/false);
    std::string text = canon->toString(/*print_source_locations=*/false);
    // The printed graph shows tensor constants as <Tensor>: two modules with the same structure
    // but different weights print alike, so the key also names the constant tensors themselves.
    // A cached runner keeps its graph (and so these tensors) alive, which keeps the addresses unique.
    for (const Node* n : g->nodes()) {
      if (n->kind() != prim::Constant || !n->hasAttribute(attr::value) || n->kindOf(attr::value) != AttributeKind::t) continue;
      text += "|" + std::to_string(reinterpret_cast<uintptr_t>(n->t(attr::value).unsafeGetTensorImpl()));
    }
    std::lock_guard<std::mutex> lk(mu_);
    auto it = by_text_.find(text);
    if (it != by_text_.end()) {
      if (auto live = it->second.lock()) return live;
      by_text_.erase(it);
    }
    // The cache only observes runners: the operator closures of the graph executors own them, so the
    // device constants of a deleted module are released with its last executor.
    for (auto e = by_text_.begin(); e != by_text_.end();) e = e->second.expired() ? by_text_.erase(e) : std::next(e);
    auto runner = std::make_shared<FusedRunner>(g);
    by_text_[text] = runner;
    return runner;
  }
  int64_t size() {
    std::lock_guard<std::mutex> lk(mu_);
    int64_t n = 0;
    for (auto& e : by_text_) n += e.second.expired() ? 0 : 1;
    return n;
  }
  void clear() {
    std::lock_guard<std::mutex> lk(mu_);
    by_text_.clear();  // existing closures keep their own runners
  }

 private:
  std::mutex mu_;
  std::unordered_map<std::string, std::weak_ptr<FusedRunner>> by_text_;
};

Operation create_fusion_operation(const Node* node) {
  auto runner = RunnerCache::get().registerFusion(node);
  return [runner](Stack& stack) { runner->run(stack); };
}

RegisterOperators reg_fusion({Operator(Symbol::fromQualString("catch_b200::FusionGroup"), create_fusion_operation,
                                       AliasAnalysisKind::CONSERVATIVE)});

}  // namespace

int64_t fusion_cache_size() { return RunnerCache::get().size(); }
void fusion_cache_clear() { RunnerCache::get().clear(); }
int64_t fusion_compile_count() { return g_compiles.load(); }
int64_t fusion_fallback_count() { return g_fallbacks.load(); }
int64_t fusion_graph_capture_count() { return g_graph_captures.load(); }
int64_t fusion_graph_replay_count() { return g_graph_replays.load(); }

}  // namespace jit
}  // namespace catch_b200
