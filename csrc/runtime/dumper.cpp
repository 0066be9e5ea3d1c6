#include "dumper.h"

#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/record_function.h>
#include <sys/stat.h>

#include <fstream>
#include <iomanip>
#include <mutex>

#include "log.h"
#include "tensor_impl.h"

namespace catch_b200 {
namespace {

struct DumpState {
  std::mutex mu;
  bool running = false;
  bool use_cpu = false;
  int level = 0;
  std::string root;
  at::CallbackHandle handle = 0;
};
DumpState& st() {
  static DumpState s;
  return s;
}

struct Frame {
  std::string dir;
  int children = 0;
  bool active = false;
};
thread_local std::vector<Frame> tl_stack;
thread_local bool tl_inside = false;  // re-entrancy guard while the tool itself runs ops

void mkdirs(const std::string& p) { ::mkdir(p.c_str(), 0777); }

void write_tensor(const std::string& path, const at::Tensor& t, int level) {
  at::Tensor c = t.detach().cpu();
  std::ofstream f(path);
  const int64_t n = c.numel();
  int64_t dumped = level == 0 ? std::min<int64_t>(n, 10) : (level == 1 ? 1 : n);
  f << "Tensor : Type = " << c10::toString(t.scalar_type()) << " : Shape = " << t.sizes() << " : Stride = " << t.strides()
    << " : Dumped = " << dumped << "\n";
  if (n == 0) return;
  at::Tensor flat = c.contiguous().view({-1});
  if (flat.is_complex()) return;
  at::Tensor d = flat.scalar_type() == at::kBool ? flat.to(at::kDouble) : flat.to(at::kDouble);
  f << std::setprecision(8);
  if (level == 1) {
    f << d.abs().sum().item<double>() << "\n";
    return;
  }
  const double* p = d.data_ptr<double>();
  for (int64_t i = 0; i < dumped; ++i) f << p[i] << "\n";
}

bool touches_device(const c10::ArrayRef<const c10::IValue>& vals) {
  for (const auto& v : vals) {
    if (v.isTensor() && is_b200(v.toTensor())) return true;
    if (v.isTensorList())
      for (const at::Tensor& t : v.toTensorList())
        if (is_b200(t)) return true;
  }
  return false;
}

c10::IValue to_cpu(const c10::IValue& v) {
  if (v.isTensor()) {
    const at::Tensor& t = v.toTensor();
    return t.defined() ? c10::IValue(t.detach().cpu()) : v;
  }
  if (v.isTensorList()) {
    c10::List<at::Tensor> out;
    for (const at::Tensor& t : v.toTensorList()) out.push_back(t.defined() ? t.detach().cpu() : t);
    return out;
  }
  if (v.isDevice() && v.toDevice().type() == c10::DeviceType::PrivateUse1) return c10::IValue(c10::Device(c10::kCPU));
  return v;
}

std::unique_ptr<at::ObserverContext> on_enter(const at::RecordFunction& fn) {
  if (tl_inside) return nullptr;
  DumpState& s = st();
  if (!s.running) return nullptr;
  tl_inside = true;
  Frame fr;
  try {
    auto inputs = fn.inputs();
    fr.active = touches_device(inputs);
    if (fr.active) {
      std::string parent = tl_stack.empty() || !tl_stack.back().active ? s.root : tl_stack.back().dir;
      int idx;
      if (tl_stack.empty() || !tl_stack.back().active) {
        static int top_counter = 0;
        std::lock_guard<std::mutex> g(s.mu);
        idx = top_counter++;
      } else {
        idx = tl_stack.back().children++;
      }
      std::string name = fn.name();
      for (auto& ch : name) if (ch == ':' || ch == '/') ch = '_';
      fr.dir = parent + "/" + std::to_string(idx) + "_" + name;
      mkdirs(fr.dir);
      int i = 0;
      for (const auto& v : inputs) {
        if (v.isTensor() && v.toTensor().defined() && is_b200(v.toTensor()))
          write_tensor(fr.dir + "/dev_" + std::to_string(i), v.toTensor(), s.level);
        ++i;
      }
      if (s.use_cpu && fn.operator_name().has_value()) {
        // run the same operator on CPU copies of the arguments, before a possibly in-place op changes them
        try {
          auto opname = *fn.operator_name();
          auto op = c10::Dispatcher::singleton().findSchema(opname);
          if (op.has_value() && inputs.size() == op->schema().arguments().size()) {
            torch::jit::Stack stack;
            for (const auto& v : inputs) stack.push_back(to_cpu(v));
            op->callBoxed(&stack);
            int k = 0;
            for (const auto& v : stack) {
              if (v.isTensor() && v.toTensor().defined())
                write_tensor(fr.dir + "/cpu_result_" + std::to_string(k), v.toTensor(), s.level);
              ++k;
            }
          }
        } catch (const std::exception& e) {
          B200LOG(DBG) << "dump tool: CPU recompute of " << fn.name() << " failed: " << e.what();
        }
      }
    }
  } catch (...) {
    fr.active = false;
  }
  tl_stack.push_back(fr);
  tl_inside = false;
  return nullptr;
}

void on_exit(const at::RecordFunction& fn, at::ObserverContext*) {
  if (tl_inside || tl_stack.empty()) return;
  DumpState& s = st();
  Frame fr = tl_stack.back();
  tl_stack.pop_back();
  if (!fr.active || !s.running) return;
  tl_inside = true;
  try {
    int k = 0;
    for (const auto& v : fn.outputs()) {
      if (v.isTensor() && v.toTensor().defined() && is_b200(v.toTensor()))
        write_tensor(fr.dir + "/dev_result_" + std::to_string(k), v.toTensor(), s.level);
      ++k;
    }
  } catch (...) {
  }
  tl_inside = false;
}

}  // namespace

void dump_start(const std::string& dir, bool enable, bool use_cpu, int level) {
  DumpState& s = st();
  dump_finish();
  if (!enable) return;
  std::lock_guard<std::mutex> g(s.mu);
  // "<dir>", "<dir>1", "<dir>2", ... : never overwrite an earlier dump
  std::string root = dir;
  struct stat sb;
  for (int i = 1; ::stat(root.c_str(), &sb) == 0; ++i) root = dir + std::to_string(i);
  mkdirs(root);
  s.root = root;
  s.use_cpu = use_cpu;
  s.level = level;
  s.running = true;
  s.handle = at::addGlobalCallback(at::RecordFunctionCallback(&on_enter, &on_exit)
                                       .needsInputs(true)
                                       .needsOutputs(true)
                                       .scopes({at::RecordScope::FUNCTION}));
}

void dump_finish() {
  DumpState& s = st();
  std::lock_guard<std::mutex> g(s.mu);
  if (!s.running) return;
  at::removeCallback(s.handle);
  s.running = false;
}

bool dump_running() { return st().running; }

}  // namespace catch_b200
