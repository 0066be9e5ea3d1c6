#include "dumper.h"

// RecordFunction::inputs() checks a flag that only a debug build of libtorch maintains (the dispatcher code that
// sets it is inlined into whoever makes the call); the shipped libtorch is a release build, so this file is compiled
// with release semantics for the torch headers even when the rest of the extension is built with assertions.
#ifndef NDEBUG
#define NDEBUG
#endif

#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/record_function.h>
#include <sys/stat.h>

#include <fstream>
#include <iomanip>
#include <iostream>
#include <map>
#include <mutex>
#include <sstream>

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

// ------------------------------------------------------------------ kernel case generator
namespace {

struct GenCaseState {
  std::mutex mu;
  int level = 0;
  std::string root;
  at::CallbackHandle handle = 0;
  std::map<std::string, int> counters;
};
GenCaseState& gc() {
  static GenCaseState s;
  return s;
}
thread_local bool tl_gc_inside = false;
thread_local int tl_gc_depth = 0;

std::string json_escape(const std::string& in) {
  std::string out;
  for (char ch : in) {
    if (ch == '"' || ch == '\\') { out += '\\'; out += ch; }
    else if (ch == '\n') out += "\\n";
    else if ((unsigned char)ch < 0x20) out += ' ';
    else out += ch;
  }
  return out;
}

template <typename L>
std::string json_ints(const L& v) {
  std::ostringstream o;
  o << "[";
  bool first = true;
  for (auto x : v) { o << (first ? "" : ", ") << (int64_t)x; first = false; }
  o << "]";
  return o.str();
}

const char* memory_format_of(const at::Tensor& t) {
  if (t.is_contiguous()) return "contiguous";
  if (t.dim() == 4 && t.is_contiguous(at::MemoryFormat::ChannelsLast)) return "channels_last";
  if (t.dim() == 5 && t.is_contiguous(at::MemoryFormat::ChannelsLast3d)) return "channels_last_3d";
  return "strided";
}

// `data_file`: where level 2 puts the bytes of a device tensor ("" = do not write)
std::string describe_tensor(const at::Tensor& t, const std::string& data_file) {
  if (!t.defined()) return "{\"kind\": \"none\"}";
  std::ostringstream o;
  o << "{\"kind\": \"tensor\", \"dtype\": \"" << c10::toString(t.scalar_type()) << "\", \"shape\": " << json_ints(t.sizes())
    << ", \"stride\": " << json_ints(t.strides()) << ", \"format\": \"" << memory_format_of(t) << "\", \"device\": \""
    << (is_b200(t) ? "device" : "cpu") << "\", \"requires_grad\": " << (t.requires_grad() ? "true" : "false");
  if (!data_file.empty() && t.numel() > 0 && !t.is_complex()) {
    at::Tensor c = t.detach().cpu().contiguous();
    std::ofstream f(data_file, std::ios::binary);
    f.write(static_cast<const char*>(c.data_ptr()), (std::streamsize)c.nbytes());
    const size_t slash = data_file.find_last_of('/');
    o << ", \"data\": \"" << json_escape(slash == std::string::npos ? data_file : data_file.substr(slash + 1)) << "\"";
  }
  o << "}";
  return o.str();
}

std::string describe_value(const c10::IValue& v, const std::string& data_prefix) {
  std::ostringstream o;
  if (v.isTensor()) return describe_tensor(v.toTensor(), data_prefix.empty() ? "" : data_prefix + ".bin");
  if (v.isNone()) return "{\"kind\": \"none\"}";
  if (v.isBool()) { o << "{\"kind\": \"bool\", \"value\": " << (v.toBool() ? "true" : "false") << "}"; return o.str(); }
  if (v.isInt()) { o << "{\"kind\": \"int\", \"value\": " << v.toInt() << "}"; return o.str(); }
  if (v.isDouble()) {
    o << std::setprecision(17) << "{\"kind\": \"float\", \"value\": \"" << v.toDouble() << "\"}";  // a string: inf / nan are not JSON
    return o.str();
  }
  if (v.isString()) { o << "{\"kind\": \"string\", \"value\": \"" << json_escape(v.toStringRef()) << "\"}"; return o.str(); }
  if (v.isDevice()) {
    o << "{\"kind\": \"device\", \"value\": \"" << (v.toDevice().type() == c10::DeviceType::PrivateUse1 ? "device" : "cpu") << "\"}";
    return o.str();
  }
  if (v.isIntList()) { o << "{\"kind\": \"int_list\", \"value\": " << json_ints(v.toIntVector()) << "}"; return o.str(); }
  if (v.isBoolList()) {
    std::vector<int64_t> b;
    for (bool x : v.toBoolList()) b.push_back(x ? 1 : 0);
    o << "{\"kind\": \"bool_list\", \"value\": " << json_ints(b) << "}";
    return o.str();
  }
  if (v.isDoubleList()) {
    o << std::setprecision(17) << "{\"kind\": \"float_list\", \"value\": [";
    bool first = true;
    for (double x : v.toDoubleVector()) { o << (first ? "\"" : ", \"") << x << "\""; first = false; }
    o << "]}";
    return o.str();
  }
  if (v.isTensorList()) {
    o << "{\"kind\": \"tensor_list\", \"value\": [";
    int k = 0;
    for (const at::Tensor& t : v.toTensorList()) {
      o << (k ? ", " : "") << describe_tensor(t, data_prefix.empty() ? "" : data_prefix + "_" + std::to_string(k) + ".bin");
      ++k;
    }
    o << "]}";
    return o.str();
  }
  if (v.isList()) {  // e.g. optional tensor lists (indices of aten::index)
    o << "{\"kind\": \"list\", \"value\": [";
    int k = 0;
    for (const c10::IValue& e : v.toListRef()) {
      o << (k ? ", " : "") << describe_value(e, data_prefix.empty() ? "" : data_prefix + "_" + std::to_string(k));
      ++k;
    }
    o << "]}";
    return o.str();
  }
  o << "{\"kind\": \"other\", \"tag\": \"" << json_escape(v.tagKind()) << "\"}";
  return o.str();
}

std::unique_ptr<at::ObserverContext> gc_enter(const at::RecordFunction& fn) {
  ++tl_gc_depth;
  if (tl_gc_inside || tl_inside) return nullptr;
  GenCaseState& s = gc();
  const int level = s.level;
  if (level == 0 || !fn.operator_name().has_value()) return nullptr;
  tl_gc_inside = true;
  try {
    auto inputs = fn.inputs();
    auto op = c10::Dispatcher::singleton().findSchema(*fn.operator_name());
    if (touches_device(inputs) && op.has_value() && inputs.size() == op->schema().arguments().size()) {
      const auto& schema = op->schema();
      std::string name = schema.name() + (schema.overload_name().empty() ? "" : "." + schema.overload_name());
      std::string flat = name;
      for (auto& ch : flat) if (ch == ':' || ch == '/') ch = '_';
      std::string case_path;
      if (level != 3) {
        int n;
        {
          std::lock_guard<std::mutex> g(s.mu);
          n = s.counters[flat]++;
        }
        mkdirs(s.root);
        mkdirs(s.root + "/" + flat);
        case_path = s.root + "/" + flat + "/" + flat + "_" + std::to_string(n);
      }
      std::ostringstream o;
      o << "{\"op\": \"" << json_escape(name) << "\", \"schema\": \"" << json_escape(c10::toString(schema)) << "\", \"depth\": "
        << (tl_gc_depth - 1) << ", \"args\": [";
      size_t i = 0;
      for (const auto& v : inputs) {
        const auto& a = schema.arguments()[i];
        std::string d = describe_value(v, level == 2 ? case_path + ".arg" + std::to_string(i) : "");
        // {"name": ..., "type": ..., <description fields>}
        o << (i ? ",\n  " : "\n  ") << "{\"name\": \"" << json_escape(a.name()) << "\", \"type\": \"" << json_escape(a.type()->str())
          << "\", " << d.substr(1);
        ++i;
      }
      o << "\n]}\n";
      if (level == 3) {
        std::cerr << "[gen_case] " << o.str();
      } else {
        std::ofstream f(case_path + ".json");
        f << o.str();
      }
    }
  } catch (const std::exception& e) {
    B200LOG(DBG) << "case generator: " << fn.name() << ": " << e.what();
  }
  tl_gc_inside = false;
  return nullptr;
}

void gc_exit(const at::RecordFunction&, at::ObserverContext*) { --tl_gc_depth; }

}  // namespace

void gencase_set(int level, const std::string& dir) {
  GenCaseState& s = gc();
  std::lock_guard<std::mutex> g(s.mu);
  if (s.level != 0) {
    at::removeCallback(s.handle);
    s.level = 0;
  }
  if (level <= 0) return;
  s.root = dir;
  s.level = level > 3 ? 3 : level;
  tl_gc_depth = 0;
  s.handle = at::addGlobalCallback(at::RecordFunctionCallback(&gc_enter, &gc_exit).needsInputs(true).scopes({at::RecordScope::FUNCTION}));
}

int gencase_level() { return gc().level; }

}  // namespace catch_b200
