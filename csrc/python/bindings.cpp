// Python-visible native surface (module catch_b200._C).
//
// Parity: torch_mlu/csrc/interface/python_variable_methods.cpp:55-204 -- device
// functions, device properties, queue and notifier classes, memory statistics,
// pinning, seeds, version, dump-tool and fusion toggles -- with the GIL
// released around every call that can block on the device.
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "../runtime/caching_allocator.h"
#include "../runtime/device.h"
#include "../runtime/generator.h"
#include "../runtime/graph.h"
#include "../runtime/host_allocator.h"
#include "../runtime/log.h"
#include "../runtime/notifier.h"
#include "../runtime/queue.h"

namespace py = pybind11;
using namespace catch_b200;

namespace catch_b200 {
namespace ops {
at::Tensor pin_memory(const at::Tensor& t);
bool tensor_is_pinned(const at::Tensor& t);
}  // namespace ops
void bind_extras(py::module& m);  // dumper / jit / distributed / profiler bindings (extras.cpp)
}  // namespace catch_b200

namespace {
struct PyNotifier {
  explicit PyNotifier(bool timing) : n(std::make_shared<Notifier>(timing)) {}
  std::shared_ptr<Notifier> n;
};
}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "Native runtime of the b200 PyTorch device backend";

  // ---- device
  m.def("_backend_name", [] { return std::string(backend().name()); });
  m.def("_is_hostsim", [] { return hostsim(); });
  m.def("_device_count", [] { return device_count(); });
  m.def("_set_device", [](int d) { set_device(d); });
  m.def("_current_device", [] { return current_device(); });
  m.def("_synchronize", [](int d) {
    py::gil_scoped_release nogil;
    synchronize(d);
  }, py::arg("device") = -1);
  py::class_<DeviceProp>(m, "_B200DeviceProperties")
      .def_readonly("name", &DeviceProp::name)
      .def_readonly("major", &DeviceProp::major)
      .def_readonly("minor", &DeviceProp::minor)
      .def_readonly("total_memory", &DeviceProp::total_memory)
      .def_readonly("multi_processor_count", &DeviceProp::multi_processor_count)
      .def_readonly("max_shared_memory_per_block_optin", &DeviceProp::max_shared_memory_per_block_optin)
      .def_readonly("l2_cache_size", &DeviceProp::l2_cache_size)
      .def("__repr__", [](const DeviceProp& p) {
        std::ostringstream os;
        os << "_B200DeviceProperties(name='" << p.name << "', major=" << p.major << ", minor=" << p.minor
           << ", total_memory=" << p.total_memory / (1024 * 1024) << "MB, multi_processor_count="
           << p.multi_processor_count << ")";
        return os.str();
      });
  m.def("_get_device_properties", [](int d) { return device_properties(d); });
  m.def("_get_version", [] { return version_string(); });
  m.def("_hostsim_set_memory_limit", [](size_t b) { hostsim_set_memory_limit(b); });

  // ---- queues
  py::class_<Queue>(m, "_Queue")
      .def_property_readonly("device_index", &Queue::device_index)
      .def_property_readonly("id", &Queue::id)
      .def_property_readonly("handle", [](const Queue& q) { return reinterpret_cast<uintptr_t>(q.handle()); })
      .def("query", &Queue::query)
      .def("synchronize", [](const Queue& q) {
        py::gil_scoped_release nogil;
        q.synchronize();
      })
      .def("__eq__", [](const Queue& a, const Queue& b) { return a == b; })
      .def("__hash__", [](const Queue& q) { return std::hash<Queue>()(q); })
      .def("__repr__", [](const Queue& q) {
        std::ostringstream os;
        os << "<b200 Queue device=" << q.device_index() << " id=" << q.id() << ">";
        return os.str();
      });
  m.def("_getQueueFromPool", [](int d) { return getQueueFromPool(d); }, py::arg("device") = -1);
  m.def("_getDefaultQueue", [](int d) { return getDefaultQueue(d); }, py::arg("device") = -1);
  m.def("_getCurrentQueue", [](int d) { return getCurrentQueue(d); }, py::arg("device") = -1);
  m.def("_getQueueById", [](int d, int id) { return getQueueById(d, id); });
  m.def("_setCurrentQueue", [](const Queue& q) { setCurrentQueue(q); });

  // ---- executable graphs
  py::class_<DeviceGraph>(m, "_Graph")
      .def(py::init<>())
      .def("capture_begin", &DeviceGraph::capture_begin)
      .def("capture_end", &DeviceGraph::capture_end)
      .def("capture_abort", &DeviceGraph::capture_abort)
      .def("replay", &DeviceGraph::replay)
      .def("reset", [](DeviceGraph& g) {
        py::gil_scoped_release nogil;
        g.reset();
      })
      .def_property_readonly("valid", &DeviceGraph::valid)
      .def_property_readonly("num_nodes", &DeviceGraph::num_nodes);
  // allocator pools behind graph capture (exposed for tests of the pool bookkeeping without a device)
  m.def("_new_private_pool", [] { return newPrivatePool(); });
  m.def("_set_thread_private_pool", [](uint64_t p) { return setThreadPrivatePool(p); });
  m.def("_retire_private_pool", [](uint64_t p) { retirePrivatePool(p); });
  m.def("_graphs_supported", [] { return backend().supports_graphs(); });
  m.def("_graph_capture_active", [] { return graphCaptureActive(); });

  // ---- notifiers
  py::class_<PyNotifier>(m, "_Notifier")
      .def(py::init<bool>(), py::arg("enable_timing") = true)
      .def("place", [](PyNotifier& s) { s.n->place(); })
      .def("place", [](PyNotifier& s, const Queue& q) { s.n->place(q); })
      .def("wait", [](PyNotifier& s, const Queue& q) { s.n->wait(q); })
      .def("query", [](PyNotifier& s) { return s.n->query(); })
      .def("synchronize", [](PyNotifier& s) {
        py::gil_scoped_release nogil;
        s.n->synchronize();
      })
      .def("elapsed_time", [](PyNotifier& s, PyNotifier& e) {
        py::gil_scoped_release nogil;
        return s.n->elapsed_time(*e.n);
      })
      .def("hardware_time", [](PyNotifier& s, PyNotifier& e) {
        py::gil_scoped_release nogil;
        return s.n->hardware_time(*e.n);
      });

  // ---- memory
  m.def("_memory_allocated", [](int d) { return memoryStats(d).allocated; });
  m.def("_max_memory_allocated", [](int d) { return memoryStats(d).max_allocated; });
  m.def("_memory_reserved", [](int d) { return memoryStats(d).reserved; });
  m.def("_max_memory_reserved", [](int d) { return memoryStats(d).max_reserved; });
  m.def("_memory_stats", [](int d) {
    MemoryStats s = memoryStats(d);
    py::dict r;
    r["allocated_bytes.current"] = s.allocated;
    r["allocated_bytes.peak"] = s.max_allocated;
    r["reserved_bytes.current"] = s.reserved;
    r["reserved_bytes.peak"] = s.max_reserved;
    r["num_alloc"] = s.num_alloc;
    r["num_free"] = s.num_free;
    r["segments"] = s.num_segments;
    r["num_ooms"] = s.num_ooms;
    r["num_alloc_retries"] = s.num_retries;
    return r;
  });
  m.def("_memory_summary", [](int d) { return memorySummary(d); });
  m.def("_reset_peak_memory_stats", [](int d) { resetPeakStats(d); });
  m.def("_empty_cache", [] {
    py::gil_scoped_release nogil;
    emptyCache();
  });
  m.def("_set_memory_strategy", [](bool native) { setNativeMemoryStrategy(native); });
  m.def("_get_memory_strategy", [] { return nativeMemoryStrategy(); });
  m.def("_set_memory_fraction", [](double fraction, int d) { setMemoryFraction(fraction, d); });
  m.def("_memory_reserve_limit", [](int d) { return memoryReserveLimit(d); });
  // raw blocks from the caching allocator (torch.cuda.caching_allocator_alloc / _delete)
  m.def("_raw_alloc", [](size_t bytes, int d, const Queue* q) {
    return reinterpret_cast<uintptr_t>(raw_alloc(bytes, d, q ? *q : getCurrentQueue(d)));
  }, py::arg("bytes"), py::arg("device"), py::arg("queue") = nullptr);
  m.def("_raw_free", [](uintptr_t ptr) { raw_free(reinterpret_cast<void*>(ptr)); });
  // Python frames of the allocating thread for the debug allocator's origin records.
  setAllocationContextHook(+[]() -> std::string {
    if (!Py_IsInitialized() || _Py_IsFinalizing()) return std::string();
    py::gil_scoped_acquire gil;  // most allocations come from bindings that released the interpreter lock
    std::string out;
    PyFrameObject* f = PyEval_GetFrame();  // borrowed
    Py_XINCREF(f);
    for (int depth = 0; f && depth < 12; ++depth) {
      PyCodeObject* code = PyFrame_GetCode(f);
      const char* file = PyUnicode_AsUTF8(code->co_filename);
      const char* name = PyUnicode_AsUTF8(code->co_name);
      out += "    " + std::string(file ? file : "?") + ":" + std::to_string(PyFrame_GetLineNumber(f)) + " in " +
             std::string(name ? name : "?") + "\n";
      Py_DECREF(code);
      PyFrameObject* back = PyFrame_GetBack(f);
      Py_DECREF(f);
      f = back;
    }
    Py_XDECREF(f);
    if (PyErr_Occurred()) PyErr_Clear();
    return out;
  });
  m.def("_memory_debug_origin", [](const at::Tensor& t) { return memoryDebugOrigin(t.storage().data()); });
  m.def("_set_memory_debug", [](bool on) { setMemoryDebug(on); });
  m.def("_memory_debug_enabled", [] { return memoryDebugEnabled(); });
  m.def("_memory_debug", [](std::optional<at::Tensor> t) {
    DebugReport r = memoryDebugCheck(t.has_value() && t->defined() ? t->storage().data() : nullptr);
    return py::make_tuple(r.blocks_checked, r.corrupted, r.detail);
  }, py::arg("tensor") = py::none());
  m.def("_record_queue", [](const at::Tensor& t, const Queue& q) { recordQueue(t.storage().data_ptr(), q); });
  m.def("_pin_memory", [](const at::Tensor& t) { return ops::pin_memory(t); });
  m.def("_is_pinned", [](const at::Tensor& t) { return ops::tensor_is_pinned(t); });
  m.def("_pinned_empty_cache", [] { pinnedEmptyCache(); });
  m.def("_pinned_cached_bytes", [] { return pinnedCachedBytes(); });
  m.def("_notifier_pool_clean", [] { NotifierPool::instance().clean(); });

  // ---- RNG
  m.def("_manual_seed", [](int d, uint64_t s) { manual_seed(d, s); });
  m.def("_manual_seed_all", [](uint64_t s) { manual_seed_all(s); });
  m.def("_default_generator", [](int d) { return getDefaultB200Generator(static_cast<c10::DeviceIndex>(d)); });

  // ---- logging / flags
  m.def("_set_min_log_level", [](int l) { set_min_log_level(l); });
  m.def("_get_min_log_level", [] { return min_log_level(); });
  m.def("_log", [](int lvl, const std::string& msg) {
    if (lvl < min_log_level()) return;
    LogMessage("python", 0, "log", static_cast<LogLevel>(lvl)).stream() << msg;
  });
  m.def("_reload_flags", [] { reload_flags(); });
  m.def("_set_flag", [](const std::string& k, bool v) {
    Flags& f = flags();
    if (k == "async_disable") f.async_disable = v;
    else if (k == "op_trycatch") f.op_trycatch = v;
    else if (k == "test_cpu_dispatch") f.test_cpu_dispatch = v;
    else if (k == "fallback_to_cpu") f.fallback_to_cpu = v;
    else if (k == "blocking_wait") f.blocking_wait = v;
    else TORCH_CHECK(false, "unknown flag ", k);
  });
  m.def("_get_flag", [](const std::string& k) {
    Flags& f = flags();
    if (k == "async_disable") return f.async_disable;
    if (k == "op_trycatch") return f.op_trycatch;
    if (k == "test_cpu_dispatch") return f.test_cpu_dispatch;
    if (k == "fallback_to_cpu") return f.fallback_to_cpu;
    if (k == "blocking_wait") return f.blocking_wait;
    if (k == "memory_debug") return f.memory_debug;
    TORCH_CHECK(false, "unknown flag ", k);
  });

  bind_extras(m);
}
