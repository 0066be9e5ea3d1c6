// Bindings of the dump tool, JIT fusion toggles and profiler helpers.
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include <torch/csrc/jit/python/pybind_utils.h>

#include "../device/kernels_api.h"
#include "../jit/fusion.h"
#include "../runtime/dumper.h"
#include "../runtime/profiler.h"

namespace py = pybind11;

namespace catch_b200 {
void bind_aux(py::module& m) {
  m.def("_dump_start", &dump_start, py::arg("dir"), py::arg("enable") = true, py::arg("use_cpu") = false, py::arg("level") = 0);
  m.def("_dump_finish", &dump_finish);
  m.def("_dump_running", &dump_running);
  m.def("_dump_gencase", &gencase_set, py::arg("level"), py::arg("dir") = "./gen_case");
  m.def("_gencase_level", &gencase_level);
  // kernel selection knob for benchmarks and tests: see b200_conv_wgrad_halo_mode
  m.def("_conv_wgrad_halo_mode", [](int mode) { return b200_conv_wgrad_halo_mode(mode); }, py::arg("mode") = -1);
  m.def("_jit_can_fuse_on_b200", &jit::fusion_enabled);
  m.def("_jit_override_can_fuse_on_b200", &jit::set_fusion_enabled);
  m.def("_jit_register_passes", &jit::register_passes);
  m.def("_jit_fusion_cache_size", &jit::fusion_cache_size);
  m.def("_jit_fusion_cache_clear", &jit::fusion_cache_clear);
  m.def("_jit_fusion_graph_capture_count", &jit::fusion_graph_capture_count);
  m.def("_jit_fusion_graph_replay_count", &jit::fusion_graph_replay_count);
  m.def("_jit_fusion_compile_count", &jit::fusion_compile_count);
  m.def("_jit_fusion_fallback_count", &jit::fusion_fallback_count);
  m.def("_jit_pass_lower_graph", [](std::shared_ptr<torch::jit::Graph>& g) { jit::LowerGraph(g); });
  m.def("_jit_pass_fuse_kernels", [](std::shared_ptr<torch::jit::Graph>& g) { jit::FuseKernels(g); });
  m.def("_jit_pass_unfuse_graph", [](std::shared_ptr<torch::jit::Graph>& g) { jit::UnfuseGraph(g); });
  m.def("_kernel_trace_start", &kernel_trace_start);
  m.def("_kernel_trace_stop", [] {
    std::vector<KernelEvent> evs;
    {
      py::gil_scoped_release nogil;
      evs = kernel_trace_stop();
    }
    py::list out;
    for (auto& e : evs) out.append(py::make_tuple(e.name, e.op, e.kind, e.device, e.queue, e.cpu_ns, e.start_us, e.dur_us));
    return out;
  });
  m.def("_trace_mark", [](const std::string& s) { trace_mark(s.c_str()); });
  m.def("_trace_range_push", [](const std::string& s) { trace_range_push(s.c_str()); });
  m.def("_trace_range_pop", &trace_range_pop);
  m.def("_jit_pass_segment_graph", [](std::shared_ptr<torch::jit::Graph>& g) { jit::SegmentGraph(g); });
}
}  // namespace catch_b200
