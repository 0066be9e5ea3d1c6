// Bindings of the distributed backend and the auxiliary subsystems.
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <pybind11/chrono.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

#include "../distributed/process_group.h"
#include "../ops/kernels.h"

namespace py = pybind11;

namespace catch_b200 {

void bind_aux(py::module& m);  // dumper / profiler / jit (aux.cpp)

void bind_extras(py::module& m) {
  py::module::import("torch.distributed");
  py::class_<ProcessGroupB200, c10d::Backend, c10::intrusive_ptr<ProcessGroupB200>>(m, "ProcessGroupB200")
      .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout) {
             return c10::make_intrusive<ProcessGroupB200>(store, rank, size, timeout);
           }),
           py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout") = std::chrono::milliseconds(600000))
      .def("symm_empty", &ProcessGroupB200::symm_empty)
      .def("shard_elems", &ProcessGroupB200::shard_elems)
      .def("allreduce_symm", &ProcessGroupB200::allreduce_symm, py::arg("tensor"), py::arg("op") = 0, py::arg("scale") = 1.0,
           py::arg("test_no_signal") = false, py::call_guard<py::gil_scoped_release>())
      .def("fused_allreduce_step", &ProcessGroupB200::fused_allreduce_step, py::arg("grads"), py::arg("params"),
           py::arg("state1"), py::arg("state2"), py::arg("kind"), py::arg("lr"), py::arg("momentum"), py::arg("dampening"),
           py::arg("weight_decay"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("step"), py::arg("nesterov"),
           py::arg("first_step"), py::arg("scale"), py::arg("lowp") = std::nullopt, py::arg("cast_src") = std::nullopt,
           py::arg("zero_grads") = false, py::call_guard<py::gil_scoped_release>())
      .def("set_wait_limit_ms", &ProcessGroupB200::set_wait_limit_ms)
      .def("status_word", &ProcessGroupB200::status_word)
      .def("dead_peer", &ProcessGroupB200::dead_peer)
      .def("clear_status", &ProcessGroupB200::clear_status)
      .def("device_index", &ProcessGroupB200::device_index)
      .def("multicast_enabled", &ProcessGroupB200::multicast_enabled, py::call_guard<py::gil_scoped_release>());
  m.def("_stop_all_watchdogs", [] { stop_all_watchdogs(); }, py::call_guard<py::gil_scoped_release>());
  m.def("_kernel_launch_count", [] { return ops::kernel_launch_count(); });
  m.def("_reset_kernel_launch_count", [] { ops::reset_kernel_launch_count(); });
  bind_aux(m);
}

}  // namespace catch_b200
