// Bindings of dump tool / profiler / JIT toggles (filled in as those subsystems land).
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

namespace py = pybind11;

namespace catch_b200 {
void bind_aux(py::module& m) { (void)m; }
}  // namespace catch_b200
