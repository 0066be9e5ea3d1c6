// Bindings of the auxiliary subsystems (grown as the subsystems land).
#include <torch/csrc/utils/pybind.h>
#include <torch/extension.h>

namespace py = pybind11;

namespace catch_b200 {
void bind_extras(py::module& m) { (void)m; }
}  // namespace catch_b200
