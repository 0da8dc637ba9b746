// Bindings of the MoE kernels (routing, split scan, dispatch, grouped GEMM, combine).
#include <torch/extension.h>

namespace py = pybind11;

void bind_moe(py::module_& m) { (void)m; }
