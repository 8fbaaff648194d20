// Bindings of the kernels that live outside the core translation unit
// (attention, softmax, dropout, MoE router / permutation, NVFP4, fused
// communication).  Kept separate so that touching one family does not rebuild
// the rest.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <teb200/api.h>
#include <teb200/misc.h>
#include <teb200/quant.h>
#include <torch/extension.h>

#include <optional>

namespace py = pybind11;
using OptT = std::optional<at::Tensor>;

void register_extra(py::module_& m) { (void)m; }
