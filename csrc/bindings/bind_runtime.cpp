#include <torch/extension.h>

#include "bind.hpp"

namespace mccl {
void bind_runtime(pybind11::module_& m) { (void)m; }
}  // namespace mccl
