#include <torch/extension.h>

#include "bind.hpp"

namespace mccl {
void bind_ops(pybind11::module_& m) { (void)m; }
}  // namespace mccl
