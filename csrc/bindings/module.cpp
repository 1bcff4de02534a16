#include <torch/extension.h>

#include "bind.hpp"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "mccl_b200 native extension (sm_100a)";
  mccl::bind_pg(m);
  mccl::bind_comm(m);
  mccl::bind_runtime(m);
  mccl::bind_ops(m);
}
