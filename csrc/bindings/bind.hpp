// Registration hooks of the extension module; one per subsystem so that each
// translation unit only pulls in the headers it needs.
#pragma once

#include <pybind11/pybind11.h>

namespace mccl {
void bind_pg(pybind11::module_& m);       // process group, metrics, logging
void bind_comm(pybind11::module_& m);     // device communicator, symmetric heap, kernels
void bind_runtime(pybind11::module_& m);  // dmem, coherence, scheduler, cluster manager, agent
void bind_ops(pybind11::module_& m);      // model operators (GEMM, norms, optimizer)
}  // namespace mccl
