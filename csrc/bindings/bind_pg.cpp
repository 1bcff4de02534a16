// Python bindings of the process group, metrics and logging.
//
// Parity: the reference's extension exports a single function,
// _create_process_group_mccl(store, rank, size, timeout)
// (csrc/backend/Registration.cpp:22-39); its tests and examples also expect
// __version__, __protocol_version__ and a metrics accessor on the module
// (tests/test_build.py:43-46, examples/ddp_dummy_train.py:214-222).
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/extension.h>
#include <pybind11/chrono.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>

#include "../core/log.hpp"
#include "../core/version.hpp"
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>

#include "../engine/metrics.hpp"
#include "../pg/device_comm.hpp"
#include "../pg/process_group.hpp"
#include "bind.hpp"

namespace py = pybind11;

namespace mccl {

void bind_pg(py::module_& m) {
  m.attr("__version__") = MCCL_VERSION_STRING;
  m.attr("__protocol_version__") = MCCL_PROTOCOL_VERSION;

  py::register_exception<MCCLError>(m, "MCCLError", PyExc_RuntimeError);
  auto base = m.attr("MCCLError");
  py::register_exception<TransportError>(m, "TransportError", base.ptr());
  py::register_exception<CudaError>(m, "CudaError", base.ptr());
  py::register_exception<TensorError>(m, "TensorError", base.ptr());
  py::register_exception<TimeoutError>(m, "TimeoutError", base.ptr());
  py::register_exception<ProtocolError>(m, "ProtocolError", base.ptr());

  py::class_<ProcessGroupMCCL, c10d::Backend, c10::intrusive_ptr<ProcessGroupMCCL>>(m, "ProcessGroupMCCL")
      .def("last_algo", &ProcessGroupMCCL::lastAlgo)
      .def("check_device_status", &ProcessGroupMCCL::checkDeviceStatus)
      .def(
          "allreduce_with",
          [](ProcessGroupMCCL& pg, at::Tensor t, const std::string& op, const std::string& wire, const std::string& algo) {
            auto parse_op = [](const std::string& s) {
              if (s == "sum") return RedOp::SUM;
              if (s == "avg" || s == "mean") return RedOp::AVG;
              if (s == "min") return RedOp::MIN;
              if (s == "max") return RedOp::MAX;
              if (s == "product" || s == "prod") return RedOp::PRODUCT;
              MCCL_CHECK(false, "allreduce_with: unknown reduce op '" << s << "'");
              return RedOp::SUM;
            };
            auto parse_algo = [](const std::string& s) {
              if (s.empty() || s == "auto") return Algo::AUTO;
              if (s == "ring") return Algo::RING;
              if (s == "tree") return Algo::TREE;
              if (s == "butterfly" || s == "twoshot") return Algo::BUTTERFLY;
              if (s == "oneshot") return Algo::ONESHOT;
              if (s == "nvls") return Algo::NVLS;
              if (s == "twoshot_push" || s == "butterfly_push") return Algo::BUTTERFLY_PUSH;
              MCCL_CHECK(false, "allreduce_with: unknown algorithm '" << s << "'");
              return Algo::AUTO;
            };
            std::vector<at::Tensor> ts{t};
            return pg.allreduceWith(ts, parse_op(op), parse_algo(algo), wire == "bf16" ? WireDtype::BF16 : WireDtype::NATIVE);
          },
          py::arg("tensor"), py::arg("op") = "sum", py::arg("wire") = "native", py::arg("algo") = "auto",
          py::call_guard<py::gil_scoped_release>(),
          "In-place allreduce with the wire dtype and algorithm as arguments (the environment is not consulted).")
      .def(
          "set_p2p_factory",
          [](ProcessGroupMCCL& pg, py::function factory) {
            // The group may be destroyed on a thread without the GIL (or while
            // the interpreter shuts down), so the callable is never decref'd.
            auto holder = std::shared_ptr<py::function>(new py::function(std::move(factory)), [](py::function* f) {
              f->release();
              delete f;
            });
            pg.setP2PFactory([holder]() -> c10::intrusive_ptr<c10d::Backend> {
              py::gil_scoped_acquire gil;
              py::object obj = (*holder)();
              return obj.cast<c10::intrusive_ptr<c10d::Backend>>();
            });
          },
          py::arg("factory"))
      .def(
          "device_comm",
          [](ProcessGroupMCCL& pg, int64_t device_index) {
            return pg.deviceComm(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device_index)));
          },
          py::arg("device_index"), py::call_guard<py::gil_scoped_release>());

  m.def(
      "_create_process_group_mccl",
      [](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout, int64_t arena_mb) {
        auto pg = c10::make_intrusive<ProcessGroupMCCL>(store, rank, size, timeout);
        if (arena_mb > 0) pg->setArenaBytes(arena_mb << 20);
        return pg;
      },
      py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout") = std::chrono::milliseconds(30 * 60 * 1000),
      py::arg("arena_mb") = 0,
      py::call_guard<py::gil_scoped_release>());

  m.def("set_log_level", [](const std::string& name) { set_log_level(name); });
  m.def("get_log_level", [] { return static_cast<int>(log_level()); });

  // ---- metrics ----
  py::class_<MetricsSummary>(m, "MetricsSummary")
      .def_readonly("total_ops", &MetricsSummary::total_ops)
      .def_readonly("total_bytes", &MetricsSummary::total_bytes)
      .def_readonly("total_errors", &MetricsSummary::total_errors)
      .def_readonly("transport_bytes_sent", &MetricsSummary::transport_bytes_sent)
      .def_readonly("transport_bytes_received", &MetricsSummary::transport_bytes_received)
      .def_readonly("avg_latency_ms", &MetricsSummary::avg_latency_ms)
      .def_readonly("p50_latency_ms", &MetricsSummary::p50_latency_ms)
      .def_readonly("p99_latency_ms", &MetricsSummary::p99_latency_ms)
      .def_readonly("peak_gbps", &MetricsSummary::peak_gbps)
      .def_readonly("avg_sync_ms", &MetricsSummary::avg_sync_ms)
      .def_readonly("avg_network_ms", &MetricsSummary::avg_network_ms)
      .def_readonly("avg_reduce_ms", &MetricsSummary::avg_reduce_ms)
      .def_readonly("avg_device_ms", &MetricsSummary::avg_device_ms)
      .def_readonly("avg_queue_wait_ms", &MetricsSummary::avg_queue_wait_ms)
      .def_readonly("avg_execution_ms", &MetricsSummary::avg_execution_ms)
      .def_readonly("ops_by_name", &MetricsSummary::ops_by_name)
      .def_readonly("bytes_by_algo", &MetricsSummary::bytes_by_algo);
  m.def("get_metrics", [] { return Metrics::global().summarize(); });
  m.def("set_trace", [](const std::string& path) { Metrics::global().set_trace(path); }, py::arg("path"),
        "Append every finished op to <path>.<pid> as one Chrome-trace event per line; an empty path stops tracing.");
  m.def("enable_nvtx", [](bool on) {
    if (on)
      Metrics::global().set_nvtx([](const char* name) -> uint64_t { return static_cast<uint64_t>(nvtxRangeStartA(name)); },
                                 [](uint64_t id) { nvtxRangeEnd(static_cast<nvtxRangeId_t>(id)); });
    else
      Metrics::global().set_nvtx(nullptr, nullptr);
  }, py::arg("on") = true, "Bracket every collective with an NVTX range (also switched on by MCCL_NVTX=1 at import).");
  if (const char* nv = std::getenv("MCCL_NVTX"))
    if (nv[0] == '1')
      Metrics::global().set_nvtx([](const char* name) -> uint64_t { return static_cast<uint64_t>(nvtxRangeStartA(name)); },
                                 [](uint64_t id) { nvtxRangeEnd(static_cast<nvtxRangeId_t>(id)); });
  m.def("reset_metrics", [] { Metrics::global().reset(); });
  m.def("metrics_history", [] {
    py::list out;
    for (auto& r : Metrics::global().history()) {
      py::dict d;
      d["seq"] = r.seq;
      d["name"] = r.name;
      d["algo"] = r.algo;
      d["bytes"] = r.bytes;
      d["latency_ms"] = r.latency_ms();
      d["queue_wait_ms"] = r.queue_wait_ms();
      d["network_ms"] = r.network_ms;
      d["reduce_ms"] = r.reduce_ms;
      d["device_ms"] = r.device_ms;
      d["failed"] = r.failed;
      out.append(d);
    }
    return out;
  });
}

}  // namespace mccl
