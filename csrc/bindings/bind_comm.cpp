// Python bindings of the device communicator, the symmetric heap and the
// stand-alone element-wise kernels.
//
// The kernel bindings answer the names the reference's kernel unit tests call
// on the extension module (_metal_accumulate_chunk, _metal_elementwise_min /
// max / product, _metal_scale_inplace, _metal_accumulate_and_scale:
// tests/test_local_kernels.py:25-32,71); here they are exported as _mccl_*
// with the old names kept as aliases, each returning the destination tensor.
// CPU tensors run the host restatement of the same arithmetic.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../core/errors.hpp"
#include "../kernels/collectives.hpp"
#include "../pg/cpu_algos.hpp"
#include "../pg/device_comm.hpp"
#include "../symm/symm_mesh.hpp"
#include "bind.hpp"

namespace py = pybind11;

namespace mccl {

namespace {

DType dtype_of(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return DType::F32;
    case at::kDouble: return DType::F64;
    case at::kHalf: return DType::F16;
    case at::kBFloat16: return DType::BF16;
    case at::kInt: return DType::I32;
    case at::kLong: return DType::I64;
    case at::kChar: return DType::I8;
    case at::kShort: return DType::I16;
    case at::kByte: return DType::U8;
    case at::kBool: return DType::BOOL;
    default: MCCL_CHECK_T(false, TensorError, "unsupported dtype " << c10::toString(t.scalar_type()));
  }
  return DType::F32;
}

dev::ElemType elem_of(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return dev::ElemType::F32;
    case at::kHalf: return dev::ElemType::F16;
    case at::kBFloat16: return dev::ElemType::BF16;
    case at::kDouble: return dev::ElemType::F64;
    case at::kInt: return dev::ElemType::I32;
    case at::kLong: return dev::ElemType::I64;
    default: MCCL_CHECK_T(false, TensorError, "device kernels do not cover dtype " << c10::toString(t.scalar_type()));
  }
  return dev::ElemType::F32;
}

RedOp parse_op(const std::string& s) {
  if (s == "sum") return RedOp::SUM;
  if (s == "avg" || s == "mean") return RedOp::AVG;
  if (s == "min") return RedOp::MIN;
  if (s == "max") return RedOp::MAX;
  if (s == "product" || s == "prod") return RedOp::PRODUCT;
  if (s == "band") return RedOp::BAND;
  if (s == "bor") return RedOp::BOR;
  if (s == "bxor") return RedOp::BXOR;
  MCCL_CHECK(false, "unknown reduce op '" << s << "'");
  return RedOp::SUM;
}

Algo parse_algo(const std::string& s) {
  if (s == "auto" || s.empty()) return Algo::AUTO;
  if (s == "ring") return Algo::RING;
  if (s == "tree") return Algo::TREE;
  if (s == "butterfly" || s == "twoshot") return Algo::BUTTERFLY;
  if (s == "oneshot") return Algo::ONESHOT;
  if (s == "nvls") return Algo::NVLS;
  if (s == "twoshot_push" || s == "butterfly_push") return Algo::BUTTERFLY_PUSH;
  MCCL_CHECK(false, "unknown allreduce algorithm '" << s << "'");
  return Algo::AUTO;
}

WireDtype parse_wire(const std::string& s) { return s == "bf16" ? WireDtype::BF16 : WireDtype::NATIVE; }

int dev_op(RedOp op) {
  switch (op) {
    case RedOp::SUM: return dev::OP_SUM;
    case RedOp::AVG: return dev::OP_AVG;
    case RedOp::MIN: return dev::OP_MIN;
    case RedOp::MAX: return dev::OP_MAX;
    case RedOp::PRODUCT: return dev::OP_PROD;
    case RedOp::BAND: return dev::OP_BAND;
    case RedOp::BOR: return dev::OP_BOR;
    default: return dev::OP_BXOR;
  }
}

void check_list(DeviceComm& c, const std::vector<at::Tensor>& ts, const char* what) {
  MCCL_CHECK_TENSOR(static_cast<int>(ts.size()) == c.nlocal(),
                    what << ": expected " << c.nlocal() << " tensor(s), got " << ts.size());
  for (auto& t : ts) {
    MCCL_CHECK_TENSOR(t.is_cuda() && t.get_device() == c.device(), what << ": tensors must live on cuda:" << c.device());
    MCCL_CHECK_TENSOR(t.is_contiguous(), what << ": tensors must be contiguous");
    MCCL_CHECK_TENSOR(t.scalar_type() == ts[0].scalar_type() && t.numel() == ts[0].numel(), what << ": tensors must match");
  }
}

std::vector<const void*> cptrs(const std::vector<at::Tensor>& ts) {
  std::vector<const void*> p;
  for (auto& t : ts) p.push_back(t.data_ptr());
  return p;
}
std::vector<void*> mptrs(const std::vector<at::Tensor>& ts) {
  std::vector<void*> p;
  for (auto& t : ts) p.push_back(t.data_ptr());
  return p;
}
void* cur_stream(int device) { return static_cast<void*>(at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream()); }

// dst ∘= src on either device.
at::Tensor binary_kernel(at::Tensor dst, const at::Tensor& src, RedOp op) {
  MCCL_CHECK_TENSOR(dst.scalar_type() == src.scalar_type() && dst.numel() == src.numel() && dst.device() == src.device(),
                    "kernel operands must match in dtype, size and device");
  MCCL_CHECK_TENSOR(dst.is_contiguous() && src.is_contiguous(), "kernel operands must be contiguous");
  if (dst.is_cuda()) {
    c10::cuda::CUDAGuard g(dst.device());
    cudaError_t rc = dev::launch_reduce2(elem_of(dst), dev_op(op), dst.data_ptr(), src.data_ptr(), dst.numel(),
                                         at::cuda::getCurrentCUDAStream().stream());
    MCCL_CHECK_T(rc == cudaSuccess, CudaError, "reduce2 launch failed: " << cudaGetErrorString(rc));
  } else {
    reduce_into(dtype_of(dst), op, dst.data_ptr(), src.data_ptr(), static_cast<size_t>(dst.numel()));
  }
  return dst;
}

}  // namespace

void bind_comm(py::module_& m) {
  py::class_<SymmAlloc, std::shared_ptr<SymmAlloc>>(m, "SymmAlloc")
      .def_readonly("nbytes", &SymmAlloc::bytes)
      .def_readonly("world", &SymmAlloc::world)
      .def_readonly("rank", &SymmAlloc::rank)
      .def_property_readonly("has_multicast", [](const SymmAlloc& a) { return a.mc_ptr != nullptr; })
      .def("ptr", [](const SymmAlloc& a, int r) { return reinterpret_cast<uintptr_t>(a.ptrs[r]); })
      .def(
          "tensor",
          [](std::shared_ptr<SymmAlloc> a, int r, int64_t byte_offset, std::vector<int64_t> shape, at::ScalarType dtype,
             int device) {
            int64_t n = 1;
            for (auto s : shape) n *= s;
            MCCL_CHECK_TENSOR(r >= 0 && r < a->world && a->ptrs[r] != nullptr, "no mapping for rank " << r);
            MCCL_CHECK_TENSOR(byte_offset >= 0 && byte_offset + n * static_cast<int64_t>(c10::elementSize(dtype)) <=
                                                      static_cast<int64_t>(a->bytes),
                              "view exceeds the symmetric allocation");
            auto opts = at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
            // target_device: a peer's block is physically on another GPU, which the pointer query behind from_blob
            // would report; the mapping is addressable from `device`, and that is where kernels on it run
            return at::for_blob(static_cast<char*>(a->ptrs[r]) + byte_offset, shape)
                .deleter([a](void*) {})
                .options(opts)
                .target_device(opts.device())
                .make_tensor();
          },
          py::arg("rank"), py::arg("byte_offset"), py::arg("shape"), py::arg("dtype"), py::arg("device"),
          "View of rank `rank`'s block (as mapped in this process) as a tensor; the view keeps the allocation alive.  For "
          "rank != this rank the tensor aliases another GPU's memory: use it only with plain elementwise copies or this "
          "package's own kernels, never as an operand of a library kernel (matmul, attention, ...), which may issue "
          "cluster-multicast bulk loads that must not read a peer's memory.");

  py::class_<DeviceComm, std::shared_ptr<DeviceComm>>(m, "DeviceComm")
      .def(py::init([](int world, int device) { return std::make_shared<DeviceComm>(world, device, EnvConfig::from_env()); }),
           py::arg("world"), py::arg("device") = 0,
           "Single-process communicator with `world` virtual ranks on one GPU (kernel tests).")
      .def_property_readonly("rank", &DeviceComm::rank)
      .def_property_readonly("world", &DeviceComm::world)
      .def_property_readonly("device", &DeviceComm::device)
      .def_property_readonly("nlocal", &DeviceComm::nlocal)
      .def_property_readonly("nvls_available", &DeviceComm::nvls_available)
      .def_property_readonly("arena_bytes", &DeviceComm::arena_bytes)
      .def_property_readonly("symm_mode", [](DeviceComm& c) { return std::string(c.symm_mode()); })
      .def_property_readonly("launches", &DeviceComm::launches)
      .def("status", &DeviceComm::status)
      .def("check_status", &DeviceComm::check_status)
      .def("clear_status", &DeviceComm::clear_status)
      .def("check_canaries", &DeviceComm::check_canaries)
      .def_property_readonly("debug_bounds", &DeviceComm::debug_bounds)
      .def("set_debug_arena_limit", &DeviceComm::set_debug_arena_limit, py::arg("nbytes"))
      .def("inject_skip_signals", &DeviceComm::inject_skip_signals, py::arg("count") = 1)
      .def("set_device_timeout_ms", &DeviceComm::set_device_timeout_ms)
      .def_property_readonly("device_timeout_ms", &DeviceComm::device_timeout_ms)
      .def_property_readonly("max_ctas", &DeviceComm::max_ctas)
      .def_property_readonly("launch_threads", &DeviceComm::launch_threads)
      .def_property_readonly("launch_shape_auto", &DeviceComm::launch_shape_auto)
      .def("set_launch_shape", &DeviceComm::set_launch_shape, py::arg("max_ctas") = 0, py::arg("threads") = 0)
      .def("decide_allreduce",
           [](DeviceComm& c, const std::string& algo, int64_t numel, at::ScalarType dt, const std::string& op,
              const std::string& wire, int64_t tree_below) {
             at::Tensor probe = at::empty({0}, at::TensorOptions().dtype(dt));
             return std::string(algo_name(c.decide_allreduce(parse_algo(algo), static_cast<size_t>(numel), dtype_of(probe),
                                                             parse_op(op), parse_wire(wire), tree_below)));
           },
           py::arg("algo"), py::arg("numel"), py::arg("dtype"), py::arg("op") = "sum", py::arg("wire") = "native",
           py::arg("tree_below") = 262144)
      .def(
          "allreduce",
          [](DeviceComm& c, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, const std::string& op,
             const std::string& algo, const std::string& wire, int64_t tree_below) {
            check_list(c, ins, "allreduce(in)");
            check_list(c, outs, "allreduce(out)");
            c10::cuda::CUDAGuard g(ins[0].device());
            auto ip = cptrs(ins);
            auto op_ = mptrs(outs);
            Algo ran = c.allreduce(ip.data(), op_.data(), static_cast<size_t>(ins[0].numel()), dtype_of(ins[0]),
                                   parse_op(op), parse_algo(algo), parse_wire(wire), tree_below, cur_stream(c.device()));
            return std::string(algo_name(ran));
          },
          py::arg("ins"), py::arg("outs"), py::arg("op") = "sum", py::arg("algo") = "auto", py::arg("wire") = "native",
          py::arg("tree_below") = 262144)
      .def(
          "reduce_scatter",
          [](DeviceComm& c, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, const std::string& op,
             const std::string& wire) {
            check_list(c, ins, "reduce_scatter(in)");
            check_list(c, outs, "reduce_scatter(out)");
            MCCL_CHECK_TENSOR(ins[0].numel() == outs[0].numel() * c.world(), "reduce_scatter: in must hold world * out elements");
            c10::cuda::CUDAGuard g(ins[0].device());
            auto ip = cptrs(ins);
            auto op_ = mptrs(outs);
            c.reduce_scatter(ip.data(), op_.data(), static_cast<size_t>(outs[0].numel()), dtype_of(ins[0]), parse_op(op),
                             parse_wire(wire), cur_stream(c.device()));
          },
          py::arg("ins"), py::arg("outs"), py::arg("op") = "sum", py::arg("wire") = "native")
      .def(
          "allgather",
          [](DeviceComm& c, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs) {
            check_list(c, ins, "allgather(in)");
            check_list(c, outs, "allgather(out)");
            MCCL_CHECK_TENSOR(outs[0].numel() == ins[0].numel() * c.world(), "allgather: out must hold world * in elements");
            c10::cuda::CUDAGuard g(ins[0].device());
            auto ip = cptrs(ins);
            auto op_ = mptrs(outs);
            c.allgather(ip.data(), op_.data(), static_cast<size_t>(ins[0].numel()) * ins[0].element_size(), cur_stream(c.device()));
          },
          py::arg("ins"), py::arg("outs"))
      .def(
          "broadcast",
          [](DeviceComm& c, std::vector<at::Tensor> datas, int root) {
            check_list(c, datas, "broadcast");
            c10::cuda::CUDAGuard g(datas[0].device());
            auto dp = mptrs(datas);
            c.broadcast(dp.data(), static_cast<size_t>(datas[0].numel()) * datas[0].element_size(), root, cur_stream(c.device()));
          },
          py::arg("tensors"), py::arg("root") = 0)
      .def(
          "alltoallv",
          [](DeviceComm& c, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs,
             std::vector<std::vector<int64_t>> in_splits, std::vector<std::vector<int64_t>> out_splits) {
            MCCL_CHECK_TENSOR(static_cast<int>(ins.size()) == c.nlocal() && static_cast<int>(outs.size()) == c.nlocal(),
                              "alltoallv: need one input and one output per local rank");
            const int N = c.world();
            std::vector<std::vector<size_t>> ioff(ins.size()), ilen(ins.size()), ooff(ins.size()), olen(ins.size());
            for (size_t v = 0; v < ins.size(); ++v) {
              size_t es = ins[v].element_size(), a = 0, b = 0;
              for (int p = 0; p < N; ++p) {
                ioff[v].push_back(a);
                ilen[v].push_back(static_cast<size_t>(in_splits[v][p]) * es);
                a += ilen[v].back();
                ooff[v].push_back(b);
                olen[v].push_back(static_cast<size_t>(out_splits[v][p]) * es);
                b += olen[v].back();
              }
            }
            c10::cuda::CUDAGuard g(ins[0].device());
            auto ip = cptrs(ins);
            auto op_ = mptrs(outs);
            c.alltoallv(ip.data(), op_.data(), ioff, ilen, ooff, olen, cur_stream(c.device()));
          },
          py::arg("ins"), py::arg("outs"), py::arg("in_splits"), py::arg("out_splits"),
          "Split sizes are element counts per peer, one list per local rank.")
      .def(
          "send",
          [](DeviceComm& c, const at::Tensor& t, int peer) {
            MCCL_CHECK_TENSOR(t.is_cuda() && t.is_contiguous() && t.get_device() == c.device(), "send: contiguous tensor on cuda:" << c.device() << " expected");
            c10::cuda::CUDAGuard g(t.device());
            c.send(t.data_ptr(), static_cast<size_t>(t.numel()) * t.element_size(), peer, cur_stream(c.device()));
          },
          py::arg("tensor"), py::arg("peer"))
      .def(
          "recv",
          [](DeviceComm& c, at::Tensor t, int peer) {
            MCCL_CHECK_TENSOR(t.is_cuda() && t.is_contiguous() && t.get_device() == c.device(), "recv: contiguous tensor on cuda:" << c.device() << " expected");
            c10::cuda::CUDAGuard g(t.device());
            c.recv(t.data_ptr(), static_cast<size_t>(t.numel()) * t.element_size(), peer, cur_stream(c.device()));
          },
          py::arg("tensor"), py::arg("peer"))
      .def(
          "p2p_emulated",
          [](DeviceComm& c, std::vector<at::Tensor> bufs, std::vector<int> peers, std::vector<bool> is_send) {
            MCCL_CHECK_TENSOR(static_cast<int>(bufs.size()) == c.nlocal() && peers.size() == bufs.size() && is_send.size() == bufs.size(),
                              "p2p_emulated: one buffer, peer and direction per virtual rank expected");
            std::vector<DeviceComm::P2POp> ops(bufs.size());
            size_t nbytes = 0;
            for (size_t v = 0; v < bufs.size(); ++v) {
              if (peers[v] < 0) continue;
              MCCL_CHECK_TENSOR(bufs[v].is_cuda() && bufs[v].is_contiguous(), "p2p_emulated: contiguous CUDA tensors expected");
              const size_t nb = static_cast<size_t>(bufs[v].numel()) * bufs[v].element_size();
              MCCL_CHECK_TENSOR(nbytes == 0 || nb == nbytes, "p2p_emulated: all transfers of one launch have the same size");
              nbytes = nb;
              ops[v].buf = bufs[v].data_ptr();
              ops[v].peer = peers[v];
              ops[v].is_send = is_send[v];
            }
            c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(c.device())));
            c.p2p_emulated(ops, nbytes, cur_stream(c.device()));
          },
          py::arg("bufs"), py::arg("peers"), py::arg("is_send"),
          "Single-GPU emulation: virtual rank v sends bufs[v] to / receives bufs[v] from peers[v] (-1: idle), all in one launch.")
      .def_property_readonly("p2p_slot_bytes", &DeviceComm::p2p_slot_bytes)
      .def("barrier", [](DeviceComm& c) {
        c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(c.device())));
        c.barrier(cur_stream(c.device()));
      })
      .def("symm_alloc", &DeviceComm::symm_alloc, py::arg("nbytes"), py::call_guard<py::gil_scoped_release>())
      .def(
          "allreduce_symm",
          [](DeviceComm& c, std::shared_ptr<SymmAlloc> buf, int64_t byte_offset, int64_t numel, at::ScalarType dt,
             const std::string& op) {
            at::Tensor probe = at::empty({0}, at::TensorOptions().dtype(dt));
            c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(c.device())));
            Algo ran = c.allreduce_symm(*buf, static_cast<size_t>(byte_offset), static_cast<size_t>(numel), dtype_of(probe),
                                        parse_op(op), cur_stream(c.device()));
            return std::string(algo_name(ran));
          },
          py::arg("buf"), py::arg("byte_offset"), py::arg("numel"), py::arg("dtype"), py::arg("op") = "sum");

  // ---- stand-alone element-wise kernels ----
  m.def("_mccl_accumulate_chunk", [](at::Tensor d, const at::Tensor& s) { return binary_kernel(d, s, RedOp::SUM); });
  m.def("_mccl_elementwise_min", [](at::Tensor d, const at::Tensor& s) { return binary_kernel(d, s, RedOp::MIN); });
  m.def("_mccl_elementwise_max", [](at::Tensor d, const at::Tensor& s) { return binary_kernel(d, s, RedOp::MAX); });
  m.def("_mccl_elementwise_product", [](at::Tensor d, const at::Tensor& s) { return binary_kernel(d, s, RedOp::PRODUCT); });
  m.def("_mccl_scale_inplace", [](at::Tensor t, double scale) {
    MCCL_CHECK_TENSOR(t.is_contiguous(), "scale: tensor must be contiguous");
    if (t.is_cuda()) {
      c10::cuda::CUDAGuard g(t.device());
      cudaError_t rc = dev::launch_scale(elem_of(t), t.data_ptr(), t.numel(), static_cast<float>(scale),
                                         at::cuda::getCurrentCUDAStream().stream());
      MCCL_CHECK_T(rc == cudaSuccess, CudaError, "scale launch failed: " << cudaGetErrorString(rc));
    } else {
      scale_inplace(dtype_of(t), t.data_ptr(), static_cast<size_t>(t.numel()), scale);
    }
    return t;
  });
  m.def("_mccl_accumulate_and_scale", [](at::Tensor d, const at::Tensor& s, double scale) {
    MCCL_CHECK_TENSOR(d.scalar_type() == s.scalar_type() && d.numel() == s.numel() && d.device() == s.device(),
                      "kernel operands must match in dtype, size and device");
    MCCL_CHECK_TENSOR(d.is_contiguous() && s.is_contiguous(), "kernel operands must be contiguous");
    if (d.is_cuda()) {
      c10::cuda::CUDAGuard g(d.device());
      cudaError_t rc = dev::launch_reduce2_scale(elem_of(d), d.data_ptr(), s.data_ptr(), d.numel(), static_cast<float>(scale),
                                                 at::cuda::getCurrentCUDAStream().stream());
      MCCL_CHECK_T(rc == cudaSuccess, CudaError, "reduce2_scale launch failed: " << cudaGetErrorString(rc));
    } else {
      reduce_scale(dtype_of(d), d.data_ptr(), s.data_ptr(), static_cast<size_t>(d.numel()), scale);
    }
    return d;
  });
  for (const char* n : {"accumulate_chunk", "elementwise_min", "elementwise_max", "elementwise_product", "scale_inplace",
                        "accumulate_and_scale"})
    m.attr((std::string("_metal_") + n).c_str()) = m.attr((std::string("_mccl_") + n).c_str());
}

}  // namespace mccl
