// Python bindings of the model-operator kernels.  Every function checks its
// operands, allocates outputs through torch, and launches on the current
// CUDA stream of the operands' device (so the calls can be captured in a CUDA
// graph).  There is no CPU fallback here: a CPU tensor is an error.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../core/errors.hpp"
#include "../core/launch.hpp"
#include "../core/timeline.hpp"
#include "../ops/ops.hpp"
#include "../ops/tp_gemm.hpp"
#include "../pg/device_comm.hpp"
#include "../symm/symm_mesh.hpp"
#include "bind.hpp"

namespace py = pybind11;

namespace mccl {

namespace {

void need_cuda(const at::Tensor& t, const char* what) {
  MCCL_CHECK_TENSOR(t.defined() && t.is_cuda(), what << ": expected a CUDA tensor");
}
void need(const at::Tensor& t, at::ScalarType dt, const char* what) {
  need_cuda(t, what);
  MCCL_CHECK_TENSOR(t.scalar_type() == dt, what << ": expected dtype " << c10::toString(dt) << ", got "
                                                << c10::toString(t.scalar_type()));
  MCCL_CHECK_TENSOR(t.is_contiguous(), what << ": expected a contiguous tensor");
}
cudaStream_t stream_of(const at::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }
void check_launch(cudaError_t rc, const char* what) {
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, what << " failed: " << cudaGetErrorString(rc));
}
__nv_bfloat16* bf(const at::Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }

int parse_epilogue(const std::string& s, bool has_bias) {
  if (s == "none") return has_bias ? ops::EPI_BIAS : ops::EPI_NONE;
  if (s == "gelu") return has_bias ? ops::EPI_BIAS_GELU : ops::EPI_GELU;
  if (s == "gelu_d") return has_bias ? ops::EPI_BIAS_GELU_D : ops::EPI_GELU_D;   // aux = gelu'(z) instead of z
  MCCL_CHECK(false, "unknown GEMM epilogue '" << s << "'");
  return 0;
}

}  // namespace

void bind_ops(py::module_& m) {
  m.def("op_launch_count", [] { return ops::launch_count(); });
  m.def("gemm_error_flag", [] { return ops::gemm_error_flag(); });
  // ---- launch tracer: every kernel of this package goes through MCCL_LAUNCH (csrc/core/launch.hpp) ----
  m.def("launch_counts", [] { return launch_counts(); }, "Launches per kernel name since the process started.");
  m.def("launch_counts_reset", [] { launch_counts_reset(); });
  m.def("launch_total", [] { return launch_total(); });
  m.def("set_gemm_kernel", &ops::set_gemm_kernel, py::arg("name"),
        "Kernel for plain products from now on: 'pair' (CTA pairs, tcgen05.mma.cta_group::2; the default), 'persistent' "
        "(one CTA per SM), 'tile' (one tile per CTA); '' returns to MCCL_GEMM_KERNEL / the default.");
  m.def("set_gemm_cta_limit", &ops::set_gemm_cta_limit, py::arg("ctas"),
        "Caps the CTAs (SMs) of plain GEMM launches from now on; 0 = one per SM.");
  m.def("gemm_cta_limit", &ops::gemm_cta_limit);
  m.def("gemm_sm_count", &ops::gemm_sm_count);

  // ---- device timeline (kernels stamp %globaltimer; see csrc/core/timeline.hpp) ----
  m.def("timeline_enable", [](int device, int capacity, int every, int detail) {
    c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
    timeline_enable(capacity, every, detail);
  }, py::arg("device"), py::arg("capacity") = 65536, py::arg("every") = 1, py::arg("detail") = 0);
  m.def("timeline_disable", [](int device) {
    c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
    timeline_disable();
  }, py::arg("device"));
  m.def("timeline_drain", [](int device) {
    c10::cuda::CUDAGuard g(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
    std::vector<TimelineRec> recs = timeline_drain();
    at::Tensor out = at::empty({static_cast<int64_t>(recs.size()), 6}, at::TensorOptions().dtype(at::kLong));
    int64_t* p = out.data_ptr<int64_t>();
    for (size_t i = 0; i < recs.size(); ++i) {
      p[6 * i + 0] = static_cast<int64_t>(recs[i].t0);
      p[6 * i + 1] = static_cast<int64_t>(recs[i].t1);
      p[6 * i + 2] = recs[i].kind;
      p[6 * i + 3] = recs[i].tag;
      p[6 * i + 4] = recs[i].sm;
      p[6 * i + 5] = recs[i].cta;
    }
    return out;
  }, py::arg("device"), "Rows of (t0 ns, t1 ns, kind, tag, sm, cta), sorted by t0; rewinds the buffer.");

  // D[M,N] = A[M,K] · B[N,K]^T.  A and B are 2-D bf16 with unit inner stride
  // (row strides may exceed the row length).  With a_t (b_t) the operand is
  // passed as stored [K, M] ([K, N]) and read MN-major, so no transposed copy is
  // needed for weight-gradient and input-gradient products.
  // Returns (D, pre_activation or None).
  m.def(
      "gemm_bf16",
      [](const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& bias, const std::string& epilogue,
         bool out_fp32, const c10::optional<at::Tensor>& out, bool accumulate, bool a_t, bool b_t,
         const c10::optional<at::Tensor>& residual, const c10::optional<at::Tensor>& mul) {
        need_cuda(a, "gemm(a)");
        need_cuda(b, "gemm(b)");
        MCCL_CHECK_TENSOR(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: operands must be bf16");
        MCCL_CHECK_TENSOR(a.dim() == 2 && b.dim() == 2, "gemm: 2-D operands expected");
        MCCL_CHECK_TENSOR(a.stride(1) == 1 && b.stride(1) == 1, "gemm: operands need unit inner stride");
        c10::cuda::CUDAGuard guard(a.device());
        // a_t: a is stored [K, M]; b_t: b is stored [K, N].
        const int64_t M = a_t ? a.size(1) : a.size(0), K = a_t ? a.size(0) : a.size(1);
        const int64_t N = b_t ? b.size(1) : b.size(0);
        MCCL_CHECK_TENSOR((b_t ? b.size(0) : b.size(1)) == K, "gemm: contraction sizes differ");
        at::Tensor d;
        if (out.has_value()) {
          d = *out;
          need_cuda(d, "gemm(out)");
          MCCL_CHECK_TENSOR(d.dim() == 2 && d.size(0) == M && d.size(1) == N && d.stride(1) == 1, "gemm: bad output shape");
          MCCL_CHECK_TENSOR(d.scalar_type() == (out_fp32 ? at::kFloat : at::kBFloat16), "gemm: output dtype mismatch");
        } else {
          d = at::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
        }
        ops::GemmArgs g;
        g.a = bf(a);
        g.b = bf(b);
        g.d = d.data_ptr();
        g.m = static_cast<int>(M);
        g.n = static_cast<int>(N);
        g.k = static_cast<int>(K);
        g.lda = static_cast<int>(a.stride(0));
        g.ldb = static_cast<int>(b.stride(0));
        g.ldd = static_cast<int>(d.stride(0));
        g.d_fp32 = out_fp32;
        g.accumulate = accumulate;
        g.a_mn_major = a_t;
        g.b_mn_major = b_t;
        at::Tensor bias_f;
        if (bias.has_value() && bias->defined()) {
          need(*bias, at::kFloat, "gemm(bias)");
          MCCL_CHECK_TENSOR(bias->numel() == N, "gemm: bias must have N elements");
          g.bias = bias->data_ptr<float>();
        }
        g.epilogue = parse_epilogue(epilogue, g.bias != nullptr);
        at::Tensor aux;
        if (g.epilogue == ops::EPI_BIAS_GELU || g.epilogue == ops::EPI_GELU || g.epilogue == ops::EPI_BIAS_GELU_D ||
            g.epilogue == ops::EPI_GELU_D) {
          MCCL_CHECK_TENSOR(d.is_contiguous(), "gemm: GELU epilogue needs a contiguous output");
          aux = at::empty({M, N}, a.options());
          g.aux = bf(aux);
        }
        if (residual.has_value() && residual->defined()) {
          need(*residual, at::kBFloat16, "gemm(residual)");
          MCCL_CHECK_TENSOR(residual->numel() == M * N && d.is_contiguous(), "gemm: residual must be a contiguous [M, N] tensor");
          g.residual = bf(*residual);
        }
        if (mul.has_value() && mul->defined()) {
          need(*mul, at::kBFloat16, "gemm(mul)");
          MCCL_CHECK_TENSOR(mul->numel() == M * N && d.is_contiguous() && !out_fp32,
                            "gemm: mul must be a contiguous [M, N] bf16 tensor and the output bf16");
          g.mul = bf(*mul);
        }
        cudaError_t rc = ops::gemm_bf16_tn(g, stream_of(a));
        MCCL_CHECK_T(rc == cudaSuccess, CudaError,
                     "gemm_bf16 [" << M << "x" << N << "x" << K << ", lda " << g.lda << ", ldb " << g.ldb << ", ldd " << g.ldd
                                   << "] failed: " << cudaGetErrorString(rc) << " " << ops::gemm_last_reason());
        return std::make_pair(d, aux.defined() ? c10::optional<at::Tensor>(aux) : c10::nullopt);
      },
      py::arg("a"), py::arg("b"), py::arg("bias") = py::none(), py::arg("epilogue") = "none", py::arg("out_fp32") = false,
      py::arg("out") = py::none(), py::arg("accumulate") = false, py::arg("a_t") = false, py::arg("b_t") = false,
      py::arg("residual") = py::none(), py::arg("mul") = py::none());

  m.def(
      "norm_fwd",
      [](const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& b, double eps) {
        need(x, at::kBFloat16, "norm(x)");
        need(w, at::kFloat, "norm(weight)");
        c10::cuda::CUDAGuard guard(x.device());
        const int64_t dim = x.size(-1), rows = x.numel() / dim;
        MCCL_CHECK_TENSOR(w.numel() == dim, "norm: weight must have `dim` elements");
        const float* bp = nullptr;
        if (b.has_value() && b->defined()) {
          need(*b, at::kFloat, "norm(bias)");
          bp = b->data_ptr<float>();
        }
        at::Tensor y = at::empty_like(x);
        at::Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
        at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
        check_launch(ops::norm_fwd(bf(x), w.data_ptr<float>(), bp, bf(y), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                   static_cast<int>(rows), static_cast<int>(dim), static_cast<float>(eps), stream_of(x)),
                     "norm_fwd");
        return std::make_tuple(y, mean, rstd);
      },
      py::arg("x"), py::arg("weight"), py::arg("bias") = py::none(), py::arg("eps") = 1e-5);

  m.def(
      "norm_bwd",
      [](const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& mean, const at::Tensor& rstd,
         bool layernorm, const c10::optional<at::Tensor>& dw_out, const c10::optional<at::Tensor>& db_out, bool accumulate,
         const c10::optional<at::Tensor>& dx_add, int parts) {
        need(dy, at::kBFloat16, "norm_bwd(dy)");
        const __nv_bfloat16* addp = nullptr;
        if (dx_add.has_value() && dx_add->defined()) {
          need(*dx_add, at::kBFloat16, "norm_bwd(dx_add)");
          MCCL_CHECK_TENSOR(dx_add->numel() == x.numel(), "norm_bwd: dx_add must have the shape of x");
          addp = bf(*dx_add);
        }
        need(x, at::kBFloat16, "norm_bwd(x)");
        need(w, at::kFloat, "norm_bwd(weight)");
        need(mean, at::kFloat, "norm_bwd(mean)");
        need(rstd, at::kFloat, "norm_bwd(rstd)");
        c10::cuda::CUDAGuard guard(x.device());
        const int64_t dim = x.size(-1), rows = x.numel() / dim;
        at::Tensor dx = (parts & 1) ? at::empty_like(x) : at::Tensor();   // parts: 1 = dx only, 2 = parameter gradients only
        // dw_out / db_out: write the parameter gradients straight into these fp32 buffers
        at::Tensor dw = dw_out.has_value() ? *dw_out : at::empty({dim}, x.options().dtype(at::kFloat));
        at::Tensor db = !layernorm ? at::Tensor() : (db_out.has_value() ? *db_out : at::empty({dim}, x.options().dtype(at::kFloat)));
        need(dw, at::kFloat, "norm_bwd(dw)");
        if (layernorm) need(db, at::kFloat, "norm_bwd(db)");
        MCCL_CHECK_TENSOR(dw.numel() == dim && (!layernorm || db.numel() == dim), "norm_bwd: gradient buffers must have `dim` elements");
        // accumulate: add into dw / db (one pass, atomics) instead of overwriting them (two passes, fixed order)
        at::Tensor scratch;
        if (!accumulate)
          scratch = at::empty({2 * ops::colsum_slabs(static_cast<int>(rows)) * dim}, x.options().dtype(at::kFloat));
        check_launch(ops::norm_bwd(bf(dy), bf(x), w.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                   dx.defined() ? bf(dx) : nullptr,
                                   dw.data_ptr<float>(), layernorm ? db.data_ptr<float>() : nullptr,
                                   accumulate ? nullptr : scratch.data_ptr<float>(),
                                   static_cast<int>(rows),
                                   static_cast<int>(dim), layernorm, stream_of(x), addp, parts),
                     "norm_bwd");
        return std::make_tuple(dx.defined() ? c10::optional<at::Tensor>(dx) : c10::nullopt, dw,
                               db.defined() ? c10::optional<at::Tensor>(db) : c10::nullopt);
      },
      py::arg("dy"), py::arg("x"), py::arg("weight"), py::arg("mean"), py::arg("rstd"), py::arg("layernorm"),
      py::arg("dw_out") = py::none(), py::arg("db_out") = py::none(), py::arg("accumulate") = false,
      py::arg("dx_add") = py::none(), py::arg("parts") = 3);

  m.def(
      "adamw_flat",
      [](at::Tensor p, const at::Tensor& g, at::Tensor mm, at::Tensor v, const c10::optional<at::Tensor>& p16, double lr,
         double b1, double b2, double eps, double wd, const at::Tensor& step, double grad_scale, bool zero_grad, int ctas_per_sm) {
        need(p, at::kFloat, "adamw(p)");
        need(g, at::kFloat, "adamw(g)");
        need(mm, at::kFloat, "adamw(m)");
        need(v, at::kFloat, "adamw(v)");
        need(step, at::kFloat, "adamw(step)");
        MCCL_CHECK_TENSOR(g.numel() == p.numel() && mm.numel() == p.numel() && v.numel() == p.numel(), "adamw: size mismatch");
        c10::cuda::CUDAGuard guard(p.device());
        __nv_bfloat16* p16p = nullptr;
        if (p16.has_value() && p16->defined()) {
          need(*p16, at::kBFloat16, "adamw(p_bf16)");
          MCCL_CHECK_TENSOR(p16->numel() == p.numel(), "adamw: bf16 copy size mismatch");
          p16p = bf(*p16);
        }
        check_launch(ops::adamw_flat(p.data_ptr<float>(), const_cast<float*>(g.data_ptr<float>()), mm.data_ptr<float>(),
                                     v.data_ptr<float>(), p16p, p.numel(), static_cast<float>(lr), static_cast<float>(b1),
                                     static_cast<float>(b2), static_cast<float>(eps), static_cast<float>(wd),
                                     step.data_ptr<float>(), static_cast<float>(grad_scale), stream_of(p), zero_grad, ctas_per_sm),
                     "adamw_flat");
      },
      py::arg("p"), py::arg("g"), py::arg("m"), py::arg("v"), py::arg("p_bf16") = py::none(), py::arg("lr") = 1e-3,
      py::arg("beta1") = 0.9, py::arg("beta2") = 0.999, py::arg("eps") = 1e-8, py::arg("weight_decay") = 0.01,
      py::arg("step") = at::Tensor(), py::arg("grad_scale") = 1.0, py::arg("zero_grad") = false, py::arg("ctas_per_sm") = 8);

  m.def(
      "ce_fwd_bwd",
      [](at::Tensor logits, const at::Tensor& targets, double grad_scale) {
        need(logits, at::kBFloat16, "cross_entropy(logits)");
        need(targets, at::kLong, "cross_entropy(targets)");
        MCCL_CHECK_TENSOR(logits.dim() == 2 && targets.numel() == logits.size(0), "cross_entropy: logits [T,V], targets [T]");
        c10::cuda::CUDAGuard guard(logits.device());
        at::Tensor loss_rows = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
        check_launch(ops::cross_entropy_fwd_bwd(bf(logits), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                                                loss_rows.data_ptr<float>(), static_cast<int>(logits.size(0)),
                                                static_cast<int>(logits.size(1)), static_cast<float>(grad_scale),
                                                stream_of(logits)),
                     "cross_entropy");
        return loss_rows;
      },
      py::arg("logits"), py::arg("targets"), py::arg("grad_scale") = 1.0,
      "Returns per-row losses; overwrites logits with (softmax - onehot) * grad_scale.");

  // ---- causal self-attention (head dimension 64) on the fused QKV projection ----
  m.def(
      "attn_fwd",
      [](const at::Tensor& qkv, double scale) {
        need(qkv, at::kBFloat16, "attention(qkv)");
        MCCL_CHECK_TENSOR(qkv.dim() == 5 && qkv.size(2) == 3 && qkv.size(4) == 64, "attention: qkv must be [B, S, 3, H, 64]");
        const int64_t B = qkv.size(0), S = qkv.size(1), H = qkv.size(3);
        c10::cuda::CUDAGuard guard(qkv.device());
        at::Tensor o = at::empty({B, S, H * 64}, qkv.options());
        at::Tensor lse = at::empty({B, H, S}, qkv.options().dtype(at::kFloat));
        cudaError_t rc = ops::attention_fwd(bf(qkv), bf(o), lse.data_ptr<float>(), static_cast<int>(B), static_cast<int>(S),
                                            static_cast<int>(H), static_cast<float>(scale), stream_of(qkv));
        MCCL_CHECK_T(rc == cudaSuccess, CudaError, "attention forward [B " << B << ", S " << S << ", H " << H << "] failed: "
                                                                           << cudaGetErrorString(rc));
        return std::make_pair(o, lse);
      },
      py::arg("qkv"), py::arg("scale"), "Causal attention; returns (o [B, S, H*64] bf16, lse [B, H, S] fp32, log2 domain).  S % 128 == 0.");
  m.def(
      "attn_bwd",
      [](const at::Tensor& qkv, const at::Tensor& o, const at::Tensor& d_o, const at::Tensor& lse, double scale) {
        need(qkv, at::kBFloat16, "attention_bwd(qkv)");
        need(o, at::kBFloat16, "attention_bwd(o)");
        need(d_o, at::kBFloat16, "attention_bwd(d_o)");
        need(lse, at::kFloat, "attention_bwd(lse)");
        MCCL_CHECK_TENSOR(qkv.dim() == 5 && qkv.size(2) == 3 && qkv.size(4) == 64, "attention_bwd: qkv must be [B, S, 3, H, 64]");
        const int64_t B = qkv.size(0), S = qkv.size(1), H = qkv.size(3);
        MCCL_CHECK_TENSOR(o.numel() == B * S * H * 64 && d_o.numel() == o.numel() && lse.numel() == B * H * S,
                          "attention_bwd: operand sizes do not match qkv");
        c10::cuda::CUDAGuard guard(qkv.device());
        at::Tensor dqkv = at::empty_like(qkv);
        cudaError_t rc = ops::attention_bwd(bf(qkv), bf(o), bf(d_o), lse.data_ptr<float>(), bf(dqkv), static_cast<int>(B),
                                            static_cast<int>(S), static_cast<int>(H), static_cast<float>(scale), stream_of(qkv));
        MCCL_CHECK_T(rc == cudaSuccess, CudaError, "attention backward [B " << B << ", S " << S << ", H " << H << "] failed: "
                                                                            << cudaGetErrorString(rc));
        return dqkv;
      },
      py::arg("qkv"), py::arg("o"), py::arg("d_o"), py::arg("lse"), py::arg("scale"),
      "Gradient of the whole qkv tensor.  S must be 128 or 256.");

  // ---- tensor-parallel GEMMs fused with their collective ----
  py::class_<ops::TpGemm>(m, "TpGemm")
      .def(py::init<std::shared_ptr<DeviceComm>, size_t>(), py::arg("comm"), py::arg("max_rs_elems"),
           py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("world", &ops::TpGemm::world)
      .def_property_readonly("rank", &ops::TpGemm::rank)
      .def("status", &ops::TpGemm::status)
      .def("check_status", &ops::TpGemm::check_status)
      .def(
          "ag_gemm",
          [](ops::TpGemm& t, std::shared_ptr<SymmAlloc> x_sym, int64_t x_off, int64_t rows_local, const at::Tensor& w, bool w_kn,
             const c10::optional<at::Tensor>& bias, const std::string& epilogue) {
            need_cuda(w, "ag_gemm(w)");
            MCCL_CHECK_TENSOR(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1, "ag_gemm: w must be 2-D bf16");
            c10::cuda::CUDAGuard guard(w.device());
            const int64_t K = w_kn ? w.size(0) : w.size(1), N = w_kn ? w.size(1) : w.size(0);
            const int64_t rows = rows_local * t.world();
            at::Tensor y = at::empty({rows, N}, w.options());
            at::Tensor gathered = at::empty({rows, K}, w.options());
            const float* bp = nullptr;
            if (bias.has_value() && bias->defined()) {
              need(*bias, at::kFloat, "ag_gemm(bias)");
              bp = bias->data_ptr<float>();
            }
            const int epi = parse_epilogue(epilogue, bp != nullptr);
            at::Tensor aux;
            if (epi == ops::EPI_BIAS_GELU || epi == ops::EPI_GELU) aux = at::empty({rows, N}, w.options());
            t.ag_gemm(*x_sym, static_cast<size_t>(x_off), static_cast<int>(rows_local), static_cast<int>(K), bf(w),
                      static_cast<int>(w.stride(0)), w_kn, static_cast<int>(N), bf(y), bf(gathered), bp, epi,
                      aux.defined() ? bf(aux) : nullptr, stream_of(w));
            ops::count_launch(1);
            return std::make_tuple(y, gathered, aux.defined() ? c10::optional<at::Tensor>(aux) : c10::nullopt);
          },
          py::arg("x_sym"), py::arg("x_offset"), py::arg("rows_local"), py::arg("w"), py::arg("w_kn") = false,
          py::arg("bias") = py::none(), py::arg("epilogue") = "none",
          "Returns (all_gather(x) @ w^T, gathered x, pre-activation or None).")
      .def(
          "gemm_rs",
          [](ops::TpGemm& t, const at::Tensor& x, const at::Tensor& w, bool w_kn) {
            need_cuda(x, "gemm_rs(x)");
            need_cuda(w, "gemm_rs(w)");
            MCCL_CHECK_TENSOR(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "gemm_rs: x must be 2-D bf16");
            MCCL_CHECK_TENSOR(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1, "gemm_rs: w must be 2-D bf16");
            c10::cuda::CUDAGuard guard(x.device());
            const int64_t K = w_kn ? w.size(0) : w.size(1), N = w_kn ? w.size(1) : w.size(0);
            MCCL_CHECK_TENSOR(x.size(1) == K && x.size(0) % t.world() == 0, "gemm_rs: shapes [world*rows, K] x [N, K] expected");
            const int64_t rows_local = x.size(0) / t.world();
            at::Tensor out = at::empty({rows_local, N}, x.options());
            t.gemm_rs(bf(x), static_cast<int>(x.stride(0)), static_cast<int>(rows_local), static_cast<int>(K), bf(w),
                      static_cast<int>(w.stride(0)), w_kn, static_cast<int>(N), bf(out), stream_of(x));
            ops::count_launch(1);
            return out;
          },
          py::arg("x"), py::arg("w"), py::arg("w_kn") = false, "Returns this rank's rows of reduce_scatter(x @ w^T).");

  m.def("colsum_bf16", [](const at::Tensor& x, const c10::optional<at::Tensor>& out_opt, bool accumulate) {
    need(x, at::kBFloat16, "colsum(x)");
    MCCL_CHECK_TENSOR(x.dim() == 2, "colsum: 2-D tensor expected");
    c10::cuda::CUDAGuard guard(x.device());
    const int rows = static_cast<int>(x.size(0)), dim = static_cast<int>(x.size(1));
    at::Tensor out = out_opt.has_value() ? *out_opt : at::empty({dim}, x.options().dtype(at::kFloat));
    need(out, at::kFloat, "colsum(out)");
    MCCL_CHECK_TENSOR(out.numel() == dim, "colsum: output must have one element per column");
    MCCL_CHECK_TENSOR(!accumulate || out_opt.has_value(), "colsum: accumulate needs an output to add into");
    at::Tensor scratch;
    if (!accumulate) scratch = at::empty({ops::colsum_slabs(rows) * dim}, x.options().dtype(at::kFloat));
    check_launch(ops::colsum_bf16(bf(x), out.data_ptr<float>(), accumulate ? nullptr : scratch.data_ptr<float>(), rows, dim,
                                  stream_of(x)),
                 "colsum");
    return out;
  }, py::arg("x"), py::arg("out") = py::none(), py::arg("accumulate") = false);
  m.def("transpose_bf16", [](const at::Tensor& x) {
    need(x, at::kBFloat16, "transpose(x)");
    MCCL_CHECK_TENSOR(x.dim() == 2, "transpose: 2-D tensor expected");
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = at::empty({x.size(1), x.size(0)}, x.options());
    check_launch(ops::transpose_bf16(bf(x), bf(y), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), stream_of(x)),
                 "transpose");
    return y;
  });
  m.def("transpose_bf16_out", [](const at::Tensor& x, at::Tensor y) {
    need(x, at::kBFloat16, "transpose(x)");
    need(y, at::kBFloat16, "transpose(out)");
    MCCL_CHECK_TENSOR(x.dim() == 2 && y.numel() == x.numel(), "transpose: bad shapes");
    c10::cuda::CUDAGuard guard(x.device());
    check_launch(ops::transpose_bf16(bf(x), bf(y), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), stream_of(x)),
                 "transpose");
  });
  m.def("cast_bf16", [](const at::Tensor& x, const c10::optional<at::Tensor>& out) {
    need(x, at::kFloat, "cast(x)");
    c10::cuda::CUDAGuard guard(x.device());
    at::Tensor y = out.has_value() ? *out : at::empty_like(x, x.options().dtype(at::kBFloat16));
    need(y, at::kBFloat16, "cast(out)");
    check_launch(ops::cast_f32_bf16(x.data_ptr<float>(), bf(y), x.numel(), stream_of(x)), "cast");
    return y;
  }, py::arg("x"), py::arg("out") = py::none());
  m.def("gelu_bwd", [](const at::Tensor& dy, const at::Tensor& z) {
    need(dy, at::kBFloat16, "gelu_bwd(dy)");
    need(z, at::kBFloat16, "gelu_bwd(z)");
    MCCL_CHECK_TENSOR(dy.numel() == z.numel(), "gelu_bwd: size mismatch");
    c10::cuda::CUDAGuard guard(dy.device());
    at::Tensor dz = at::empty_like(dy);
    check_launch(ops::gelu_bwd(bf(dy), bf(z), bf(dz), dy.numel(), stream_of(dy)), "gelu_bwd");
    return dz;
  });
  m.def("embed_fwd", [](const at::Tensor& ids, const at::Tensor& tok, const c10::optional<at::Tensor>& pos, int64_t seq) {
    need(ids, at::kLong, "embed_fwd(ids)");
    need(tok, at::kFloat, "embed_fwd(tok)");
    MCCL_CHECK_TENSOR(tok.dim() == 2 && tok.size(1) % 8 == 0, "embed_fwd: table [vocab, dim] with dim % 8 == 0 expected");
    const float* pp = nullptr;
    if (pos.has_value() && pos->defined()) {
      need(*pos, at::kFloat, "embed_fwd(pos)");
      MCCL_CHECK_TENSOR(pos->dim() == 2 && pos->size(1) == tok.size(1) && pos->size(0) >= seq, "embed_fwd: position table too small");
      pp = pos->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(ids.device());
    at::Tensor y = at::empty({ids.numel(), tok.size(1)}, tok.options().dtype(at::kBFloat16));
    check_launch(ops::embed_fwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                                tok.data_ptr<float>(), pp, bf(y), static_cast<int>(ids.numel()), static_cast<int>(seq),
                                static_cast<int>(tok.size(1)), static_cast<int>(tok.size(0)), stream_of(ids)),
                 "embed_fwd");
    return y;
  }, py::arg("ids"), py::arg("tok"), py::arg("pos") = py::none(), py::arg("seq") = 1);
  m.def("embed_bwd", [](const at::Tensor& ids, const at::Tensor& dy, const c10::optional<at::Tensor>& dtok,
                        const c10::optional<at::Tensor>& dpos, int64_t seq, double scale) {
    need(ids, at::kLong, "embed_bwd(ids)");
    need(dy, at::kBFloat16, "embed_bwd(dy)");
    MCCL_CHECK_TENSOR(dy.dim() == 2 && dy.size(1) % 8 == 0 && dy.size(0) == ids.numel(), "embed_bwd: dy must be [tokens, dim] with dim % 8 == 0");
    const int64_t dim = dy.size(1);
    float* tp = nullptr;
    int64_t vocab = 0;
    if (dtok.has_value() && dtok->defined()) {
      need(*dtok, at::kFloat, "embed_bwd(dtok)");
      MCCL_CHECK_TENSOR(dtok->dim() == 2 && dtok->size(1) == dim, "embed_bwd: dtok must be [vocab, dim]");
      tp = dtok->data_ptr<float>();
      vocab = dtok->size(0);
    }
    float* pp = nullptr;
    if (dpos.has_value() && dpos->defined()) {
      need(*dpos, at::kFloat, "embed_bwd(dpos)");
      MCCL_CHECK_TENSOR(dpos->dim() == 2 && dpos->size(1) == dim && dpos->size(0) >= seq, "embed_bwd: position table too small");
      pp = dpos->data_ptr<float>();
    }
    MCCL_CHECK_TENSOR(tp != nullptr || pp != nullptr, "embed_bwd: no gradient buffer given");
    c10::cuda::CUDAGuard guard(ids.device());
    check_launch(ops::embed_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), bf(dy), tp, pp,
                                static_cast<int>(ids.numel()), static_cast<int>(seq), static_cast<int>(dim),
                                static_cast<int>(vocab), stream_of(ids), static_cast<float>(scale)),
                 "embed_bwd");
  }, py::arg("ids"), py::arg("dy"), py::arg("dtok"), py::arg("dpos") = py::none(), py::arg("seq") = 1, py::arg("scale") = 1.0,
        "Adds scale * dy[t] into dtok[ids[t]] and dpos[t % seq] (either table may be None).");
}

}  // namespace mccl
