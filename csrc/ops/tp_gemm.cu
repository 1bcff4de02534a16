#include "tp_gemm.hpp"

#include <cstdlib>
#include <cstring>

#include "../core/errors.hpp"
#include "../symm/cu_driver.hpp"
#include "gemm_persistent.cuh"

namespace mccl {
namespace ops {

TpGemm::TpGemm(std::shared_ptr<DeviceComm> comm, size_t max_rs_elems) : comm_(std::move(comm)), max_rs_elems_(max_rs_elems) {
  MCCL_CHECK(comm_->nlocal() == 1 && comm_->world() >= 2 && comm_->world() <= kFuseMaxRanks,
             "tensor-parallel GEMMs need one process per GPU and 2..8 ranks");
  MCCL_CUDA_CHECK(cudaSetDevice(comm_->device()));
  sig_ = comm_->symm_alloc(static_cast<size_t>(kFuseSigWords) * sizeof(uint32_t));
  stage_ = comm_->symm_alloc(2 * static_cast<size_t>(comm_->world()) * max_rs_elems * sizeof(__nv_bfloat16));
  MCCL_CUDA_CHECK(cudaMalloc(&words_, 32 * sizeof(uint32_t)));
  MCCL_CUDA_CHECK(cudaMemset(words_, 0, 32 * sizeof(uint32_t)));
  MCCL_CUDA_CHECK(cudaHostAlloc(&status_host_, sizeof(int), cudaHostAllocMapped));
  *status_host_ = 0;
  MCCL_CUDA_CHECK(cudaHostGetDevicePointer(&status_dev_, status_host_, 0));
  cudaDeviceGetAttribute(&sms_, cudaDevAttrMultiProcessorCount, comm_->device());
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  comm_->mesh().store_barrier("tpgemm-ready-" + std::to_string(sig_->id));
}

TpGemm::~TpGemm() {
  if (words_) cudaFree(words_);
  if (status_host_) cudaFreeHost(status_host_);
}

int TpGemm::status() const { return *reinterpret_cast<volatile int*>(status_host_); }

void TpGemm::check_status() const {
  const int s = status();
  MCCL_CHECK_T(s == 0, TimeoutError,
               "tensor-parallel GEMM: rank " << comm_->rank() << " waited too long for rank " << (s & 0xff) << " in the "
                                             << ((s & 0x200) ? "reduce-scatter" : "all-gather") << " fusion");
}

namespace {
int env_int(const char* name, int def, int lo, int hi) {
  const char* v = std::getenv(name);
  if (!v || !*v) return def;
  const int x = std::atoi(v);
  return x < lo ? lo : (x > hi ? hi : x);
}
void fill_common(FusedDev& f, DeviceComm& comm, const SymmAlloc& sig, int* status_dev) {
  f.world = comm.world();
  f.rank = comm.rank();
  f.timeout_ns = static_cast<unsigned long long>(comm.device_timeout_ms()) * 1000000ull;   // same bound as the collectives
  f.status = status_dev;
  for (int r = 0; r < f.world; ++r) f.sig[r] = static_cast<uint32_t*>(sig.ptrs[r]);
}
}  // namespace

void TpGemm::ag_gemm(const SymmAlloc& x_sym, size_t x_off, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
                     __nv_bfloat16* y, __nv_bfloat16* gathered, const float* bias, int epilogue, __nv_bfloat16* aux,
                     cudaStream_t stream) {
  MCCL_CHECK(rows_local > 0 && rows_local % 128 == 0, "ag_gemm: rows per rank (" << rows_local << ") must be a multiple of 128");
  MCCL_CHECK(k % 64 == 0 && n % 8 == 0, "ag_gemm: K must be a multiple of 64 and N of 8");
  const size_t chunk_bytes = static_cast<size_t>(rows_local) * k * sizeof(__nv_bfloat16);
  MCCL_CHECK(x_off % 16 == 0 && x_off + chunk_bytes <= x_sym.bytes, "ag_gemm: shard does not fit its symmetric allocation");
  FusedDev f;
  fill_common(f, *comm_, *sig_, status_dev_);
  f.mode = FUSE_ALLGATHER_A;
  f.chunk_rows = rows_local;
  f.copy_ctas = kFuseCopyCtas;
  f.epoch_ptr = words_ + 0;
  for (int r = 0; r < f.world; ++r) f.a_peer[r] = static_cast<const char*>(x_sym.ptrs[r]) + x_off;
  f.a_gathered = gathered;
  f.chunk_bytes = chunk_bytes;
  f.chunk_flags = words_ + 8;
  f.chunk_counters = words_ + 16;
  GemmArgs a;
  a.a = gathered;
  a.b = w;
  a.d = y;
  a.aux = aux;
  a.bias = bias;
  a.m = rows_local * f.world;
  a.n = n;
  a.k = k;
  a.lda = k;
  a.ldb = ldw;
  a.ldd = n;
  a.b_mn_major = w_kn;
  a.epilogue = epilogue;
  MCCL_CUDA_CHECK(launch_bump_epoch(words_ + 0, nullptr, stream));
  cudaError_t rc = launch_gemm_persistent(a, f, sms_, stream);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "ag_gemm launch failed: " << cudaGetErrorString(rc));
}

void TpGemm::gemm_rs(const __nv_bfloat16* x, int ldx, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
                     __nv_bfloat16* out, cudaStream_t stream) {
  MCCL_CHECK(rows_local > 0 && rows_local % 128 == 0, "gemm_rs: rows per rank (" << rows_local << ") must be a multiple of 128");
  MCCL_CHECK(k % 64 == 0 && n % 8 == 0, "gemm_rs: K must be a multiple of 64 and N of 8");
  const size_t slot_elems = static_cast<size_t>(rows_local) * n;
  MCCL_CHECK(slot_elems <= max_rs_elems_, "gemm_rs: chunk of " << slot_elems << " elements exceeds the staging slots ("
                                                               << max_rs_elems_ << "); build TpGemm with a larger bound");
  FusedDev f;
  fill_common(f, *comm_, *sig_, status_dev_);
  f.mode = FUSE_REDUCE_SCATTER_D;
  f.chunk_rows = rows_local;
  static const int reduce_ctas = env_int("MCCL_TP_REDUCE_CTAS", kFuseReduceCtas, 1, 64);
  static const int max_phases = env_int("MCCL_TP_PHASES", kFuseMaxPhases, 1, kFuseMaxPhases);
  f.copy_ctas = reduce_ctas;
  f.epoch_ptr = words_ + 1;
  f.phase_counters = words_ + 24;
  f.work_counter = words_ + 28;
  f.rs_out = out;
  const int chunk_mt = rows_local / 128;
  f.rs_phases = (max_phases >= 4 && chunk_mt % 4 == 0) ? 4 : ((max_phases >= 2 && chunk_mt % 2 == 0) ? 2 : 1);
  // every rank's partial product [world * rows_local, N] lives in its half (by call parity) of the symmetric staging
  const size_t parity_elems = static_cast<size_t>(f.world) * max_rs_elems_;
  for (int par = 0; par < 2; ++par)
    for (int r = 0; r < f.world; ++r) f.rs_partial[par][r] = static_cast<__nv_bfloat16*>(stage_->ptrs[r]) + par * parity_elems;
  GemmArgs a;
  a.a = x;
  a.b = w;
  a.d = out;   // replaced inside the kernel by this rank's partial-product buffer
  a.m = rows_local * f.world;
  a.n = n;
  a.k = k;
  a.lda = ldx;
  a.ldb = ldw;
  a.ldd = n;
  a.b_mn_major = w_kn;
  MCCL_CUDA_CHECK(launch_bump_epoch(words_ + 1, words_ + 28, stream));
  cudaError_t rc = launch_gemm_persistent(a, f, sms_, stream);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "gemm_rs launch failed: " << cudaGetErrorString(rc));
}

}  // namespace ops
}  // namespace mccl
