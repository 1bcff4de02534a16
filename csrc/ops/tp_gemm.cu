#include "tp_gemm.hpp"

#include <cstdlib>
#include <cstring>

#include "../core/errors.hpp"
#include "../symm/cu_driver.hpp"
#include "gemm_persistent.cuh"

namespace mccl {
namespace ops {

TpGemm::TpGemm(std::shared_ptr<DeviceComm> comm, size_t max_chunk_elems, int ag_slots)
    : comm_(std::move(comm)), max_chunk_elems_(max_chunk_elems), ag_slots_(ag_slots < 2 ? 2 : ag_slots) {
  MCCL_CHECK(comm_->nlocal() == 1 && comm_->world() >= 2 && comm_->world() <= kFuseMaxRanks,
             "tensor-parallel GEMMs need one process per GPU and 2..8 ranks");
  MCCL_CUDA_CHECK(cudaSetDevice(comm_->device()));
  const size_t stage_bytes = 2 * static_cast<size_t>(comm_->world()) * max_chunk_elems * sizeof(__nv_bfloat16);
  sig_ = comm_->symm_alloc(static_cast<size_t>(kFuseSigWords) * sizeof(uint32_t));
  ag_stage_ = comm_->symm_alloc(static_cast<size_t>(ag_slots_) * comm_->world() * max_chunk_elems * sizeof(__nv_bfloat16));
  rs_stage_ = comm_->symm_alloc(stage_bytes);
  MCCL_CUDA_CHECK(cudaMalloc(&partial_, static_cast<size_t>(comm_->world()) * max_chunk_elems * sizeof(__nv_bfloat16)));
  MCCL_CUDA_CHECK(cudaMalloc(&words_, kFuseWords * sizeof(uint32_t)));
  MCCL_CUDA_CHECK(cudaMemset(words_, 0, kFuseWords * sizeof(uint32_t)));
  MCCL_CUDA_CHECK(cudaHostAlloc(&status_host_, sizeof(int), cudaHostAllocMapped));
  *status_host_ = 0;
  MCCL_CUDA_CHECK(cudaHostGetDevicePointer(&status_dev_, status_host_, 0));
  cudaDeviceGetAttribute(&sms_, cudaDevAttrMultiProcessorCount, comm_->device());
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  comm_->mesh().store_barrier("tpgemm-ready-" + std::to_string(sig_->id));
}

TpGemm::~TpGemm() {
  if (partial_) cudaFree(partial_);
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
// Data-moving CTAs of a fusion: enough that sending the remote bytes takes no longer than the tiles on the
// remaining SMs or than the link allows.  One SM sustains roughly `kPushPerSm` bytes/s of bulk stores to peers.
constexpr double kPushPerSm = 40e9, kLink = 700e9, kTilePeak = 1.38e15;
int choose_copy_ctas(double remote_bytes, double flops, int sms) {
  static const int forced = env_int("MCCL_TP_COPY_CTAS", 0, 0, kFuseMaxCopyCtas);
  if (forced > 0) return forced;
  int best = 8;
  double best_t = 1e30;
  for (int c = 8; c <= kFuseMaxCopyCtas && c < sms - 8; c += 8) {
    const double t_comm = remote_bytes / (kPushPerSm * c), t_gemm = flops / (kTilePeak * (sms - c) / sms);
    double t = t_comm > t_gemm ? t_comm : t_gemm;
    if (t < remote_bytes / kLink) t = remote_bytes / kLink;
    if (t < best_t * 0.97) {   // prefer fewer copy CTAs unless more of them help noticeably
      best_t = t;
      best = c;
    }
  }
  return best;
}
void fill_common(FusedDev& f, DeviceComm& comm, const SymmAlloc& sig, int* status_dev) {
  f.world = comm.world();
  f.rank = comm.rank();
  f.timeout_ns = 10ull * 1000 * 1000 * 1000;
  f.status = status_dev;
  for (int r = 0; r < f.world; ++r) f.sig[r] = static_cast<uint32_t*>(sig.ptrs[r]);
}
}  // namespace

__nv_bfloat16* TpGemm::ag_gemm(const __nv_bfloat16* x, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
                               __nv_bfloat16* y, const float* bias, int epilogue, __nv_bfloat16* aux, cudaStream_t stream,
                               uint64_t* generation) {
  MCCL_CHECK(rows_local > 0 && rows_local % 128 == 0, "ag_gemm: rows per rank (" << rows_local << ") must be a multiple of 128");
  MCCL_CHECK(k % 64 == 0 && n % 8 == 0, "ag_gemm: K must be a multiple of 64 and N of 8");
  const size_t chunk_elems = static_cast<size_t>(rows_local) * k;
  MCCL_CHECK(chunk_elems <= max_chunk_elems_, "ag_gemm: shard of " << chunk_elems << " elements exceeds the staging ("
                                                                   << max_chunk_elems_ << "); build TpGemm with a larger bound");
  MCCL_CHECK(reinterpret_cast<uintptr_t>(x) % 16 == 0, "ag_gemm: the shard must be 16-byte aligned");
  FusedDev f;
  fill_common(f, *comm_, *sig_, status_dev_);
  f.mode = FUSE_ALLGATHER_A;
  f.chunk_rows = rows_local;
  f.chunk_bytes = chunk_elems * sizeof(__nv_bfloat16);
  f.copy_ctas = choose_copy_ctas(static_cast<double>(f.world - 1) * f.chunk_bytes, 2.0 * rows_local * f.world * n * k, sms_);
  f.epoch_ptr = words_ + kFuseWordAgEpoch;
  f.step_counters = words_ + kFuseWordStep;
  f.a_own = x;
  const size_t slot_elems = static_cast<size_t>(f.world) * max_chunk_elems_;
  const size_t slot = static_cast<size_t>(ag_calls_ % static_cast<uint64_t>(ag_slots_));
  for (int p = 0; p < f.world; ++p) f.a_stage[p] = static_cast<__nv_bfloat16*>(ag_stage_->ptrs[p]) + slot * slot_elems;
  GemmArgs a;
  a.a = x;   // the own shard; the other chunks come from the staging
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
  BumpArgs b;
  b.epoch = words_ + kFuseWordAgEpoch;
  MCCL_CUDA_CHECK(launch_bump_epoch(b, stream));
  cudaError_t rc = launch_gemm_persistent(a, f, sms_, stream);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "ag_gemm launch failed: " << cudaGetErrorString(rc));
  if (generation) *generation = ag_calls_;
  ++ag_calls_;
  return static_cast<__nv_bfloat16*>(f.a_stage[f.rank]);
}

void TpGemm::gemm_rs(const __nv_bfloat16* x, int ldx, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
                     __nv_bfloat16* out, cudaStream_t stream) {
  MCCL_CHECK(rows_local > 0 && rows_local % 128 == 0, "gemm_rs: rows per rank (" << rows_local << ") must be a multiple of 128");
  MCCL_CHECK(k % 64 == 0 && n % 8 == 0, "gemm_rs: K must be a multiple of 64 and N of 8");
  const size_t chunk_elems = static_cast<size_t>(rows_local) * n;
  MCCL_CHECK(chunk_elems <= max_chunk_elems_, "gemm_rs: chunk of " << chunk_elems << " elements exceeds the staging ("
                                                                   << max_chunk_elems_ << "); build TpGemm with a larger bound");
  FusedDev f;
  fill_common(f, *comm_, *sig_, status_dev_);
  f.mode = FUSE_REDUCE_SCATTER_D;
  f.chunk_rows = rows_local;
  f.chunk_bytes = chunk_elems * sizeof(__nv_bfloat16);
  static const int max_phases = env_int("MCCL_TP_PHASES", kFuseMaxPhases, 1, kFuseMaxPhases);
  f.copy_ctas = choose_copy_ctas(static_cast<double>(f.world - 1) * f.chunk_bytes, 2.0 * rows_local * f.world * n * k, sms_);
  f.epoch_ptr = words_ + kFuseWordRsEpoch;
  f.phase_counters = words_ + kFuseWordPhase;
  f.push_counters = words_ + kFuseWordPush;
  f.work_counter = words_ + kFuseWordWork;
  f.rs_partial = partial_;
  f.rs_out = out;
  const int chunk_mt = rows_local / 128;
  f.rs_phases = (max_phases >= 4 && chunk_mt % 4 == 0) ? 4 : ((max_phases >= 2 && chunk_mt % 2 == 0) ? 2 : 1);
  const size_t parity_elems = static_cast<size_t>(f.world) * max_chunk_elems_;
  for (int par = 0; par < 2; ++par)
    for (int p = 0; p < f.world; ++p) f.rs_stage[par][p] = static_cast<__nv_bfloat16*>(rs_stage_->ptrs[p]) + par * parity_elems;
  GemmArgs a;
  a.a = x;
  a.b = w;
  a.d = partial_;
  a.m = rows_local * f.world;
  a.n = n;
  a.k = k;
  a.lda = ldx;
  a.ldb = ldw;
  a.ldd = n;
  a.b_mn_major = w_kn;
  BumpArgs b;
  b.epoch = words_ + kFuseWordRsEpoch;
  b.zeroed = words_ + kFuseWordWork;
  MCCL_CUDA_CHECK(launch_bump_epoch(b, stream));
  cudaError_t rc = launch_gemm_persistent(a, f, sms_, stream);
  MCCL_CHECK_T(rc == cudaSuccess, CudaError, "gemm_rs launch failed: " << cudaGetErrorString(rc));
}

}  // namespace ops
}  // namespace mccl
