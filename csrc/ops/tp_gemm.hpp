// Tensor-parallel GEMMs fused with their collective (one kernel each):
//
//   ag_gemm   Y = all_gather(X) · W^T   column-parallel forward, row-parallel input gradient
//             CTAs of the same kernel pull the peers' shards of X over NVLink while the tensor
//             cores already multiply the chunks that have landed (own chunk first).
//   gemm_rs   Y_r = reduce_scatter(X · W^T)   row-parallel forward, column-parallel input gradient
//             every rank writes its partial product into a symmetric buffer, row group by row group;
//             reducer CTAs of the same kernel pull the groups of the rows they own from all ranks
//             (bulk loads over NVLink into shared memory), add them in fp32 and write the result
//             while the tensor cores work on the next group.
//
// The reference only offers `tensor_parallel_split` (a torch.chunk, mccl/distributed/sharding.py:54-69)
// and states that hand-wired column/row parallelism works over its collectives (README.md:76);
// these kernels are the NVLink-era form of that hand wiring.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <memory>

#include "../pg/device_comm.hpp"
#include "../symm/symm_mesh.hpp"

namespace mccl {
namespace ops {

class TpGemm {
 public:
  // max_rs_elems: largest chunk_rows * N a gemm_rs call will produce (sizes the staging slots).
  TpGemm(std::shared_ptr<DeviceComm> comm, size_t max_rs_elems);
  ~TpGemm();
  TpGemm(const TpGemm&) = delete;
  TpGemm& operator=(const TpGemm&) = delete;

  int world() const { return comm_->world(); }
  int rank() const { return comm_->rank(); }

  // x_sym: symmetric allocation holding this rank's [rows_local, K] bf16 shard at byte offset x_off
  // (same offset on every rank).  w: [N, K] (w_kn = false) or [K, N] (w_kn = true), row stride ldw.
  // gathered: local [world * rows_local, K] scratch that receives all shards (kept for the backward
  // pass).  y: [world * rows_local, N] bf16, row stride N.  rows_local must be a multiple of 128.
  void ag_gemm(const SymmAlloc& x_sym, size_t x_off, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
               __nv_bfloat16* y, __nv_bfloat16* gathered, const float* bias, int epilogue, __nv_bfloat16* aux,
               cudaStream_t stream);
  // x: local [world * rows_local, K] bf16 (row stride ldx); out: [rows_local, N] bf16.
  void gemm_rs(const __nv_bfloat16* x, int ldx, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
               __nv_bfloat16* out, cudaStream_t stream);

  int status() const;        // 0 while healthy
  void check_status() const; // throws TimeoutError when a cross-GPU wait ran out

 private:
  std::shared_ptr<DeviceComm> comm_;
  std::shared_ptr<SymmAlloc> sig_, stage_;
  size_t max_rs_elems_;
  uint32_t* words_ = nullptr;   // device: [0] ag epoch, [1] rs epoch, [8..16) chunk flags, [16..24) chunk counters, [24..28) phase counters, [28] piece counter
  int* status_host_ = nullptr;
  int* status_dev_ = nullptr;
  int sms_ = 148;
};

}  // namespace ops
}  // namespace mccl
