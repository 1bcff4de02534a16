// Tensor-parallel GEMMs fused with their collective (one kernel each):
//
//   ag_gemm   Y = all_gather(X) · W^T   column-parallel forward, row-parallel input gradient
//             copy CTAs of the same kernel push this rank's shard of X into the peers' staging (posted
//             bulk stores over NVLink, one peer per step so that every rank receives one chunk per
//             step) while the tensor cores already multiply the chunks that have landed, own chunk first.
//   gemm_rs   Y_r = reduce_scatter(X · W^T)   row-parallel forward, column-parallel input gradient
//             every rank writes its partial product row group by row group; pusher CTAs of the same
//             kernel send the rows other ranks own into the owner's staging while the tensor cores
//             work on the next group; whoever is free adds the world slots of its own rows in fp32.
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
  // max_chunk_elems: largest rows_local * K an ag_gemm call and rows_local * N a gemm_rs call will see.
  // ag_slots: length of the ring of gathered buffers (each world * max_chunk_elems bf16, symmetric); the
  // buffer an ag_gemm call returns is overwritten ag_slots calls later, so the ring must span the distance
  // between a forward call and the backward use of what it gathered (ag_valid tells).
  TpGemm(std::shared_ptr<DeviceComm> comm, size_t max_chunk_elems, int ag_slots = 4);
  ~TpGemm();
  TpGemm(const TpGemm&) = delete;
  TpGemm& operator=(const TpGemm&) = delete;

  int world() const { return comm_->world(); }
  int rank() const { return comm_->rank(); }

  // x: this rank's [rows_local, K] bf16 shard (dense, local).  w: [N, K] (w_kn = false) or [K, N]
  // (w_kn = true), row stride ldw.  y: [world * rows_local, N] bf16, row stride N.  rows_local must be a
  // multiple of 128.  Returns the ring slot that now holds all shards, [world * rows_local, K] dense, and
  // its generation number through *generation.
  __nv_bfloat16* ag_gemm(const __nv_bfloat16* x, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
                         __nv_bfloat16* y, const float* bias, int epilogue, __nv_bfloat16* aux, cudaStream_t stream,
                         uint64_t* generation);
  // True while the buffer returned by call `generation` has not been handed out again.
  bool ag_valid(uint64_t generation) const { return generation + static_cast<uint64_t>(ag_slots_) > ag_calls_; }
  int ag_slots() const { return ag_slots_; }
  // x: local [world * rows_local, K] bf16 (row stride ldx); out: [rows_local, N] bf16.
  void gemm_rs(const __nv_bfloat16* x, int ldx, int rows_local, int k, const __nv_bfloat16* w, int ldw, bool w_kn, int n,
               __nv_bfloat16* out, cudaStream_t stream);

  int status() const;        // 0 while healthy
  void check_status() const; // throws TimeoutError when a cross-GPU wait ran out

 private:
  std::shared_ptr<DeviceComm> comm_;
  std::shared_ptr<SymmAlloc> sig_, ag_stage_, rs_stage_;
  __nv_bfloat16* partial_ = nullptr;   // local partial product of gemm_rs, world * max_chunk_elems
  size_t max_chunk_elems_;
  int ag_slots_ = 4;
  uint64_t ag_calls_ = 0;
  uint32_t* words_ = nullptr;   // device counters, kFuseWord* in gemm_persistent.cuh
  int* status_host_ = nullptr;
  int* status_dev_ = nullptr;
  int sms_ = 148;
};

}  // namespace ops
}  // namespace mccl
