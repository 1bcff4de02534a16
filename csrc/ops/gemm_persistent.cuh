// Interface of the persistent GEMM kernel, including the hooks the
// tensor-parallel fusions use.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "ops.hpp"

namespace mccl {
namespace ops {

enum FuseMode : int {
  FUSE_NONE = 0,
  FUSE_ALLGATHER_A = 1,        // rows of A arrive chunk by chunk (one chunk per rank) while tiles are computed
  FUSE_REDUCE_SCATTER_D = 2,   // rows of D belong to different ranks; partial tiles go to the owner, who reduces
};

constexpr int kFuseMaxRanks = 8;
constexpr int kFuseCopyCtas = 16;   // CTAs of the all-gather fusion that move data (fixed: counters depend on it)

// Everything the fused roles need.  Pointers into other GPUs' memory are peer
// mappings (plain loads / stores over NVLink); no TMA descriptor ever covers them.
struct FusedDev {
  int mode = FUSE_NONE;
  int world = 1;
  int rank = 0;
  int chunk_rows = 0;                         // rows per rank chunk, a multiple of 128
  int k_splits = 1;                           // split-K factor (set by the launcher)
  int copy_ctas = 0;                          // all-gather: CTAs [0, copy_ctas) pull the peers' shards
  const uint32_t* epoch_ptr = nullptr;        // device word: number of this fused call (bumped before the launch)
  unsigned long long timeout_ns = 0;          // bound of every cross-GPU wait
  int* status = nullptr;                      // written (non-zero) when such a wait runs out
  uint32_t* sig[kFuseMaxRanks] = {};          // every rank's signal words for these fusions (peer-mapped)
  // all-gather → GEMM
  const void* a_peer[kFuseMaxRanks] = {};     // rank r's shard of A
  void* a_gathered = nullptr;                 // local [world * chunk_rows, K] buffer the tiles are loaded from
  unsigned long long chunk_bytes = 0;
  uint32_t* chunk_flags = nullptr;            // local [world]: chunk c has landed when chunk_flags[c] >= epoch
  uint32_t* chunk_counters = nullptr;         // local [world]: copy CTAs that finished chunk c (cumulative)
  // GEMM → reduce-scatter
  void* d_owner[2][kFuseMaxRanks] = {};       // [epoch parity][owner]: where this rank's partial rows of that chunk go
  const void* rs_slots[2] = {};               // [epoch parity]: my staging, world slots of chunk_rows x N bf16
  void* rs_out = nullptr;                     // [chunk_rows, N] bf16 result of the reduction
  uint32_t* done_counter = nullptr;           // local: GEMM CTAs that finished their tiles (cumulative)
  int rs_gemm_ctas = 0;                       // fixed number of GEMM CTAs of the reduce-scatter fusion
};

// Signal-word layout (uint32 per entry) inside sig[r]:
//   [0, 8)                 reduce-scatter "pushes done" flags, indexed by source rank
//   [8 + 8*c, 8 + 8*c + 8) all-gather meeting flags of copy CTA c, indexed by source rank
constexpr int kFuseSigWords = 8 + 8 * kFuseCopyCtas;

// max_ctas <= 0: one CTA per SM.
cudaError_t launch_gemm_persistent(const GemmArgs& a, const FusedDev& f, int max_ctas, cudaStream_t stream);
// ++*epoch (one thread); enqueue before a fused launch.
cudaError_t launch_bump_epoch(uint32_t* epoch, cudaStream_t stream);

}  // namespace ops
}  // namespace mccl
