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
  FUSE_REDUCE_SCATTER_D = 2,   // rows of D belong to different ranks; the owner pulls and adds the partial rows
};

constexpr int kFuseMaxRanks = 8;
constexpr int kFuseCopyCtas = 16;     // all-gather fusion: CTAs that move data (fixed: counters depend on it)
constexpr int kFuseReduceCtas = 16;   // reduce-scatter fusion: CTAs that only pull and add partial rows (default)
constexpr int kFuseMaxPhases = 4;     // reduce-scatter fusion: row groups of a chunk that complete one after another

// Everything the fused roles need.  Pointers into other GPUs' memory are peer
// mappings read with plain or bulk (never multicast) loads over NVLink.
struct FusedDev {
  int mode = FUSE_NONE;
  int world = 1;
  int rank = 0;
  int chunk_rows = 0;                         // rows per rank chunk, a multiple of 128
  int k_splits = 1;                           // split-K factor (set by the launcher)
  int copy_ctas = 0;                          // CTAs [0, copy_ctas) move data instead of computing tiles
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
  // GEMM → reduce-scatter.  Every rank writes its partial product [world * chunk_rows, N] (bf16, dense)
  // into its own buffer; rank o then reads rows [o * chunk_rows, (o + 1) * chunk_rows) of every buffer.
  void* rs_partial[2][kFuseMaxRanks] = {};    // [epoch parity][r]: rank r's partial product (mine is written, all are read)
  void* rs_out = nullptr;                     // [chunk_rows, N] bf16 result of the reduction
  int rs_phases = 1;                          // row groups per chunk (1, 2 or 4)
  uint32_t* phase_counters = nullptr;         // local [kFuseMaxPhases]: epilogue warps done with a phase (self-resetting)
  uint32_t* work_counter = nullptr;           // local: next piece of the reduction (zeroed before the launch)
};

// Signal-word layout (uint32 per entry) inside sig[r]:
//   [4*s, 4*s + 4)           reduce-scatter: rank s has written phase 0..3 of its partial product
//   [32 + 8*c, 32 + 8*c + 8) all-gather meeting flags of copy CTA c, indexed by source rank
constexpr int kFuseSigRs = 0;
constexpr int kFuseSigAg = 4 * kFuseMaxRanks;
constexpr int kFuseSigWords = kFuseSigAg + 8 * kFuseCopyCtas;

// max_ctas <= 0: one CTA per SM.
cudaError_t launch_gemm_persistent(const GemmArgs& a, const FusedDev& f, int max_ctas, cudaStream_t stream);
// The same product on CTA pairs (tcgen05.mma.cta_group::2; gemm_pair.cu): no fused roles, fewer operand bytes per SM.
cudaError_t launch_gemm_pair(const GemmArgs& a, cudaStream_t stream);
// ++*epoch and *zeroed = 0 (zeroed may be null), one thread; enqueue before a fused launch.
cudaError_t launch_bump_epoch(uint32_t* epoch, uint32_t* zeroed, cudaStream_t stream);

}  // namespace ops
}  // namespace mccl
