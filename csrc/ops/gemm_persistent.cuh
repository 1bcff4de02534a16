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
constexpr int kFuseCopyCtas = 16;     // all-gather fusion: CTAs that move data (default; at most kFuseMaxCopyCtas)
constexpr int kFuseMaxCopyCtas = 96;
constexpr int kFuseReduceCtas = 16;   // reduce-scatter fusion: CTAs that only pull and add partial rows (default)
constexpr int kFuseMaxPhases = 4;     // reduce-scatter fusion: row groups of a chunk that complete one after another

// Everything the fused roles need.  Data crosses NVLink as posted writes: a rank pushes what it
// produced into the consumer's symmetric staging (bulk stores from shared memory, never a multicast
// load), then raises a flag there.  Pointers into other GPUs' memory are peer mappings.
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
  unsigned long long chunk_bytes = 0;         // bytes of one rank's chunk (A shard, or D rows of one owner)
  // all-gather → GEMM.  Rank r pushes its shard into chunk r of every peer's gathered buffer (a slot of the
  // symmetric ring), one peer after the other ((r+1), (r+2), ...), so every rank receives one chunk per
  // step; the tiles read the own shard in place and the other chunks from the slot, in arrival order.
  const void* a_own = nullptr;                // this rank's [chunk_rows, K] shard (local)
  void* a_stage[kFuseMaxRanks] = {};          // [p]: rank p's slot for this call, [world * chunk_rows, K]
  uint32_t* step_counters = nullptr;          // local [world]: copy CTAs done with push step k (self-resetting)
  // GEMM → reduce-scatter.  Every rank writes its partial product [world * chunk_rows, N] (bf16, dense) to
  // local memory, row group by row group; pusher CTAs send the rows other ranks own into slot `rank` of the
  // owner's staging; the owner adds the world slots (its own rows straight from its partial product).
  void* rs_partial = nullptr;                 // local partial product
  void* rs_stage[2][kFuseMaxRanks] = {};      // [epoch parity][p]: rank p's staging, world slots of chunk_rows x N
  void* rs_out = nullptr;                     // [chunk_rows, N] bf16 result of the reduction
  int rs_phases = 1;                          // row groups per chunk (1, 2 or 4)
  uint32_t* phase_counters = nullptr;         // local [kFuseMaxPhases]: epilogue warps done with a phase (self-resetting)
  uint32_t* push_counters = nullptr;          // local [world * kFuseMaxPhases]: pushers done with (owner, phase) (self-resetting)
  uint32_t* work_counter = nullptr;           // local: next piece of the reduction (zeroed before the launch)
};

// Signal-word layout (uint32 per entry) inside sig[r]:
//   [4*s + ph]  reduce-scatter: rank s's rows of phase ph for rank r are in r's staging (s == r: r's own
//               partial product has reached phase ph)
//   [32 + s]    all-gather: rank s's shard is in r's staging
constexpr int kFuseSigRs = 0;
constexpr int kFuseSigAg = 4 * kFuseMaxRanks;
constexpr int kFuseSigWords = 64;
// Local counter words of one TpGemm object.
constexpr int kFuseWordAgEpoch = 0, kFuseWordRsEpoch = 1, kFuseWordStep = 8, kFuseWordPhase = 24, kFuseWordWork = 28,
              kFuseWordPush = 32, kFuseWords = 64;

struct BumpArgs {
  uint32_t* epoch = nullptr;                   // device word to increment
  uint32_t* zeroed = nullptr;                  // device word to clear (may be null)
};

// max_ctas <= 0: one CTA per SM.
cudaError_t launch_gemm_persistent(const GemmArgs& a, const FusedDev& f, int max_ctas, cudaStream_t stream);
// One thread: ++*epoch, clear, announce; enqueue before a fused launch.
cudaError_t launch_bump_epoch(const BumpArgs& b, cudaStream_t stream);

}  // namespace ops
}  // namespace mccl
