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
  FUSE_ALLGATHER_A = 1,        // rows of A arrive chunk by chunk (one chunk per rank)
  FUSE_REDUCE_SCATTER_D = 2,   // rows of D belong to different ranks, chunk by chunk
};

struct FusedDev {
  int mode = FUSE_NONE;
  int world = 1;
  int rank = 0;
  int chunk_rows = 0;                    // rows per rank chunk, a multiple of 128
  const uint32_t* chunk_flags = nullptr; // all-gather: chunk c has landed when chunk_flags[c] >= epoch
  uint32_t epoch = 0;
  void* d_owner[8] = {};
  int k_splits = 1;                      // split-K factor (set by the launcher)                 // reduce-scatter: where this rank's partial rows of chunk c go
};

// max_ctas <= 0: one CTA per SM.  The fusions pass a smaller number to leave
// SMs to the CTAs that move data.
cudaError_t launch_gemm_persistent(const GemmArgs& a, const FusedDev& f, int max_ctas, cudaStream_t stream);

}  // namespace ops
}  // namespace mccl
