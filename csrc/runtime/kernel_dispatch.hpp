// Partitioning of a 1-D kernel grid over the nodes of a group, and the
// pipeline-stage bookkeeping of the distributed runtime.
//
// Parity: the reference's ShaderDispatch::data_parallel splits `total` threads
// evenly over the nodes and gives the remainder to the last node; a
// PipelineStage names the node that runs a stage and which of two buffers
// (double buffering) a micro-batch uses (csrc/runtime/ShaderDispatch.hpp:63-122).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace mccl {

struct NodeWork {
  int node = 0;
  uint64_t offset = 0;   // first element of this node's slice
  uint64_t count = 0;    // elements in the slice
};

struct KernelDispatch {
  // Even split; the last node also takes the remainder.
  static std::vector<NodeWork> data_parallel(uint64_t total, int num_nodes) {
    std::vector<NodeWork> out;
    if (num_nodes <= 0) return out;
    const uint64_t per = total / static_cast<uint64_t>(num_nodes);
    uint64_t off = 0;
    for (int n = 0; n < num_nodes; ++n) {
      NodeWork w;
      w.node = n;
      w.offset = off;
      w.count = (n == num_nodes - 1) ? total - off : per;
      off += w.count;
      out.push_back(w);
    }
    return out;
  }
};

struct PipelineStage {
  int stage = 0;
  int node = 0;
  std::string kernel;
  int buffer_slot(uint64_t micro_batch) const { return static_cast<int>(micro_batch & 1u); }
};

// Order in which (stage, micro-batch) pairs run for a fill / steady / drain schedule.
struct PipelineStep {
  uint64_t time = 0;
  int stage = 0;
  uint64_t micro_batch = 0;
};
inline std::vector<PipelineStep> pipeline_schedule(int stages, uint64_t micro_batches) {
  std::vector<PipelineStep> out;
  if (stages <= 0) return out;
  for (uint64_t t = 0; t < micro_batches + static_cast<uint64_t>(stages) - 1; ++t)
    for (int s = 0; s < stages; ++s)
      if (t >= static_cast<uint64_t>(s) && t - static_cast<uint64_t>(s) < micro_batches) out.push_back({t, s, t - static_cast<uint64_t>(s)});
  return out;
}

}  // namespace mccl
