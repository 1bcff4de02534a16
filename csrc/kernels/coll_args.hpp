// Launch arguments and arena layouts shared by the host launcher and the
// collective kernels.  Every layout is a pure function of (world, numel, wire
// element size), so all ranks agree on it without exchanging anything.
#pragma once

#include <cstddef>
#include <cstdint>

namespace mccl {
namespace dev {

constexpr int kArgRanks = 8;

// Reduction operators understood by the kernels.
enum Op : int { OP_SUM = 0, OP_AVG = 1, OP_MIN = 2, OP_MAX = 3, OP_PROD = 4, OP_BAND = 5, OP_BOR = 6, OP_BXOR = 7 };

struct CollArgs {
  const void* in[kArgRanks];   // per virtual rank (index 0 outside 1-GPU emulation)
  void* out[kArgRanks];
  long long numel;             // elements of the whole message
  long long per;               // elements per chunk, a multiple of 16
  long long stride;            // reduce-scatter: elements between chunks in the input;
                               // allgather: bytes between ranks' blocks in the output
  int op;                      // dev::Op
  int root;
  float inv_world;
  int reserved;
};

// All-to-all: byte offsets / lengths per peer, per virtual rank.
struct A2AArgs {
  const void* in[kArgRanks];
  void* out[kArgRanks];
  unsigned long long in_off[kArgRanks][kArgRanks];   // [virtual rank][peer]
  unsigned long long in_len[kArgRanks][kArgRanks];
  unsigned long long out_off[kArgRanks][kArgRanks];
  unsigned long long out_len[kArgRanks][kArgRanks];
  unsigned long long slot_bytes;                     // arena bytes reserved per destination
};

// Point-to-point transfer: one entry per virtual rank of the launch.
struct P2PArgs {
  void* buf[kArgRanks];              // send source or receive destination
  int peer[kArgRanks];               // -1: this virtual rank takes no part
  int is_send[kArgRanks];
  unsigned long long nbytes;
};

// Chunk length in elements: ceil(numel / world) rounded up to 16 elements so
// that every chunk starts on a 16-byte boundary for every element size.
inline long long chunk_elems(long long numel, int world) {
  long long per = (numel + world - 1) / world;
  return (per + 15) / 16 * 16;
}

// Arena bytes one launch of each schedule needs (per half).
inline size_t twoshot_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>(chunk_elems(numel, world)) * wire_es * static_cast<size_t>(world + 1);
}
inline size_t twoshot_push_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>(chunk_elems(numel, world)) * wire_es * static_cast<size_t>(2 * world);
}
inline size_t oneshot_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>((numel + 15) / 16 * 16) * wire_es * static_cast<size_t>(world);
}
inline size_t ring_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>(chunk_elems(numel, world)) * wire_es * static_cast<size_t>(2 * (world - 1));
}
inline int tree_rounds(int world) {
  int r = 0;
  while ((1 << r) < world) ++r;
  return r;
}
inline size_t tree_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>((numel + 15) / 16 * 16) * wire_es * static_cast<size_t>(tree_rounds(world) + 1);
}
inline size_t nvls_bytes(long long numel, int world, size_t wire_es) {
  return static_cast<size_t>(chunk_elems(numel, world)) * wire_es * static_cast<size_t>(world) * 2;
}

}  // namespace dev
}  // namespace mccl
