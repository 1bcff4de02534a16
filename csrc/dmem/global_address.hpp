// Global addresses and region descriptors of the distributed-memory (PGAS) layer.
//
// Parity: the reference addresses remote memory by {u16 node, u32 region,
// u64 offset} with a 14-byte wire form and a packed 64-bit key
// (node << 48 | region << 16), and describes a region by its global address,
// local pointer, length, RDMA keys and READABLE / WRITABLE / SHARED / PRIVATE
// flags (csrc/dmem/GlobalAddress.hpp:11-84).  The RDMA keys become a heap id
// and a generation number (a region lives inside a peer-mapped symmetric heap
// allocation).  The structs are usable from device code.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define MCCL_HD __host__ __device__
#else
#define MCCL_HD
#endif

namespace mccl {

constexpr int kDmemMaxNodes = 8;
constexpr int kDmemMaxRegionsPerNode = 256;

struct GlobalAddress {
  uint16_t node_id = 0;
  uint32_t region_id = 0;
  uint64_t offset = 0;

  MCCL_HD GlobalAddress() {}
  MCCL_HD GlobalAddress(uint16_t n, uint32_t r, uint64_t o) : node_id(n), region_id(r), offset(o) {}
  MCCL_HD uint64_t pack() const { return (static_cast<uint64_t>(node_id) << 48) | (static_cast<uint64_t>(region_id) << 16); }
  MCCL_HD GlobalAddress operator+(uint64_t d) const { return GlobalAddress(node_id, region_id, offset + d); }
  MCCL_HD bool operator==(const GlobalAddress& o) const { return node_id == o.node_id && region_id == o.region_id && offset == o.offset; }

  static constexpr int kWireBytes = 14;
  void to_wire(uint8_t* p) const {
    std::memcpy(p, &node_id, 2);
    std::memcpy(p + 2, &region_id, 4);
    std::memcpy(p + 6, &offset, 8);
  }
  static GlobalAddress from_wire(const uint8_t* p) {
    GlobalAddress g;
    std::memcpy(&g.node_id, p, 2);
    std::memcpy(&g.region_id, p + 2, 4);
    std::memcpy(&g.offset, p + 6, 8);
    return g;
  }
};

enum RegionFlags : uint32_t {
  REGION_READABLE = 1u << 0,
  REGION_WRITABLE = 1u << 1,
  REGION_SHARED = 1u << 2,
  REGION_PRIVATE = 1u << 3,
  REGION_DEVICE = 1u << 4,   // lives in GPU memory (symmetric heap); otherwise host memory
  REGION_HOST_HEAP = 1u << 5,  // carved from a shared-memory host heap (a heap id that does not mean GPU memory)
};

struct MemoryRegion {
  GlobalAddress gaddr;       // offset 0 of the region
  void* local_addr = nullptr;
  uint64_t length = 0;
  uint32_t heap_id = 0;      // symmetric allocation the region was carved from (0 = host memory)
  uint32_t generation = 0;   // bumped when a region id is reused
  uint32_t flags = REGION_READABLE | REGION_WRITABLE | REGION_SHARED;
};

// Result of resolving a global address on this node.
struct AddrResolution {
  bool ok = false;
  bool local = false;
  void* ptr = nullptr;        // directly usable pointer (local memory, or the peer mapping of a symmetric heap)
  uint64_t remote_addr = 0;   // address in the owner's address space
  uint64_t max_len = 0;       // bytes available from the offset to the end of the region
};

}  // namespace mccl
