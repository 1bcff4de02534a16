// Distributed memory manager: one-sided put / get / put-with-immediate over
// memory that every node can address directly.
//
// Parity: the reference's DistributedMemoryManager registers regions with the
// RDMA device and the catalog, resolves global addresses (local → pointer,
// remote → address + key, clamped to the region), moves data with chunked RDMA
// writes / reads through a staging buffer, offers put_with_imm, fence,
// poll_completion (5 s limit), drain_pending and byte / op / error counters
// (csrc/dmem/DistributedMemoryManager.hpp:40-145, .cpp:104-527).  On one
// NVSwitch box no NIC is involved: a peer's region is mapped into this
// process (symmetric heap), so put and get are copies to or from the mapped
// address - cudaMemcpyAsync on a stream for device memory, memcpy for host
// memory - and the 1 MB chunking disappears.  A completion id stands for a
// CUDA event (device) or is complete at once (host).
//
// The fabric decides how peers are reached:
//   LocalFabric  several nodes inside one process (tests, single-process tools)
//   SymmFabric   one process per GPU; regions live in DeviceComm's symmetric heap
#pragma once

#include <atomic>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "global_address.hpp"
#include "memory_catalog.hpp"

namespace mccl {

class DistributedMemoryManager;

struct ImmRecord {
  uint16_t src_node = 0;
  uint32_t region_id = 0;
  uint64_t offset = 0;
  uint64_t length = 0;
  uint32_t imm = 0;
};

class DmemFabric {
 public:
  virtual ~DmemFabric() = default;
  virtual int num_nodes() const = 0;
  // Makes a region of `node` known to every node / forgets it.
  virtual void publish(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) = 0;
  virtual void retract(uint16_t node, uint32_t region) = 0;
  // Entry of a remote region (false when unknown).
  virtual bool fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) = 0;
  // Pointer through which `me` can reach `remote_addr` of `node` (nullptr when it cannot).
  virtual void* map(uint16_t me, uint16_t node, const RegionDirectoryEntry& e, uint64_t remote_addr) = 0;
  virtual void deliver_imm(uint16_t node, const ImmRecord& r) = 0;
  // Stream-ordered delivery: the immediate becomes visible after everything `stream` did before.
  // Returns false when the fabric cannot do that (the caller then waits for the data on the host
  // and uses deliver_imm).
  virtual bool deliver_imm_stream(uint16_t, const ImmRecord&, void* /*stream*/) { return false; }
};

struct DmemStats {
  uint64_t total_put_bytes = 0, total_get_bytes = 0, total_put_ops = 0, total_get_ops = 0, total_errors = 0;
  uint64_t regions = 0, pending = 0;
};

class DistributedMemoryManager {
 public:
  DistributedMemoryManager(uint16_t node_id, std::shared_ptr<DmemFabric> fabric);
  ~DistributedMemoryManager();

  uint16_t node_id() const { return node_id_; }
  int num_nodes() const { return fabric_->num_nodes(); }

  // Registers [ptr, ptr + nbytes) and returns the region id (> 0).  heap_id != 0 marks device
  // memory inside a symmetric allocation; remote_base is then the offset of ptr in that heap.
  uint32_t register_region(void* ptr, uint64_t nbytes, uint32_t flags = REGION_READABLE | REGION_WRITABLE | REGION_SHARED,
                           uint32_t heap_id = 0, uint64_t remote_base = 0);
  bool unregister_region(uint32_t region_id);
  bool region(uint32_t region_id, MemoryRegion* out) const;

  AddrResolution resolve(const GlobalAddress& g);

  // One-sided copies.  Return a completion id (> 0), or 0 on error (counted in stats).
  // `stream` is a cudaStream_t for device memory (ignored for host memory).
  uint64_t put(const GlobalAddress& dst, const void* src, uint64_t len, void* stream = nullptr);
  uint64_t get(void* dst, const GlobalAddress& src, uint64_t len, void* stream = nullptr);
  // put followed by delivery of a 32-bit immediate to the owner of dst.
  uint64_t put_with_imm(const GlobalAddress& dst, const void* src, uint64_t len, uint32_t imm, void* stream = nullptr);
  // Orders everything issued so far before anything issued later (device: stream event; host: a fence).
  void fence(void* stream = nullptr);
  // True when the operation finished within timeout_ms (default 5 s as in the reference).
  bool poll_completion(uint64_t wr_id, int timeout_ms = 5000);
  // Waits for every outstanding operation; returns how many were pending.
  size_t drain_pending();
  // Immediates delivered to this node since the last call.
  std::vector<ImmRecord> take_immediates();
  void push_immediate(const ImmRecord& r);  // used by fabrics

  DmemStats stats() const;
  MemoryCatalog& catalog() { return catalog_; }

 private:
  struct Pending;
  uint64_t copy(void* dst, const void* src, uint64_t len, bool device, void* stream);
  uint16_t node_id_;
  std::shared_ptr<DmemFabric> fabric_;
  MemoryCatalog catalog_;
  mutable std::mutex mu_;
  std::map<uint32_t, MemoryRegion> regions_;
  uint32_t next_region_ = 1;
  std::map<uint32_t, uint32_t> generations_;
  std::atomic<uint64_t> next_wr_{1};
  std::map<uint64_t, void*> pending_;  // wr id → cudaEvent_t
  std::deque<ImmRecord> imms_;
  DmemStats stats_;
};

// All nodes live in this process and share one address space.
class LocalFabric : public DmemFabric {
 public:
  explicit LocalFabric(int num_nodes) : nodes_(static_cast<size_t>(num_nodes), nullptr) {}
  int num_nodes() const override { return static_cast<int>(nodes_.size()); }
  void attach(uint16_t node, DistributedMemoryManager* m);
  void detach(uint16_t node);
  void publish(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) override;
  void retract(uint16_t node, uint32_t region) override;
  bool fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) override;
  void* map(uint16_t me, uint16_t node, const RegionDirectoryEntry& e, uint64_t remote_addr) override;
  void deliver_imm(uint16_t node, const ImmRecord& r) override;

 private:
  std::mutex mu_;
  std::vector<DistributedMemoryManager*> nodes_;
};

}  // namespace mccl
