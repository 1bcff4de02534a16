// dmem fabric for one process per GPU: regions live inside symmetric-heap
// allocations (cuMem VMM blocks mapped into every peer over NVLink), so a
// remote region is an ordinary pointer in this process.  Region entries
// travel through the group's key-value store once, at registration.
//
// Immediates (put_with_imm) do not go through the store: every rank owns a
// ring of records per source rank in symmetric memory.  The sender enqueues,
// on the stream that carried the data, a one-thread kernel that writes the
// record into its ring on the destination GPU and then release-stores the
// record's sequence number, so the immediate can never overtake the data and
// the host of the sender does not wait.  The receiver's take_immediates()
// copies its rings to the host and consumes the records whose sequence number
// is the next one expected.  (The reference sends the immediate as an RDMA
// write-with-immediate on the same queue pair as the data:
// csrc/dmem/DistributedMemoryManager.cpp:268-300.)
#pragma once

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../net/kv_store.hpp"
#include "../symm/symm_mesh.hpp"
#include "dmem_kernels.hpp"
#include "dmem_manager.hpp"

namespace mccl {

class SymmFabric : public DmemFabric {
 public:
  static constexpr uint32_t kImmSlots = 256;   // records in flight per (destination, source) pair

  // `imm_rings`: a symmetric allocation of world * kImmSlots * sizeof(ImmWire) bytes per rank (zeroed).
  SymmFabric(KVStore* store, int rank, int world, std::string prefix, int64_t timeout_ms,
             std::shared_ptr<SymmAlloc> imm_rings)
      : store_(store), rank_(rank), world_(world), prefix_(std::move(prefix)), timeout_ms_(timeout_ms),
        rings_(std::move(imm_rings)), sent_(static_cast<size_t>(world), 0), seen_(static_cast<size_t>(world), 0) {}
  int num_nodes() const override { return world_; }
  static size_t ring_bytes(int world) { return static_cast<size_t>(world) * kImmSlots * sizeof(ImmWire); }

  // Heaps are collective allocations: every rank adds the same id for the same allocation.
  void add_heap(uint32_t heap_id, std::shared_ptr<SymmAlloc> heap) {
    std::lock_guard<std::mutex> g(mu_);
    heaps_[heap_id] = std::move(heap);
  }
  std::shared_ptr<SymmAlloc> heap(uint32_t heap_id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = heaps_.find(heap_id);
    return it == heaps_.end() ? nullptr : it->second;
  }

  void publish(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) override {
    std::vector<uint8_t> raw(sizeof(e));
    std::memcpy(raw.data(), &e, sizeof(e));
    store_->set(key(node, region, e.epoch), raw);
    store_->add(prefix_ + "/regions/" + std::to_string(node), 1);
  }
  void retract(uint16_t, uint32_t) override {}   // a new registration of the id gets a new epoch (= key)
  bool fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) override {
    // the newest epoch of the id that has been published: probe upwards from 1
    bool found = false;
    for (uint32_t epoch = 1; epoch < 64; ++epoch) {
      try {
        auto raw = store_->get(key(node, region, epoch), found || epoch > 1 ? 1 : timeout_ms_);
        if (raw.size() != sizeof(*e)) break;
        std::memcpy(e, raw.data(), sizeof(*e));
        found = true;
      } catch (const std::exception&) {
        break;
      }
    }
    return found && e->length != 0;
  }
  void* map(uint16_t, uint16_t node, const RegionDirectoryEntry& e, uint64_t remote_addr) override {
    auto h = heap(e.rkey >> 16);
    if (!h || node >= h->world || !h->ptrs[node] || remote_addr >= h->bytes) return nullptr;
    return static_cast<char*>(h->ptrs[node]) + remote_addr;  // remote_addr is an offset inside the heap
  }
  // Host-ordered delivery (the caller has already waited for the data): same ring, default stream.
  void deliver_imm(uint16_t node, const ImmRecord& r) override { deliver_imm_stream(node, r, nullptr); }
  bool deliver_imm_stream(uint16_t node, const ImmRecord& r, void* stream) override {
    if (!rings_ || node >= world_ || !rings_->ptrs[node]) return false;
    ImmWire w{};
    {
      std::lock_guard<std::mutex> g(mu_);
      w.seq = ++sent_[node];
    }
    w.imm = r.imm;
    w.region_id = r.region_id;
    w.src_node = r.src_node;
    w.offset = r.offset;
    w.length = r.length;
    ImmWire* slot = static_cast<ImmWire*>(rings_->ptrs[node]) + static_cast<size_t>(rank_) * kImmSlots + (w.seq - 1) % kImmSlots;
    return launch_dmem_post_imm(slot, w, static_cast<cudaStream_t>(stream)) == cudaSuccess;
  }
  // Immediates addressed to this rank that have arrived since the last call, in per-source order.
  std::vector<ImmRecord> collect_imm() {
    std::vector<ImmRecord> out;
    if (!rings_) return out;
    std::vector<ImmWire> host(static_cast<size_t>(world_) * kImmSlots);
    if (cudaMemcpy(host.data(), rings_->ptrs[rank_], host.size() * sizeof(ImmWire), cudaMemcpyDeviceToHost) != cudaSuccess) return out;
    std::lock_guard<std::mutex> g(mu_);
    for (int src = 0; src < world_; ++src) {
      for (;;) {
        const ImmWire& w = host[static_cast<size_t>(src) * kImmSlots + seen_[src] % kImmSlots];
        if (w.seq != seen_[src] + 1) break;
        ImmRecord r;
        r.src_node = static_cast<uint16_t>(w.src_node);
        r.region_id = w.region_id;
        r.offset = w.offset;
        r.length = w.length;
        r.imm = w.imm;
        out.push_back(r);
        ++seen_[src];
      }
    }
    return out;
  }

 private:
  std::string key(uint16_t node, uint32_t region, uint32_t epoch) const {
    return prefix_ + "/region/" + std::to_string(node) + "/" + std::to_string(region) + "/" + std::to_string(epoch);
  }
  KVStore* store_;
  int rank_, world_;
  std::string prefix_;
  int64_t timeout_ms_;
  std::mutex mu_;
  std::map<uint32_t, std::shared_ptr<SymmAlloc>> heaps_;
  std::shared_ptr<SymmAlloc> rings_;
  std::vector<uint32_t> sent_, seen_;
};

}  // namespace mccl
