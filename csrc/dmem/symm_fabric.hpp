// dmem fabric for one process per GPU: regions live inside symmetric-heap
// allocations (peer-mapped over NVLink), region entries travel through the
// group's key-value store, immediates through store counters.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <string>

#include "../net/kv_store.hpp"
#include "../symm/symm_mesh.hpp"
#include "dmem_manager.hpp"

namespace mccl {

class SymmFabric : public DmemFabric {
 public:
  SymmFabric(KVStore* store, int rank, int world, std::string prefix, int64_t timeout_ms)
      : store_(store), rank_(rank), world_(world), prefix_(std::move(prefix)), timeout_ms_(timeout_ms) {}
  int num_nodes() const override { return world_; }

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
    store_->set(key(node, region), raw);
  }
  void retract(uint16_t node, uint32_t region) override {
    RegionDirectoryEntry gone{};  // length 0 marks a retired region (store keys cannot be deleted portably)
    publish(node, region, gone);
  }
  bool fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) override {
    try {
      auto raw = store_->get(key(node, region), timeout_ms_);
      if (raw.size() != sizeof(*e)) return false;
      std::memcpy(e, raw.data(), sizeof(*e));
      return e->length != 0;
    } catch (const std::exception&) {
      return false;
    }
  }
  void* map(uint16_t, uint16_t node, const RegionDirectoryEntry& e, uint64_t remote_addr) override {
    auto h = heap(e.rkey >> 16);
    if (!h || node >= h->world || !h->ptrs[node] || remote_addr >= h->bytes) return nullptr;
    return static_cast<char*>(h->ptrs[node]) + remote_addr;  // remote_addr is an offset inside the heap
  }
  void deliver_imm(uint16_t node, const ImmRecord& r) override {
    const int64_t seq = store_->add(prefix_ + "/immseq/" + std::to_string(node), 1);
    std::vector<uint8_t> raw(sizeof(r));
    std::memcpy(raw.data(), &r, sizeof(r));
    store_->set(prefix_ + "/imm/" + std::to_string(node) + "/" + std::to_string(seq), raw);
  }
  // Pulls immediates addressed to `node` that arrived since the last call.
  std::vector<ImmRecord> collect_imm(uint16_t node) {
    std::vector<ImmRecord> out;
    const int64_t upto = store_->add(prefix_ + "/immseq/" + std::to_string(node), 0);
    for (int64_t s = imm_seen_ + 1; s <= upto; ++s) {
      auto raw = store_->get(prefix_ + "/imm/" + std::to_string(node) + "/" + std::to_string(s), timeout_ms_);
      ImmRecord r;
      if (raw.size() == sizeof(r)) {
        std::memcpy(&r, raw.data(), sizeof(r));
        out.push_back(r);
      }
    }
    imm_seen_ = upto;
    return out;
  }

 private:
  std::string key(uint16_t node, uint32_t region) const {
    return prefix_ + "/region/" + std::to_string(node) + "/" + std::to_string(region);
  }
  KVStore* store_;
  int rank_, world_;
  std::string prefix_;
  int64_t timeout_ms_;
  std::mutex mu_;
  std::map<uint32_t, std::shared_ptr<SymmAlloc>> heaps_;
  int64_t imm_seen_ = 0;
};

}  // namespace mccl
