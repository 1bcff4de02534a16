// Replicated directory of registered regions.
//
// Parity: the reference's MemoryCatalog maps (node, region) to a 32-byte wire
// entry {local address, length, rkey, flags, epoch}, allows 256 regions per
// node, and offers upsert / remove / remove_node / lookup / serialize_into /
// deserialize_from / version (csrc/dmem/MemoryCatalog.hpp:16-88,
// MemoryCatalog.cpp:9-95).  The reference keys local entries with node 0; here
// every entry is keyed by its true node id.
#pragma once

#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "global_address.hpp"

namespace mccl {

#pragma pack(push, 1)
struct RegionDirectoryEntry {
  uint64_t local_addr = 0;
  uint64_t length = 0;
  uint32_t rkey = 0;     // heap id << 16 | generation
  uint32_t flags = 0;
  uint64_t epoch = 0;
};
#pragma pack(pop)
static_assert(sizeof(RegionDirectoryEntry) == 32, "directory entries are 32 bytes on the wire");

class MemoryCatalog {
 public:
  // Returns false when the node already has kDmemMaxRegionsPerNode regions.
  bool upsert(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) {
    std::lock_guard<std::mutex> g(mu_);
    auto key = std::make_pair(node, region);
    if (!entries_.count(key)) {
      int n = 0;
      for (auto& kv : entries_) n += kv.first.first == node;
      if (n >= kDmemMaxRegionsPerNode) return false;
    }
    entries_[key] = e;
    ++version_;
    return true;
  }
  bool remove(uint16_t node, uint32_t region) {
    std::lock_guard<std::mutex> g(mu_);
    bool hit = entries_.erase({node, region}) != 0;
    if (hit) ++version_;
    return hit;
  }
  size_t remove_node(uint16_t node) {
    std::lock_guard<std::mutex> g(mu_);
    size_t n = 0;
    for (auto it = entries_.begin(); it != entries_.end();) {
      if (it->first.first == node) {
        it = entries_.erase(it);
        ++n;
      } else {
        ++it;
      }
    }
    if (n) ++version_;
    return n;
  }
  bool lookup(uint16_t node, uint32_t region, RegionDirectoryEntry* out) const {
    std::lock_guard<std::mutex> g(mu_);
    auto it = entries_.find({node, region});
    if (it == entries_.end()) return false;
    if (out) *out = it->second;
    return true;
  }
  size_t size() const {
    std::lock_guard<std::mutex> g(mu_);
    return entries_.size();
  }
  uint64_t version() const {
    std::lock_guard<std::mutex> g(mu_);
    return version_;
  }
  // Wire form: u32 count, then per entry u16 node, u32 region, 32-byte entry.
  std::vector<uint8_t> serialize() const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<uint8_t> out(4 + entries_.size() * 38);
    uint32_t n = static_cast<uint32_t>(entries_.size());
    std::memcpy(out.data(), &n, 4);
    size_t o = 4;
    for (auto& kv : entries_) {
      std::memcpy(out.data() + o, &kv.first.first, 2);
      std::memcpy(out.data() + o + 2, &kv.first.second, 4);
      std::memcpy(out.data() + o + 6, &kv.second, 32);
      o += 38;
    }
    return out;
  }
  // Merges entries from a serialized catalog; returns how many were read (-1 on malformed input).
  int deserialize(const std::vector<uint8_t>& in) {
    if (in.size() < 4) return -1;
    uint32_t n;
    std::memcpy(&n, in.data(), 4);
    if (in.size() != 4 + static_cast<size_t>(n) * 38) return -1;
    for (uint32_t i = 0; i < n; ++i) {
      uint16_t node;
      uint32_t region;
      RegionDirectoryEntry e;
      std::memcpy(&node, in.data() + 4 + i * 38, 2);
      std::memcpy(&region, in.data() + 4 + i * 38 + 2, 4);
      std::memcpy(&e, in.data() + 4 + i * 38 + 6, 32);
      upsert(node, region, e);
    }
    return static_cast<int>(n);
  }

 private:
  mutable std::mutex mu_;
  std::map<std::pair<uint16_t, uint32_t>, RegionDirectoryEntry> entries_;
  uint64_t version_ = 0;
};

}  // namespace mccl
