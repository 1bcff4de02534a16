#include "dmem_manager.hpp"

#include <cuda_runtime_api.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "../core/errors.hpp"
#include "../core/log.hpp"

namespace mccl {

DistributedMemoryManager::DistributedMemoryManager(uint16_t node_id, std::shared_ptr<DmemFabric> fabric)
    : node_id_(node_id), fabric_(std::move(fabric)) {
  MCCL_CHECK(fabric_ != nullptr, "dmem: no fabric");
  MCCL_CHECK(node_id_ < fabric_->num_nodes() && fabric_->num_nodes() <= kDmemMaxNodes,
             "dmem: node id " << node_id_ << " outside a fabric of " << fabric_->num_nodes() << " nodes");
  if (auto* lf = dynamic_cast<LocalFabric*>(fabric_.get())) lf->attach(node_id_, this);
}

DistributedMemoryManager::~DistributedMemoryManager() {
  drain_pending();
  std::vector<uint32_t> ids;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : regions_) ids.push_back(kv.first);
  }
  for (uint32_t id : ids) unregister_region(id);
  if (auto* lf = dynamic_cast<LocalFabric*>(fabric_.get())) lf->detach(node_id_);
}

uint32_t DistributedMemoryManager::register_region(void* ptr, uint64_t nbytes, uint32_t flags, uint32_t heap_id,
                                                   uint64_t remote_base) {
  MCCL_CHECK(ptr != nullptr && nbytes > 0, "dmem: cannot register an empty region");
  MemoryRegion r;
  RegionDirectoryEntry e;
  {
    std::lock_guard<std::mutex> g(mu_);
    MCCL_CHECK(regions_.size() < static_cast<size_t>(kDmemMaxRegionsPerNode) - 1,
               "dmem: node " << node_id_ << " already has " << regions_.size() << " regions (limit "
                             << kDmemMaxRegionsPerNode - 1 << ")");
    uint32_t id = next_region_++;
    r.gaddr = GlobalAddress(node_id_, id, 0);
    r.local_addr = ptr;
    r.length = nbytes;
    r.heap_id = heap_id;
    r.generation = ++generations_[id];
    r.flags = flags | ((heap_id && !(flags & REGION_HOST_HEAP)) ? REGION_DEVICE : 0u);
    regions_[id] = r;
    ++stats_.regions;
    e.local_addr = heap_id ? remote_base : reinterpret_cast<uint64_t>(ptr);
    e.length = nbytes;
    e.rkey = (heap_id << 16) | (r.generation & 0xffffu);
    e.flags = r.flags;
    e.epoch = r.generation;
  }
  catalog_.upsert(node_id_, r.gaddr.region_id, e);
  fabric_->publish(node_id_, r.gaddr.region_id, e);
  return r.gaddr.region_id;
}

bool DistributedMemoryManager::unregister_region(uint32_t region_id) {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!regions_.erase(region_id)) return false;
    --stats_.regions;
  }
  catalog_.remove(node_id_, region_id);
  fabric_->retract(node_id_, region_id);
  return true;
}

bool DistributedMemoryManager::region(uint32_t region_id, MemoryRegion* out) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = regions_.find(region_id);
  if (it == regions_.end()) return false;
  if (out) *out = it->second;
  return true;
}

AddrResolution DistributedMemoryManager::resolve(const GlobalAddress& g) {
  AddrResolution a;
  if (g.node_id == node_id_) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = regions_.find(g.region_id);
    if (it == regions_.end() || g.offset >= it->second.length) return a;
    a.ok = a.local = true;
    a.ptr = static_cast<char*>(it->second.local_addr) + g.offset;
    a.remote_addr = reinterpret_cast<uint64_t>(a.ptr);
    a.max_len = it->second.length - g.offset;
    return a;
  }
  RegionDirectoryEntry e;
  if (!catalog_.lookup(g.node_id, g.region_id, &e)) {
    if (!fabric_->fetch(g.node_id, g.region_id, &e)) return a;
    catalog_.upsert(g.node_id, g.region_id, e);
  }
  if (g.offset >= e.length) return a;
  a.remote_addr = e.local_addr + g.offset;
  a.max_len = e.length - g.offset;
  a.ptr = fabric_->map(node_id_, g.node_id, e, a.remote_addr);
  a.ok = a.ptr != nullptr;
  return a;
}

uint64_t DistributedMemoryManager::copy(void* dst, const void* src, uint64_t len, bool device, void* stream) {
  const uint64_t wr = next_wr_.fetch_add(1);
  if (!device) {
    std::memcpy(dst, src, len);
    return wr;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(dst, src, len, cudaMemcpyDefault, st) != cudaSuccess) return 0;
  cudaEvent_t ev = nullptr;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(ev, st) != cudaSuccess) {
    if (ev) cudaEventDestroy(ev);
    return 0;
  }
  std::lock_guard<std::mutex> g(mu_);
  pending_[wr] = ev;
  return wr;
}

uint64_t DistributedMemoryManager::put(const GlobalAddress& dst, const void* src, uint64_t len, void* stream) {
  AddrResolution a = resolve(dst);
  RegionDirectoryEntry e{};
  bool device = false;
  if (a.ok) {
    if (a.local) {
      MemoryRegion r;
      device = region(dst.region_id, &r) && (r.flags & REGION_DEVICE);
    } else {
      catalog_.lookup(dst.node_id, dst.region_id, &e);
      device = (e.flags & REGION_DEVICE) != 0;
      if (!(e.flags & REGION_WRITABLE)) a.ok = false;
    }
  }
  if (!a.ok || len > a.max_len) {
    std::lock_guard<std::mutex> g(mu_);
    ++stats_.total_errors;
    return 0;
  }
  uint64_t wr = copy(a.ptr, src, len, device, stream);
  std::lock_guard<std::mutex> g(mu_);
  if (!wr) {
    ++stats_.total_errors;
    return 0;
  }
  ++stats_.total_put_ops;
  stats_.total_put_bytes += len;
  return wr;
}

uint64_t DistributedMemoryManager::get(void* dst, const GlobalAddress& src, uint64_t len, void* stream) {
  AddrResolution a = resolve(src);
  bool device = false;
  if (a.ok) {
    if (a.local) {
      MemoryRegion r;
      device = region(src.region_id, &r) && (r.flags & REGION_DEVICE);
    } else {
      RegionDirectoryEntry e{};
      catalog_.lookup(src.node_id, src.region_id, &e);
      device = (e.flags & REGION_DEVICE) != 0;
      if (!(e.flags & REGION_READABLE)) a.ok = false;
    }
  }
  if (!a.ok || len > a.max_len) {
    std::lock_guard<std::mutex> g(mu_);
    ++stats_.total_errors;
    return 0;
  }
  uint64_t wr = copy(dst, a.ptr, len, device, stream);
  std::lock_guard<std::mutex> g(mu_);
  if (!wr) {
    ++stats_.total_errors;
    return 0;
  }
  ++stats_.total_get_ops;
  stats_.total_get_bytes += len;
  return wr;
}

uint64_t DistributedMemoryManager::put_with_imm(const GlobalAddress& dst, const void* src, uint64_t len, uint32_t imm,
                                                void* stream) {
  uint64_t wr = put(dst, src, len, stream);
  if (!wr) return 0;
  ImmRecord r;
  r.src_node = node_id_;
  r.region_id = dst.region_id;
  r.offset = dst.offset;
  r.length = len;
  r.imm = imm;
  // The immediate must not overtake the data.  A fabric that can post it on the stream that carried
  // the copy keeps the order on the device; otherwise wait for the copy here first.
  if (dst.node_id != node_id_ && fabric_->deliver_imm_stream(dst.node_id, r, stream)) return wr;
  if (!poll_completion(wr)) {
    std::lock_guard<std::mutex> g(mu_);
    ++stats_.total_errors;
    return 0;
  }
  if (dst.node_id == node_id_) push_immediate(r);
  else fabric_->deliver_imm(dst.node_id, r);
  return wr;
}

void DistributedMemoryManager::fence(void* stream) {
  std::atomic_thread_fence(std::memory_order_seq_cst);
  bool any_device;
  {
    std::lock_guard<std::mutex> g(mu_);
    any_device = !pending_.empty();
  }
  if (any_device) {
    // later work on `stream` is ordered after every copy issued so far
    std::vector<void*> evs;
    {
      std::lock_guard<std::mutex> g(mu_);
      for (auto& kv : pending_) evs.push_back(kv.second);
    }
    for (void* ev : evs) cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(ev), 0);
  }
}

bool DistributedMemoryManager::poll_completion(uint64_t wr_id, int timeout_ms) {
  void* ev = nullptr;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = pending_.find(wr_id);
    if (it == pending_.end()) return wr_id != 0 && wr_id < next_wr_.load();  // host copy or already reaped
    ev = it->second;
  }
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    cudaError_t rc = cudaEventQuery(static_cast<cudaEvent_t>(ev));
    if (rc == cudaSuccess) break;
    if (rc != cudaErrorNotReady) {
      std::lock_guard<std::mutex> g(mu_);
      ++stats_.total_errors;
      break;
    }
    if (std::chrono::steady_clock::now() > deadline) return false;
    std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
  std::lock_guard<std::mutex> g(mu_);
  auto it = pending_.find(wr_id);
  if (it != pending_.end()) {
    cudaEventDestroy(static_cast<cudaEvent_t>(it->second));
    pending_.erase(it);
  }
  return true;
}

size_t DistributedMemoryManager::drain_pending() {
  std::vector<uint64_t> ids;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : pending_) ids.push_back(kv.first);
  }
  for (uint64_t id : ids) poll_completion(id, 30000);
  return ids.size();
}

std::vector<ImmRecord> DistributedMemoryManager::take_immediates() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<ImmRecord> out(imms_.begin(), imms_.end());
  imms_.clear();
  return out;
}

void DistributedMemoryManager::push_immediate(const ImmRecord& r) {
  std::lock_guard<std::mutex> g(mu_);
  imms_.push_back(r);
}

DmemStats DistributedMemoryManager::stats() const {
  std::lock_guard<std::mutex> g(mu_);
  DmemStats s = stats_;
  s.pending = pending_.size();
  return s;
}

// ------------------------------------------------------------- LocalFabric --
void LocalFabric::attach(uint16_t node, DistributedMemoryManager* m) {
  std::lock_guard<std::mutex> g(mu_);
  nodes_[node] = m;
}
void LocalFabric::detach(uint16_t node) {
  std::lock_guard<std::mutex> g(mu_);
  nodes_[node] = nullptr;
}
void LocalFabric::publish(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto* m : nodes_)
    if (m && m->node_id() != node) m->catalog().upsert(node, region, e);
}
void LocalFabric::retract(uint16_t node, uint32_t region) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto* m : nodes_)
    if (m && m->node_id() != node) m->catalog().remove(node, region);
}
bool LocalFabric::fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) {
  std::lock_guard<std::mutex> g(mu_);
  if (node >= nodes_.size() || !nodes_[node]) return false;
  return nodes_[node]->catalog().lookup(node, region, e);
}
void* LocalFabric::map(uint16_t, uint16_t, const RegionDirectoryEntry&, uint64_t remote_addr) {
  return reinterpret_cast<void*>(remote_addr);  // one address space
}
void LocalFabric::deliver_imm(uint16_t node, const ImmRecord& r) {
  std::lock_guard<std::mutex> g(mu_);
  if (node < nodes_.size() && nodes_[node]) nodes_[node]->push_immediate(r);
}

}  // namespace mccl
