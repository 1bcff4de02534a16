// Cross-process fabric and coherence bus for the ranks of one box, over POSIX
// shared memory.
//
// The reference plans its distributed memory over RDMA queue pairs between
// hosts (csrc/dmem/DistributedMemoryManager.cpp:19-39, csrc/transport/rdma/)
// and never connects the coherence protocol to a transport (CoherenceProtocol.cpp:29-65).
// On one box the processes of a job can share pages directly, so here
//   * host regions are carved from shared-memory heaps that every process of
//     the job can map (the GPU counterpart is the symmetric heap, symm_fabric.hpp),
//   * the region directory, the immediate-data queues and the coherence
//     mailboxes live in one control segment, as lock-free rings.
// Everything a node publishes is visible to the others without a round trip.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <utility>
#include <vector>

#include "../coherence/coherence.hpp"
#include "../core/errors.hpp"
#include "dmem_manager.hpp"

namespace mccl {

constexpr int kShmMaxNodes = 8;
constexpr int kShmMaxRegions = 256;
constexpr uint32_t kShmMagic = 0x4d43434cu;  // "MCCL"

// Bounded multi-producer queue of fixed-size cells (sequence-number scheme): usable from
// several processes because it holds nothing but atomics and plain data.
template <typename T, uint32_t N>
struct ShmRing {
  static_assert((N & (N - 1)) == 0, "ring size must be a power of two");
  struct Cell {
    std::atomic<uint64_t> seq;
    T value;
  };
  std::atomic<uint64_t> head, tail;
  Cell cells[N];

  void init() {
    head.store(0);
    tail.store(0);
    for (uint32_t i = 0; i < N; ++i) cells[i].seq.store(i);
  }
  bool push(const T& v) {
    uint64_t pos = tail.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells[pos & (N - 1)];
      const uint64_t seq = c.seq.load(std::memory_order_acquire);
      const int64_t dif = static_cast<int64_t>(seq) - static_cast<int64_t>(pos);
      if (dif == 0) {
        if (tail.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
          c.value = v;
          c.seq.store(pos + 1, std::memory_order_release);
          return true;
        }
      } else if (dif < 0) {
        return false;  // full
      } else {
        pos = tail.load(std::memory_order_relaxed);
      }
    }
  }
  bool pop(T* out) {
    uint64_t pos = head.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells[pos & (N - 1)];
      const uint64_t seq = c.seq.load(std::memory_order_acquire);
      const int64_t dif = static_cast<int64_t>(seq) - static_cast<int64_t>(pos + 1);
      if (dif == 0) {
        if (head.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
          *out = c.value;
          c.seq.store(pos + N, std::memory_order_release);
          return true;
        }
      } else if (dif < 0) {
        return false;  // empty
      } else {
        pos = head.load(std::memory_order_relaxed);
      }
    }
  }
};

struct ShmControl {
  std::atomic<uint32_t> magic;
  uint32_t num_nodes;
  struct DirSlot {
    std::atomic<uint32_t> version;   // odd while being written
    RegionDirectoryEntry entry;      // length 0 = unknown
  } dir[kShmMaxNodes][kShmMaxRegions];
  ShmRing<ImmRecord, 256> imm[kShmMaxNodes];
  ShmRing<CoherenceMessage, 1024> mail[kShmMaxNodes];
};

// One mapping of a named shared-memory object.
class ShmSegment {
 public:
  // create: make (and size) the object, failing if it exists; otherwise open an existing one, waiting for it.
  ShmSegment(std::string name, size_t bytes, bool create, int timeout_ms = 10000) : name_(std::move(name)) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
      fd_ = create ? shm_open(name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600) : shm_open(name_.c_str(), O_RDWR, 0600);
      if (fd_ >= 0) break;
      MCCL_CHECK_T(!create && std::chrono::steady_clock::now() < deadline, TransportError,
                   "shared memory " << name_ << ": " << std::strerror(errno));
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    owner_ = create;
    if (create) {
      MCCL_CHECK_T(ftruncate(fd_, static_cast<off_t>(bytes)) == 0, TransportError, "shared memory " << name_ << ": cannot size it");
      bytes_ = bytes;
    } else {
      struct stat st {};
      for (;;) {  // the creator may not have sized it yet
        MCCL_CHECK_T(fstat(fd_, &st) == 0, TransportError, "shared memory " << name_ << ": fstat failed");
        if (st.st_size > 0 && (bytes == 0 || static_cast<size_t>(st.st_size) >= bytes)) break;
        MCCL_CHECK_T(std::chrono::steady_clock::now() < deadline, TimeoutError, "shared memory " << name_ << " was never sized");
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
      bytes_ = static_cast<size_t>(st.st_size);
    }
    ptr_ = mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
    MCCL_CHECK_T(ptr_ != MAP_FAILED, TransportError, "shared memory " << name_ << ": mmap failed");
  }
  ~ShmSegment() {
    if (ptr_ && ptr_ != MAP_FAILED) munmap(ptr_, bytes_);
    if (fd_ >= 0) close(fd_);
    if (owner_) shm_unlink(name_.c_str());
  }
  ShmSegment(const ShmSegment&) = delete;
  ShmSegment& operator=(const ShmSegment&) = delete;
  void* ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }

 private:
  std::string name_;
  int fd_ = -1;
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
  bool owner_ = false;
};

// dmem fabric of one process of a job on this box.  `name` identifies the job; node 0 creates the
// control segment, the others attach to it.
class ShmFabric : public DmemFabric {
 public:
  ShmFabric(const std::string& name, int node, int num_nodes, int timeout_ms = 10000)
      : name_("/mccl-" + name), node_(node), num_nodes_(num_nodes), timeout_ms_(timeout_ms) {
    MCCL_CHECK(num_nodes >= 1 && num_nodes <= kShmMaxNodes && node >= 0 && node < num_nodes,
               "shared-memory fabric: node " << node << " of " << num_nodes << " (at most " << kShmMaxNodes << ")");
    control_.reset(new ShmSegment(name_, sizeof(ShmControl), node == 0, timeout_ms));
    ctl_ = static_cast<ShmControl*>(control_->ptr());
    if (node == 0) {
      ctl_->num_nodes = static_cast<uint32_t>(num_nodes);
      for (int n = 0; n < kShmMaxNodes; ++n) {
        for (int r = 0; r < kShmMaxRegions; ++r) {
          ctl_->dir[n][r].version.store(0);
          ctl_->dir[n][r].entry = RegionDirectoryEntry{};
        }
        ctl_->imm[n].init();
        ctl_->mail[n].init();
      }
      ctl_->magic.store(kShmMagic, std::memory_order_release);
    } else {
      const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
      while (ctl_->magic.load(std::memory_order_acquire) != kShmMagic) {
        MCCL_CHECK_T(std::chrono::steady_clock::now() < deadline, TimeoutError, "shared-memory fabric " << name_ << " was never initialised");
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
      MCCL_CHECK(ctl_->num_nodes == static_cast<uint32_t>(num_nodes), "shared-memory fabric " << name_ << " was created for "
                                                                                            << ctl_->num_nodes << " nodes");
    }
  }

  int node() const { return node_; }
  int num_nodes() const override { return num_nodes_; }
  ShmControl* control() { return ctl_; }

  // A heap of `bytes` bytes that every process of the job can map.  Regions registered from it pass
  // the returned id and their offset inside the heap to register_region.
  std::pair<uint32_t, void*> alloc_heap(size_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    const uint32_t id = next_heap_++;
    auto seg = std::make_shared<ShmSegment>(heap_name(node_, id), bytes, true, timeout_ms_);
    std::memset(seg->ptr(), 0, bytes);
    heaps_[{node_, id}] = seg;
    return {id, seg->ptr()};
  }

  void publish(uint16_t node, uint32_t region, const RegionDirectoryEntry& e) override {
    if (node >= kShmMaxNodes || region >= static_cast<uint32_t>(kShmMaxRegions)) return;
    auto& s = ctl_->dir[node][region];
    const uint32_t v = s.version.load(std::memory_order_relaxed);
    s.version.store(v + 1, std::memory_order_release);   // odd: being written
    std::atomic_thread_fence(std::memory_order_release);
    s.entry = e;
    s.version.store(v + 2, std::memory_order_release);
  }
  void retract(uint16_t node, uint32_t region) override { publish(node, region, RegionDirectoryEntry{}); }
  bool fetch(uint16_t node, uint32_t region, RegionDirectoryEntry* e) override {
    if (node >= kShmMaxNodes || region >= static_cast<uint32_t>(kShmMaxRegions)) return false;
    auto& s = ctl_->dir[node][region];
    for (int tries = 0; tries < 1000; ++tries) {
      const uint32_t v0 = s.version.load(std::memory_order_acquire);
      if (v0 & 1u) continue;
      RegionDirectoryEntry copy = s.entry;
      std::atomic_thread_fence(std::memory_order_acquire);
      if (s.version.load(std::memory_order_relaxed) != v0) continue;
      if (copy.length == 0) return false;
      *e = copy;
      return true;
    }
    return false;
  }
  void* map(uint16_t, uint16_t node, const RegionDirectoryEntry& e, uint64_t remote_addr) override {
    const uint32_t heap = e.rkey >> 16;
    if (heap == 0) return nullptr;   // ordinary host memory of another process cannot be reached
    std::shared_ptr<ShmSegment> seg;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = heaps_.find({node, heap});
      if (it != heaps_.end()) seg = it->second;
    }
    if (!seg) {
      try {
        seg = std::make_shared<ShmSegment>(heap_name(node, heap), 0, false, timeout_ms_);
      } catch (const std::exception&) {
        return nullptr;
      }
      std::lock_guard<std::mutex> g(mu_);
      heaps_[{node, heap}] = seg;
    }
    if (remote_addr >= seg->bytes()) return nullptr;
    return static_cast<char*>(seg->ptr()) + remote_addr;   // remote_addr is an offset inside the heap
  }
  void deliver_imm(uint16_t node, const ImmRecord& r) override {
    if (node < kShmMaxNodes) ctl_->imm[node].push(r);
  }
  std::vector<ImmRecord> collect_imm() {
    std::vector<ImmRecord> out;
    ImmRecord r;
    while (ctl_->imm[node_].pop(&r)) out.push_back(r);
    return out;
  }

 private:
  std::string heap_name(int node, uint32_t id) const { return name_ + "-h" + std::to_string(node) + "-" + std::to_string(id); }
  std::string name_;
  int node_, num_nodes_, timeout_ms_;
  std::unique_ptr<ShmSegment> control_;
  ShmControl* ctl_ = nullptr;
  std::mutex mu_;
  uint32_t next_heap_ = 1;
  std::map<std::pair<int, uint32_t>, std::shared_ptr<ShmSegment>> heaps_;
};

// Coherence messages between the processes of a job: one mailbox per node in the control segment.
class ShmBus : public CoherenceBus {
 public:
  explicit ShmBus(std::shared_ptr<ShmFabric> fabric) : fabric_(std::move(fabric)) {}
  int num_nodes() const override { return fabric_->num_nodes(); }
  void send(int dst, const CoherenceMessage& m) override {
    if (dst < 0 || dst >= fabric_->num_nodes()) return;
    auto& ring = fabric_->control()->mail[dst];
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(5);
    while (!ring.push(m)) {   // full: the receiver is behind
      MCCL_CHECK_T(std::chrono::steady_clock::now() < deadline, TimeoutError, "coherence mailbox of node " << dst << " stayed full");
      std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  bool recv(int node, CoherenceMessage* m, int timeout_ms) override {
    MCCL_CHECK(node == fabric_->node(), "a process reads only its own coherence mailbox");
    auto& ring = fabric_->control()->mail[node];
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    int idle = 0;
    for (;;) {
      if (ring.pop(m)) return true;
      if (std::chrono::steady_clock::now() >= deadline) return false;
      if (++idle < 200) std::this_thread::yield();
      else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }

 private:
  std::shared_ptr<ShmFabric> fabric_;
};

}  // namespace mccl
