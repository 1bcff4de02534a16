// Software coherence for the distributed-memory layer: a home-based directory
// protocol with release consistency at 64 KB granules.
//
// Parity: the reference defines 13 message opcodes (READ_REQ ... BARRIER_LEAVE),
// a message {op, page address, epoch, sender sequence}, a 64 KB granule with
// page_align_down / page_index helpers (csrc/coherence/CoherenceMessage.hpp:15-62),
// a directory entry {UNCACHED / SHARED / EXCLUSIVE, 8-bit sharer mask, exclusive
// owner, epoch} keyed by (region << 32 | page) (csrc/coherence/CoherenceDirectory.hpp:15-76)
// and a protocol object with acquire / release / fence / barrier_all /
// read_page / write_page_done / handle_message / invalidate_sharers /
// global_epoch (csrc/coherence/CoherenceProtocol.hpp:34-104).  The reference
// never starts a receive loop and leaves gpu_acquire / gpu_release empty
// (CoherenceProtocol.cpp:29-65,163-174); here every node runs a service thread
// that drains its mailbox, requests block until the home answers, and the GPU
// pair exists as stream-ordered kernels (csrc/dmem/dmem_kernels.cu).
//
// Messages travel over a CoherenceBus: LocalBus connects nodes inside one
// process (tests, single-process tools); a multi-process bus can carry the same
// 32-byte messages over the group's TCP mesh.  Page data moves with dmem
// put / get, i.e. over NVLink for device regions.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <map>
#include <set>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../dmem/dmem_manager.hpp"

namespace mccl {

constexpr uint64_t COHERENCE_PAGE_SIZE = 64 * 1024;
inline uint64_t page_align_down(uint64_t off) { return off & ~(COHERENCE_PAGE_SIZE - 1); }
inline uint64_t page_index(uint64_t off) { return off / COHERENCE_PAGE_SIZE; }

enum class CoherenceOp : uint8_t {
  READ_REQ = 1, READ_REPLY, READ_REPLY_DIRTY, EXCLUSIVE_REQ, EXCLUSIVE_GRANT, INVALIDATE, INVALIDATE_ACK,
  WRITEBACK_REQ, WRITEBACK_DATA, FENCE, FENCE_ACK, BARRIER_ENTER, BARRIER_LEAVE,
};
const char* coherence_op_name(CoherenceOp op);

#pragma pack(push, 1)
struct CoherenceMessage {
  uint8_t op = 0;
  uint8_t sender = 0;
  uint16_t home = 0;        // node that owns the region
  uint32_t region = 0;
  uint64_t page = 0;        // page index inside the region
  uint64_t epoch = 0;
  uint64_t sender_seq = 0;
};
#pragma pack(pop)
static_assert(sizeof(CoherenceMessage) == 32, "coherence messages are 32 bytes");

enum class PageState : uint8_t { UNCACHED = 0, SHARED = 1, EXCLUSIVE = 2 };

struct DirectoryEntry {
  PageState state = PageState::UNCACHED;
  uint8_t sharers = 0;         // bit n = node n holds a copy (8 nodes = 8 GPUs)
  uint8_t exclusive_owner = 0xff;
  uint64_t epoch = 0;
};

class CoherenceDirectory {
 public:
  static uint64_t key(uint32_t region, uint64_t page) { return (static_cast<uint64_t>(region) << 32) | (page & 0xffffffffu); }
  DirectoryEntry& entry(uint32_t region, uint64_t page) { return map_[key(region, page)]; }
  bool lookup(uint32_t region, uint64_t page, DirectoryEntry* out) const {
    auto it = map_.find(key(region, page));
    if (it == map_.end()) return false;
    if (out) *out = it->second;
    return true;
  }
  void erase_region(uint32_t region) {
    for (auto it = map_.begin(); it != map_.end();) it = (it->first >> 32) == region ? map_.erase(it) : std::next(it);
  }
  void drop_node(uint8_t node);   // a node left: forget its copies
  size_t size() const { return map_.size(); }

 private:
  std::map<uint64_t, DirectoryEntry> map_;
};

class CoherenceBus {
 public:
  virtual ~CoherenceBus() = default;
  virtual int num_nodes() const = 0;
  virtual void send(int dst, const CoherenceMessage& m) = 0;
  // Blocks up to timeout_ms for a message addressed to `node`.
  virtual bool recv(int node, CoherenceMessage* m, int timeout_ms) = 0;
};

class LocalBus : public CoherenceBus {
 public:
  explicit LocalBus(int n) : boxes_(static_cast<size_t>(n)) {}
  int num_nodes() const override { return static_cast<int>(boxes_.size()); }
  void send(int dst, const CoherenceMessage& m) override;
  bool recv(int node, CoherenceMessage* m, int timeout_ms) override;
  // Test hook: messages matching the predicate are silently dropped.
  void set_drop(std::function<bool(int dst, const CoherenceMessage&)> pred);

 private:
  struct Box {
    std::mutex mu;
    std::condition_variable cv;
    std::deque<CoherenceMessage> q;
  };
  std::vector<Box> boxes_;
  std::mutex drop_mu_;
  std::function<bool(int, const CoherenceMessage&)> drop_;
};

struct CoherenceStats {
  uint64_t messages_sent = 0, messages_handled = 0, read_misses = 0, write_misses = 0, invalidations = 0, writebacks = 0,
           timeouts = 0;
};

class CoherenceProtocol {
 public:
  CoherenceProtocol(int node, std::shared_ptr<CoherenceBus> bus, DistributedMemoryManager* dmem, int timeout_ms = 5000);
  ~CoherenceProtocol();
  void start();      // spawns the service thread
  void shutdown();   // idempotent

  // Release consistency.
  void acquire();                      // start of a read phase: advance the local epoch
  void release();                      // write dirty EXCLUSIVE pages home, tell the homes, drop to invalid
  void fence();                        // all earlier messages of this node have been handled by every peer
  void barrier_all();                  // centralised at node 0

  // Makes the page containing g readable (write=false) or writable (write=true) on this node.
  // Returns a pointer to the start of the page's bytes: the home's own memory on the home node, else a local
  // cached copy.  Throws TimeoutError when the home does not answer within the protocol timeout.
  // A page obtained for writing is pinned: a recall from the home (another node wants the page) is held back
  // until write_page_done(), so a write between the two calls can neither be lost nor touch freed memory.
  // A copy obtained for reading stays valid as memory until the next acquire() or release(), even when the
  // home invalidates it in between (it may then be stale, which release consistency allows).
  void* read_page(const GlobalAddress& g, bool write);
  void write_page_done(const GlobalAddress& g);   // marks the cached page dirty, unpins it and answers a held-back recall
  PageState local_state(const GlobalAddress& g) const;
  bool directory_lookup(uint32_t region, uint64_t page, DirectoryEntry* out) const;  // home side
  uint64_t global_epoch() const { return epoch_.load(); }
  CoherenceStats stats() const;

  void handle_message(const CoherenceMessage& m);   // public for tests; normally called by the service thread

 private:
  using PageKey = std::pair<uint16_t, uint64_t>;   // (home, directory key)
  struct CachedPage {
    PageState state = PageState::UNCACHED;
    bool dirty = false;
    bool pinned = false;           // handed out for writing, write_page_done() not called yet
    bool recall = false;           // the home asked for the page back while it was pinned
    CoherenceMessage recall_msg;
    std::vector<uint8_t> data;
  };
  struct Inflight {                // a request of this node whose data has not been installed yet
    bool invalidated = false;      // an INVALIDATE arrived meanwhile: do not cache what is being fetched
    bool recall = false;           // a WRITEBACK_REQ arrived meanwhile: answer it once the page is installed and unpinned
    CoherenceMessage recall_msg;
  };
  struct PendingTxn {         // one outstanding directory transaction per page at the home
    uint8_t requester = 0;
    bool exclusive = false;
    int acks_needed = 0;
    bool waiting_writeback = false;
    uint64_t requester_seq = 0;
  };
  void service_loop();
  void send(int dst, CoherenceOp op, uint16_t home, uint32_t region, uint64_t page, uint64_t epoch = 0, uint64_t seq = 0);
  void home_request(const CoherenceMessage& m, bool exclusive);
  void home_grant(uint32_t region, uint64_t page, const PendingTxn& t, bool refreshed);
  void home_next(uint32_t region, uint64_t page);
  int invalidate_sharers(uint32_t region, uint64_t page, uint8_t except);
  bool wait_reply(uint64_t seq, CoherenceOp* got);
  uint64_t page_bytes(const GlobalAddress& page_start);
  // Writes the page home when dirty and tells the home it is back; called without mu_ held.
  void give_back(const PageKey& k, CachedPage& cp, const CoherenceMessage& recall_msg);

  const int node_;
  std::shared_ptr<CoherenceBus> bus_;
  DistributedMemoryManager* dmem_;
  const int timeout_ms_;
  std::atomic<bool> running_{false};
  std::thread service_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  CoherenceDirectory dir_;                                  // pages this node is home of
  std::map<uint64_t, PendingTxn> pending_;                  // by directory key
  std::map<uint64_t, std::deque<CoherenceMessage>> waiting_;  // requests queued behind a pending transaction
  std::map<PageKey, CachedPage> cache_;                     // local copies
  std::map<PageKey, Inflight> inflight_;                    // requests sent, data not installed yet
  std::set<PageKey> releasing_;                             // pages release() is writing home right now
  std::vector<std::vector<uint8_t>> retired_;               // invalidated copies a reader may still hold a pointer to
  std::map<uint64_t, CoherenceOp> replies_;                 // sender_seq → reply opcode
  std::atomic<uint64_t> next_seq_{1};
  std::atomic<uint64_t> epoch_{0};
  std::atomic<uint64_t> barrier_seq_{0};
  std::atomic<uint64_t> sent_{0};
  std::map<uint64_t, int> barrier_count_;                   // node 0: epoch → arrivals
  std::map<uint64_t, bool> barrier_left_;
  int fence_acks_ = 0;
  CoherenceStats stats_;
};

}  // namespace mccl
