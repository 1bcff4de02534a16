#include "coherence.hpp"

#include <chrono>

#include "../core/errors.hpp"
#include "../core/log.hpp"

namespace mccl {

const char* coherence_op_name(CoherenceOp op) {
  static const char* n[] = {"?", "READ_REQ", "READ_REPLY", "READ_REPLY_DIRTY", "EXCLUSIVE_REQ", "EXCLUSIVE_GRANT", "INVALIDATE",
                            "INVALIDATE_ACK", "WRITEBACK_REQ", "WRITEBACK_DATA", "FENCE", "FENCE_ACK", "BARRIER_ENTER",
                            "BARRIER_LEAVE"};
  int i = static_cast<int>(op);
  return i >= 1 && i <= 13 ? n[i] : n[0];
}

void CoherenceDirectory::drop_node(uint8_t node) {
  for (auto& kv : map_) {
    DirectoryEntry& e = kv.second;
    e.sharers &= static_cast<uint8_t>(~(1u << node));
    if (e.state == PageState::EXCLUSIVE && e.exclusive_owner == node) {
      e.state = PageState::UNCACHED;
      e.exclusive_owner = 0xff;
    }
    if (e.state == PageState::SHARED && e.sharers == 0) e.state = PageState::UNCACHED;
  }
}

// ---------------------------------------------------------------- LocalBus --
void LocalBus::set_drop(std::function<bool(int, const CoherenceMessage&)> pred) {
  std::lock_guard<std::mutex> g(drop_mu_);
  drop_ = std::move(pred);
}

void LocalBus::send(int dst, const CoherenceMessage& m) {
  {
    std::lock_guard<std::mutex> g(drop_mu_);
    if (drop_ && drop_(dst, m)) return;
  }
  Box& b = boxes_[static_cast<size_t>(dst)];
  {
    std::lock_guard<std::mutex> g(b.mu);
    b.q.push_back(m);
  }
  b.cv.notify_one();
}

bool LocalBus::recv(int node, CoherenceMessage* m, int timeout_ms) {
  Box& b = boxes_[static_cast<size_t>(node)];
  std::unique_lock<std::mutex> g(b.mu);
  if (!b.cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return !b.q.empty(); })) return false;
  *m = b.q.front();
  b.q.pop_front();
  return true;
}

// ---------------------------------------------------------------- protocol --
CoherenceProtocol::CoherenceProtocol(int node, std::shared_ptr<CoherenceBus> bus, DistributedMemoryManager* dmem, int timeout_ms)
    : node_(node), bus_(std::move(bus)), dmem_(dmem), timeout_ms_(timeout_ms) {
  MCCL_CHECK(bus_ && dmem_, "coherence: needs a bus and a memory manager");
  MCCL_CHECK(bus_->num_nodes() <= 8, "coherence: the sharer mask holds 8 nodes");
}

CoherenceProtocol::~CoherenceProtocol() { shutdown(); }

void CoherenceProtocol::start() {
  if (running_.exchange(true)) return;
  service_ = std::thread([this] { service_loop(); });
}

void CoherenceProtocol::shutdown() {
  if (!running_.exchange(false)) return;
  if (service_.joinable()) service_.join();
}

void CoherenceProtocol::service_loop() {
  CoherenceMessage m;
  while (running_) {
    if (!bus_->recv(node_, &m, 20)) continue;
    try {
      handle_message(m);
    } catch (const std::exception& e) {
      MCCL_ERROR("coherence: node " << node_ << " failed handling " << coherence_op_name(static_cast<CoherenceOp>(m.op)) << ": "
                                    << e.what());
    }
  }
}

void CoherenceProtocol::send(int dst, CoherenceOp op, uint16_t home, uint32_t region, uint64_t page, uint64_t epoch, uint64_t seq) {
  CoherenceMessage m;
  m.op = static_cast<uint8_t>(op);
  m.sender = static_cast<uint8_t>(node_);
  m.home = home;
  m.region = region;
  m.page = page;
  m.epoch = epoch;
  m.sender_seq = seq;
  sent_.fetch_add(1);
  bus_->send(dst, m);
}

uint64_t CoherenceProtocol::page_bytes(const GlobalAddress& page_start) {
  AddrResolution a = dmem_->resolve(page_start);
  MCCL_CHECK(a.ok, "coherence: page " << page_start.region_id << ":" << page_start.offset << " of node "
                                      << page_start.node_id << " is not registered");
  return a.max_len < COHERENCE_PAGE_SIZE ? a.max_len : COHERENCE_PAGE_SIZE;
}

bool CoherenceProtocol::wait_reply(uint64_t seq, CoherenceOp* got) {
  std::unique_lock<std::mutex> g(mu_);
  bool ok = cv_.wait_for(g, std::chrono::milliseconds(timeout_ms_), [&] { return replies_.count(seq) != 0; });
  if (!ok) {
    ++stats_.timeouts;
    return false;
  }
  if (got) *got = replies_[seq];
  replies_.erase(seq);
  return true;
}

void* CoherenceProtocol::read_page(const GlobalAddress& g, bool write) {
  const uint64_t page = page_index(g.offset);
  const GlobalAddress start(g.node_id, g.region_id, page * COHERENCE_PAGE_SIZE);
  const uint64_t key = CoherenceDirectory::key(g.region_id, page);
  const PageKey pk{g.node_id, key};
  const bool home_is_me = g.node_id == node_;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (!home_is_me) {
      auto it = cache_.find(pk);
      if (it != cache_.end() && (it->second.state == PageState::EXCLUSIVE || (!write && it->second.state == PageState::SHARED))) {
        if (write) it->second.pinned = true;
        return it->second.data.data();
      }
      // From here until the data is installed, an INVALIDATE or a recall for this page must not be answered
      // as if this node held nothing: the grant may already be on its way.
      inflight_[pk] = Inflight();
    }
    write ? ++stats_.write_misses : ++stats_.read_misses;
  }
  const uint64_t seq = next_seq_.fetch_add(1);
  send(g.node_id, write ? CoherenceOp::EXCLUSIVE_REQ : CoherenceOp::READ_REQ, g.node_id, g.region_id, page, epoch_.load(), seq);
  CoherenceOp got;
  if (!wait_reply(seq, &got)) {
    Inflight f;
    {
      std::lock_guard<std::mutex> lk(mu_);
      auto it = inflight_.find(pk);
      if (it != inflight_.end()) {
        f = it->second;
        inflight_.erase(it);
      }
    }
    if (f.recall) send(f.recall_msg.sender, CoherenceOp::WRITEBACK_DATA, f.recall_msg.home, f.recall_msg.region, f.recall_msg.page, f.recall_msg.epoch);
    MCCL_CHECK_T(false, TimeoutError,
                 "coherence: node " << g.node_id << " did not answer a " << (write ? "write" : "read") << " request for page "
                                    << page << " of region " << g.region_id << " within " << timeout_ms_ << " ms");
  }
  if (home_is_me) {
    AddrResolution a = dmem_->resolve(start);
    MCCL_CHECK(a.ok, "coherence: local page is not registered");
    return a.ptr;
  }
  const uint64_t len = page_bytes(start);
  CachedPage cp;
  cp.data.resize(len);
  uint64_t wr = dmem_->get(cp.data.data(), start, len);
  const bool fetched = wr != 0 && dmem_->poll_completion(wr, timeout_ms_);
  cp.state = write ? PageState::EXCLUSIVE : PageState::SHARED;
  std::unique_lock<std::mutex> lk(mu_);
  Inflight f;
  {
    auto it = inflight_.find(pk);
    if (it != inflight_.end()) {
      f = it->second;
      inflight_.erase(it);
    }
  }
  if (!fetched || (!write && (f.invalidated || f.recall))) {
    // Not cacheable: the fetch failed, or the home has moved on since it answered.  A reader still gets the
    // bytes that were fetched (valid as memory until the next acquire / release), but the next access asks again.
    lk.unlock();
    if (f.recall) send(f.recall_msg.sender, CoherenceOp::WRITEBACK_DATA, f.recall_msg.home, f.recall_msg.region, f.recall_msg.page, f.recall_msg.epoch);
    MCCL_CHECK(fetched, "coherence: fetching the page data failed");
    lk.lock();
    retired_.push_back(std::move(cp.data));
    return retired_.back().data();
  }
  cp.pinned = write;
  cp.recall = f.recall;          // answered by write_page_done()
  cp.recall_msg = f.recall_msg;
  auto& slot = cache_[pk];
  slot = std::move(cp);
  return slot.data.data();
}

void CoherenceProtocol::give_back(const PageKey& k, CachedPage& cp, const CoherenceMessage& recall_msg) {
  const uint32_t region = static_cast<uint32_t>(k.second >> 32);
  const uint64_t page = k.second & 0xffffffffu;
  if (cp.state == PageState::EXCLUSIVE && cp.dirty) {
    uint64_t wr = dmem_->put(GlobalAddress(k.first, region, page * COHERENCE_PAGE_SIZE), cp.data.data(), cp.data.size());
    if (wr) dmem_->poll_completion(wr, timeout_ms_);
    std::lock_guard<std::mutex> lk(mu_);
    ++stats_.writebacks;
  }
  send(recall_msg.sender, CoherenceOp::WRITEBACK_DATA, recall_msg.home, recall_msg.region, recall_msg.page, recall_msg.epoch);
}

void CoherenceProtocol::write_page_done(const GlobalAddress& g) {
  if (g.node_id == node_) return;  // the home writes in place
  const PageKey pk{g.node_id, CoherenceDirectory::key(g.region_id, page_index(g.offset))};
  CachedPage taken;
  bool recalled = false;
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = cache_.find(pk);
    MCCL_CHECK(it != cache_.end() && it->second.state == PageState::EXCLUSIVE,
               "coherence: write_page_done on a page this node does not hold exclusively");
    it->second.dirty = true;
    it->second.pinned = false;
    if (it->second.recall) {
      // the home asked for the page while it was being written: hand it back now
      recalled = true;
      taken = std::move(it->second);
      cache_.erase(it);
    }
  }
  if (recalled) give_back(pk, taken, taken.recall_msg);
}

PageState CoherenceProtocol::local_state(const GlobalAddress& g) const {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = cache_.find({g.node_id, CoherenceDirectory::key(g.region_id, page_index(g.offset))});
  return it == cache_.end() ? PageState::UNCACHED : it->second.state;
}

bool CoherenceProtocol::directory_lookup(uint32_t region, uint64_t page, DirectoryEntry* out) const {
  std::lock_guard<std::mutex> lk(mu_);
  return dir_.lookup(region, page, out);
}

CoherenceStats CoherenceProtocol::stats() const {
  std::lock_guard<std::mutex> lk(mu_);
  CoherenceStats s = stats_;
  s.messages_sent = sent_.load();
  return s;
}

void CoherenceProtocol::acquire() {
  dmem_->drain_pending();
  epoch_.fetch_add(1);
  std::lock_guard<std::mutex> lk(mu_);
  retired_.clear();
}

void CoherenceProtocol::release() {
  std::map<PageKey, CachedPage> pages;
  {
    std::lock_guard<std::mutex> lk(mu_);
    pages.swap(cache_);
    // a recall that arrives for one of these pages while it is on its way home is answered by the
    // WRITEBACK_DATA below, not by the service thread (which no longer finds the page)
    for (auto& kv : pages) releasing_.insert(kv.first);
  }
  for (auto& kv : pages) {
    const uint16_t home = kv.first.first;
    const uint32_t region = static_cast<uint32_t>(kv.first.second >> 32);
    const uint64_t page = kv.first.second & 0xffffffffu;
    CachedPage& cp = kv.second;
    if (cp.state == PageState::EXCLUSIVE) {
      if (cp.dirty) {
        uint64_t wr = dmem_->put(GlobalAddress(home, region, page * COHERENCE_PAGE_SIZE), cp.data.data(), cp.data.size());
        MCCL_CHECK(wr != 0 && dmem_->poll_completion(wr, timeout_ms_), "coherence: writing a dirty page home failed");
        std::lock_guard<std::mutex> lk(mu_);
        ++stats_.writebacks;
      }
      send(home, CoherenceOp::WRITEBACK_DATA, home, region, page, epoch_.load());
    }
    std::lock_guard<std::mutex> lk(mu_);
    releasing_.erase(kv.first);
  }
  dmem_->drain_pending();
  std::lock_guard<std::mutex> lk(mu_);
  retired_.clear();
}

void CoherenceProtocol::fence() {
  dmem_->fence();
  const int n = bus_->num_nodes();
  {
    std::lock_guard<std::mutex> lk(mu_);
    fence_acks_ = 0;
  }
  for (int p = 0; p < n; ++p)
    if (p != node_) send(p, CoherenceOp::FENCE, 0, 0, 0, epoch_.load());
  std::unique_lock<std::mutex> lk(mu_);
  bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms_), [&] { return fence_acks_ >= n - 1; });
  if (!ok) ++stats_.timeouts;
  MCCL_CHECK_T(ok, TimeoutError, "coherence: fence got " << fence_acks_ << " of " << n - 1 << " acknowledgements within "
                                                         << timeout_ms_ << " ms");
}

void CoherenceProtocol::barrier_all() {
  epoch_.fetch_add(1);
  const uint64_t e = barrier_seq_.fetch_add(1) + 1;  // every node calls barrier_all the same number of times
  send(0, CoherenceOp::BARRIER_ENTER, 0, 0, 0, e);
  std::unique_lock<std::mutex> lk(mu_);
  bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms_), [&] { return barrier_left_.count(e) != 0; });
  if (!ok) ++stats_.timeouts;
  MCCL_CHECK_T(ok, TimeoutError, "coherence: barrier " << e << " was not released within " << timeout_ms_ << " ms");
  barrier_left_.erase(e);
}

int CoherenceProtocol::invalidate_sharers(uint32_t region, uint64_t page, uint8_t except) {
  DirectoryEntry& e = dir_.entry(region, page);
  int sent = 0;
  for (int n = 0; n < bus_->num_nodes(); ++n) {
    if (!(e.sharers & (1u << n)) || n == except || n == node_) continue;
    send(n, CoherenceOp::INVALIDATE, static_cast<uint16_t>(node_), region, page, e.epoch);
    ++sent;
  }
  stats_.invalidations += static_cast<uint64_t>(sent);
  return sent;
}

void CoherenceProtocol::home_grant(uint32_t region, uint64_t page, const PendingTxn& t, bool refreshed) {
  DirectoryEntry& e = dir_.entry(region, page);
  ++e.epoch;
  if (t.exclusive) {
    e.state = PageState::EXCLUSIVE;
    e.exclusive_owner = t.requester;
    e.sharers = static_cast<uint8_t>(1u << t.requester);
    send(t.requester, CoherenceOp::EXCLUSIVE_GRANT, static_cast<uint16_t>(node_), region, page, e.epoch, t.requester_seq);
  } else {
    e.state = PageState::SHARED;
    e.exclusive_owner = 0xff;
    e.sharers |= static_cast<uint8_t>(1u << t.requester);
    send(t.requester, refreshed ? CoherenceOp::READ_REPLY_DIRTY : CoherenceOp::READ_REPLY, static_cast<uint16_t>(node_), region,
         page, e.epoch, t.requester_seq);
  }
}

void CoherenceProtocol::home_next(uint32_t region, uint64_t page) {
  const uint64_t key = CoherenceDirectory::key(region, page);
  while (!pending_.count(key)) {
    auto it = waiting_.find(key);
    if (it == waiting_.end() || it->second.empty()) {
      if (it != waiting_.end()) waiting_.erase(it);
      return;
    }
    CoherenceMessage m = it->second.front();
    it->second.pop_front();
    home_request(m, static_cast<CoherenceOp>(m.op) == CoherenceOp::EXCLUSIVE_REQ);
  }
}

void CoherenceProtocol::home_request(const CoherenceMessage& m, bool exclusive) {
  const uint64_t key = CoherenceDirectory::key(m.region, m.page);
  if (pending_.count(key)) {
    waiting_[key].push_back(m);
    return;
  }
  DirectoryEntry& e = dir_.entry(m.region, m.page);
  PendingTxn t;
  t.requester = m.sender;
  t.exclusive = exclusive;
  t.requester_seq = m.sender_seq;
  if (e.state == PageState::EXCLUSIVE && e.exclusive_owner != m.sender && e.exclusive_owner != node_ && e.exclusive_owner != 0xff) {
    t.waiting_writeback = true;
    pending_[key] = t;
    send(e.exclusive_owner, CoherenceOp::WRITEBACK_REQ, static_cast<uint16_t>(node_), m.region, m.page, e.epoch);
    return;
  }
  if (exclusive) {
    const int n = invalidate_sharers(m.region, m.page, m.sender);
    if (n > 0) {
      t.acks_needed = n;
      pending_[key] = t;
      return;
    }
  }
  home_grant(m.region, m.page, t, false);
}

void CoherenceProtocol::handle_message(const CoherenceMessage& m) {
  std::unique_lock<std::mutex> lk(mu_);
  ++stats_.messages_handled;
  const CoherenceOp op = static_cast<CoherenceOp>(m.op);
  const uint64_t key = CoherenceDirectory::key(m.region, m.page);
  switch (op) {
    case CoherenceOp::READ_REQ: home_request(m, false); break;
    case CoherenceOp::EXCLUSIVE_REQ: home_request(m, true); break;
    case CoherenceOp::INVALIDATE_ACK: {
      auto it = pending_.find(key);
      if (it != pending_.end() && it->second.acks_needed > 0 && --it->second.acks_needed == 0) {
        PendingTxn t = it->second;
        pending_.erase(it);
        dir_.entry(m.region, m.page).sharers &= static_cast<uint8_t>((1u << t.requester) | (1u << node_));
        home_grant(m.region, m.page, t, false);
        home_next(m.region, m.page);
      }
      break;
    }
    case CoherenceOp::WRITEBACK_DATA: {
      DirectoryEntry& e = dir_.entry(m.region, m.page);
      // Only the current exclusive owner can give the page back.  (A node whose release() crossed a recall
      // answers twice; by the time the second answer arrives the page may belong to somebody else.)
      if (e.state != PageState::EXCLUSIVE || e.exclusive_owner != m.sender) break;
      e.state = PageState::UNCACHED;
      e.sharers = 0;
      e.exclusive_owner = 0xff;
      auto it = pending_.find(key);
      if (it != pending_.end() && it->second.waiting_writeback) {
        PendingTxn t = it->second;
        pending_.erase(it);
        home_grant(m.region, m.page, t, true);
        home_next(m.region, m.page);
      }
      break;
    }
    case CoherenceOp::INVALIDATE: {
      const PageKey pk{m.home, key};
      auto it = cache_.find(pk);
      if (it != cache_.end()) {
        retired_.push_back(std::move(it->second.data));   // a reader may still be looking at it
        cache_.erase(it);
      }
      auto fi = inflight_.find(pk);
      if (fi != inflight_.end()) fi->second.invalidated = true;
      send(m.sender, CoherenceOp::INVALIDATE_ACK, m.home, m.region, m.page, m.epoch);
      break;
    }
    case CoherenceOp::WRITEBACK_REQ: {
      const PageKey pk{m.home, key};
      if (releasing_.count(pk)) break;   // release() is writing it home and will say so itself
      auto it = cache_.find(pk);
      if (it != cache_.end()) {
        if (it->second.pinned) {         // being written right now: answered by write_page_done()
          it->second.recall = true;
          it->second.recall_msg = m;
          break;
        }
        CachedPage cp = std::move(it->second);
        cache_.erase(it);
        lk.unlock();
        give_back(pk, cp, m);
        lk.lock();
        break;
      }
      auto fi = inflight_.find(pk);
      if (fi != inflight_.end()) {       // granted, data not installed yet: answered once it is
        fi->second.recall = true;
        fi->second.recall_msg = m;
        break;
      }
      send(m.sender, CoherenceOp::WRITEBACK_DATA, m.home, m.region, m.page, m.epoch);
      break;
    }
    case CoherenceOp::READ_REPLY:
    case CoherenceOp::READ_REPLY_DIRTY:
    case CoherenceOp::EXCLUSIVE_GRANT:
      replies_[m.sender_seq] = op;
      cv_.notify_all();
      break;
    case CoherenceOp::FENCE: send(m.sender, CoherenceOp::FENCE_ACK, 0, 0, 0, m.epoch); break;
    case CoherenceOp::FENCE_ACK:
      ++fence_acks_;
      cv_.notify_all();
      break;
    case CoherenceOp::BARRIER_ENTER: {
      if (++barrier_count_[m.epoch] == bus_->num_nodes()) {
        barrier_count_.erase(m.epoch);
        for (int n = 0; n < bus_->num_nodes(); ++n) send(n, CoherenceOp::BARRIER_LEAVE, 0, 0, 0, m.epoch);
      }
      break;
    }
    case CoherenceOp::BARRIER_LEAVE:
      barrier_left_[m.epoch] = true;
      cv_.notify_all();
      break;
    default: break;
  }
}

}  // namespace mccl
