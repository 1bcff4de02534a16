// Minimal key-value rendezvous interface.
//
// The transports bootstrap through whatever store torch.distributed hands the
// process group (TCPStore, FileStore, HashStore behind a PrefixStore).  They
// only need set / blocking get / add, so that is all this interface asks for;
// the process group adapts c10d::Store to it and the C++ unit tests use the
// in-memory implementation below.
#pragma once

#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../core/errors.hpp"

namespace mccl {

class KVStore {
 public:
  virtual ~KVStore() = default;
  virtual void set(const std::string& key, const std::vector<uint8_t>& value) = 0;
  // Blocks until the key exists or timeout_ms elapses (TimeoutError).
  virtual std::vector<uint8_t> get(const std::string& key, int64_t timeout_ms) = 0;
  // Atomic add on an integer key (missing key counts as 0); returns new value.
  virtual int64_t add(const std::string& key, int64_t delta) = 0;

  void set_str(const std::string& key, const std::string& v) {
    set(key, std::vector<uint8_t>(v.begin(), v.end()));
  }
  std::string get_str(const std::string& key, int64_t timeout_ms) {
    auto v = get(key, timeout_ms);
    return std::string(v.begin(), v.end());
  }
};

// Process-local store shared by threads; used by unit tests that run several
// "ranks" as threads of one process.
class MemoryKVStore : public KVStore {
 public:
  void set(const std::string& key, const std::vector<uint8_t>& value) override {
    {
      std::lock_guard<std::mutex> g(mu_);
      data_[key] = value;
    }
    cv_.notify_all();
  }
  std::vector<uint8_t> get(const std::string& key, int64_t timeout_ms) override {
    std::unique_lock<std::mutex> g(mu_);
    bool ok = cv_.wait_for(g, std::chrono::milliseconds(timeout_ms),
                           [&] { return data_.count(key) != 0; });
    MCCL_CHECK_T(ok, TimeoutError, "store: key '" << key << "' not set within " << timeout_ms << " ms");
    return data_[key];
  }
  int64_t add(const std::string& key, int64_t delta) override {
    int64_t now;
    {
      std::lock_guard<std::mutex> g(mu_);
      int64_t cur = 0;
      auto it = data_.find(key);
      if (it != data_.end()) cur = std::stoll(std::string(it->second.begin(), it->second.end()));
      now = cur + delta;
      std::string s = std::to_string(now);
      data_[key] = std::vector<uint8_t>(s.begin(), s.end());
    }
    cv_.notify_all();
    return now;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<std::string, std::vector<uint8_t>> data_;
};

// Store-based barrier.  Every rank sets <prefix>/barrier/<tag>/<rank> and then
// waits for every other rank's key; keys are never deleted, so tags must be
// unique per use (reference behaviour: csrc/runtime/Rendezvous.cpp:58-79).
class Rendezvous {
 public:
  Rendezvous(KVStore* store, int rank, int world, int64_t timeout_ms, std::string prefix = "mccl")
      : store_(store), rank_(rank), world_(world), timeout_ms_(timeout_ms), prefix_(std::move(prefix)) {}

  void barrier(const std::string& tag) {
    store_->set_str(key("barrier/" + tag, rank_), "1");
    for (int r = 0; r < world_; ++r) {
      if (r == rank_) continue;
      try {
        store_->get(key("barrier/" + tag, r), timeout_ms_);
      } catch (const TimeoutError&) {
        MCCL_CHECK_T(false, TimeoutError,
                     "barrier '" << tag << "': rank " << r << " did not arrive within " << timeout_ms_ << " ms");
      }
    }
  }

  // Publishes this rank's endpoint string and returns everybody's, indexed by rank.
  std::vector<std::string> exchange_endpoints(const std::string& mine, const std::string& what = "endpoint") {
    store_->set_str(key(what, rank_), mine);
    std::vector<std::string> all(world_);
    for (int r = 0; r < world_; ++r)
      all[r] = (r == rank_) ? mine : store_->get_str(key(what, r), timeout_ms_);
    return all;
  }

  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  std::string key(const std::string& what, int r) const {
    return prefix_ + "/" + what + "/" + std::to_string(r);
  }
  KVStore* store_;
  int rank_, world_;
  int64_t timeout_ms_;
  std::string prefix_;
};

}  // namespace mccl
