// Cluster membership, failure detection and the scheduler loop (host only).
//
// Parity: the reference's ClusterManager tracks up to 8 nodes, handles join /
// leave / heartbeat, elects the lowest online node id as leader, and on the
// head runs three threads: a heartbeat sender that PINGs every online node's
// agent over TCP every 500 ms with a 1 s socket timeout, a monitor that marks a
// node OFFLINE after 2000 ms of silence, and a scheduler tick every second;
// a failed node is purged from the memory catalog, its jobs are evicted and a
// leader is re-elected (csrc/runtime/ClusterManager.hpp:18-119,
// ClusterManager.cpp:54-401).  The intervals are parameters here so that tests
// can run the same logic in tens of milliseconds.
#pragma once

#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../dmem/memory_catalog.hpp"
#include "scheduler.hpp"

namespace mccl {

constexpr int kMaxClusterNodes = 8;

enum class NodeStatus : int { ONLINE = 0, SUSPECT = 1, OFFLINE = 2 };

struct NodeInfo {
  int node_id = 0;
  std::string host = "127.0.0.1";
  int agent_port = 0;
  NodeStatus status = NodeStatus::OFFLINE;
  double last_heartbeat = 0;   // seconds, steady clock
  uint64_t memory_total = 0, memory_used = 0;
  uint64_t heartbeats = 0;
};

struct ClusterTimings {
  int heartbeat_interval_ms = 500;
  int heartbeat_timeout_ms = 2000;
  int ping_socket_timeout_ms = 1000;
  int scheduler_tick_ms = 1000;
};

class ClusterManager {
 public:
  ClusterManager(int self_node, ClusterTimings t = ClusterTimings());
  ~ClusterManager();

  // Membership.
  bool handle_join(const NodeInfo& info);          // false when the cluster is full or the id is out of range
  bool handle_leave(int node_id);
  bool handle_heartbeat(int node_id, uint64_t memory_used = 0);
  void handle_node_failure(int node_id);
  int leader() const;                               // lowest online node id, -1 when none
  bool is_leader() const { return leader() == self_; }
  std::vector<NodeInfo> nodes() const;
  int online_count() const;
  uint64_t version() const { return version_.load(); }

  // Head-only service threads (heartbeat sender, monitor, scheduler tick).
  void start();
  void stop();
  bool running() const { return running_.load(); }

  // Region directory shared with the memory layer.
  bool publish_region(int node_id, uint32_t region, const RegionDirectoryEntry& e);
  bool lookup_region(int node_id, uint32_t region, RegionDirectoryEntry* out) const;
  MemoryCatalog& catalog() { return catalog_; }
  Scheduler& scheduler() { return scheduler_; }

  // Called (on a service thread) when a node is declared failed / when jobs start.
  void on_failure(std::function<void(int)> cb) { failure_cb_ = std::move(cb); }
  void on_placement(std::function<void(const Placement&)> cb) { placement_cb_ = std::move(cb); }

 private:
  void heartbeat_sender_loop();
  void heartbeat_monitor_loop();
  void scheduler_loop();
  void elect_locked();
  static double now();

  const int self_;
  const ClusterTimings t_;
  mutable std::mutex mu_;
  std::map<int, NodeInfo> nodes_;
  int leader_ = -1;
  std::atomic<uint64_t> version_{0};
  std::atomic<bool> running_{false};
  std::thread sender_, monitor_, sched_;
  MemoryCatalog catalog_;
  Scheduler scheduler_;
  std::function<void(int)> failure_cb_;
  std::function<void(const Placement&)> placement_cb_;
};

}  // namespace mccl
