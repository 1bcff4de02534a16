#include "cluster_manager.hpp"

#include <chrono>

#include "../core/log.hpp"
#include "agent.hpp"

namespace mccl {

double ClusterManager::now() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

ClusterManager::ClusterManager(int self_node, ClusterTimings t) : self_(self_node), t_(t) {}
ClusterManager::~ClusterManager() { stop(); }

void ClusterManager::elect_locked() {
  int best = -1;
  for (auto& kv : nodes_)
    if (kv.second.status == NodeStatus::ONLINE && (best < 0 || kv.first < best)) best = kv.first;
  if (best != leader_) {
    leader_ = best;
    MCCL_INFO("cluster: leader is now node " << best);
  }
}

bool ClusterManager::handle_join(const NodeInfo& info) {
  std::lock_guard<std::mutex> g(mu_);
  if (info.node_id < 0 || info.node_id >= kMaxClusterNodes) return false;
  if (!nodes_.count(info.node_id) && static_cast<int>(nodes_.size()) >= kMaxClusterNodes) return false;
  NodeInfo n = info;
  n.status = NodeStatus::ONLINE;
  n.last_heartbeat = now();
  nodes_[info.node_id] = n;
  ++version_;
  elect_locked();
  return true;
}

bool ClusterManager::handle_leave(int node_id) {
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = nodes_.find(node_id);
    if (it == nodes_.end()) return false;
    nodes_.erase(it);
    ++version_;
    elect_locked();
  }
  catalog_.remove_node(static_cast<uint16_t>(node_id));
  scheduler_.evict_node(node_id);
  return true;
}

bool ClusterManager::handle_heartbeat(int node_id, uint64_t memory_used) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = nodes_.find(node_id);
  if (it == nodes_.end()) return false;
  it->second.last_heartbeat = now();
  ++it->second.heartbeats;
  if (memory_used) it->second.memory_used = memory_used;
  if (it->second.status != NodeStatus::ONLINE) {
    it->second.status = NodeStatus::ONLINE;   // the node came back
    ++version_;
    elect_locked();
  }
  return true;
}

void ClusterManager::handle_node_failure(int node_id) {
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = nodes_.find(node_id);
    if (it == nodes_.end() || it->second.status == NodeStatus::OFFLINE) return;
    it->second.status = NodeStatus::OFFLINE;
    ++version_;
    elect_locked();
  }
  MCCL_WARN("cluster: node " << node_id << " declared OFFLINE");
  catalog_.remove_node(static_cast<uint16_t>(node_id));
  scheduler_.evict_node(node_id);
  if (failure_cb_) failure_cb_(node_id);
}

int ClusterManager::leader() const {
  std::lock_guard<std::mutex> g(mu_);
  return leader_;
}

std::vector<NodeInfo> ClusterManager::nodes() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<NodeInfo> out;
  for (auto& kv : nodes_) out.push_back(kv.second);
  return out;
}

int ClusterManager::online_count() const {
  std::lock_guard<std::mutex> g(mu_);
  int n = 0;
  for (auto& kv : nodes_) n += kv.second.status == NodeStatus::ONLINE;
  return n;
}

bool ClusterManager::publish_region(int node_id, uint32_t region, const RegionDirectoryEntry& e) {
  return catalog_.upsert(static_cast<uint16_t>(node_id), region, e);
}
bool ClusterManager::lookup_region(int node_id, uint32_t region, RegionDirectoryEntry* out) const {
  return catalog_.lookup(static_cast<uint16_t>(node_id), region, out);
}

void ClusterManager::start() {
  if (running_.exchange(true)) return;
  sender_ = std::thread([this] { heartbeat_sender_loop(); });
  monitor_ = std::thread([this] { heartbeat_monitor_loop(); });
  sched_ = std::thread([this] { scheduler_loop(); });
}

void ClusterManager::stop() {
  if (!running_.exchange(false)) return;
  for (std::thread* t : {&sender_, &monitor_, &sched_})
    if (t->joinable()) t->join();
}

namespace {
void nap(std::atomic<bool>& running, int ms) {
  auto until = std::chrono::steady_clock::now() + std::chrono::milliseconds(ms);
  while (running && std::chrono::steady_clock::now() < until) std::this_thread::sleep_for(std::chrono::milliseconds(5));
}
}  // namespace

void ClusterManager::heartbeat_sender_loop() {
  while (running_) {
    for (auto& n : nodes()) {
      if (!running_) break;
      if (n.status == NodeStatus::OFFLINE || n.agent_port <= 0) continue;
      AgentReply r = agent_request(n.host, n.agent_port, AgentCmd::PING, {}, t_.ping_socket_timeout_ms);
      if (r.ok && r.status == AgentStatus::OK) handle_heartbeat(n.node_id);
    }
    nap(running_, t_.heartbeat_interval_ms);
  }
}

void ClusterManager::heartbeat_monitor_loop() {
  while (running_) {
    const double t = now();
    std::vector<int> dead;
    {
      std::lock_guard<std::mutex> g(mu_);
      for (auto& kv : nodes_)
        if (kv.second.status != NodeStatus::OFFLINE && kv.second.agent_port > 0 &&
            (t - kv.second.last_heartbeat) * 1000.0 > t_.heartbeat_timeout_ms)
          dead.push_back(kv.first);
    }
    for (int id : dead) handle_node_failure(id);
    nap(running_, t_.heartbeat_interval_ms);
  }
}

void ClusterManager::scheduler_loop() {
  while (running_) {
    std::vector<NodeLoad> loads;
    for (auto& n : nodes()) {
      NodeLoad l;
      l.node_id = n.node_id;
      l.online = n.status == NodeStatus::ONLINE;
      l.memory_total = n.memory_total;
      l.memory_used = n.memory_used;
      loads.push_back(l);
    }
    TickResult r = scheduler_.schedule_tick(loads);
    if (placement_cb_)
      for (auto& p : r.started) placement_cb_(p);
    nap(running_, t_.scheduler_tick_ms);
  }
}

}  // namespace mccl
