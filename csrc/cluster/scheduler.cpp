#include "scheduler.hpp"

#include <algorithm>

namespace mccl {

namespace {
double steady_seconds() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

const char* job_state_name(JobState s) {
  static const char* n[] = {"PENDING", "RUNNING", "COMPLETED", "FAILED", "RESCHEDULING", "CANCELLED"};
  return n[static_cast<int>(s)];
}
const char* job_priority_name(JobPriority p) {
  static const char* n[] = {"LOW", "NORMAL", "HIGH", "CRITICAL"};
  return n[static_cast<int>(p)];
}

Scheduler::Scheduler(Clock clock) : clock_(clock ? clock : &steady_seconds) {}

double Scheduler::now() const { return clock_(); }

uint64_t Scheduler::submit(const JobSpec& spec) {
  std::lock_guard<std::mutex> g(mu_);
  Job j;
  j.id = next_id_++;
  j.spec = spec;
  if (j.spec.nodes_required < 1) j.spec.nodes_required = 1;
  j.submit_seq = next_seq_++;
  j.submitted_at = now();
  jobs_[j.id] = j;
  pending_.push_back(j.id);
  return j.id;
}

void Scheduler::account(Job& j, double until) {
  if (j.state == JobState::RUNNING && j.started_at > 0)
    usage_[j.spec.tenant] += (until - j.started_at) * static_cast<double>(j.nodes.size());
}

bool Scheduler::cancel(uint64_t id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = jobs_.find(id);
  if (it == jobs_.end()) return false;
  Job& j = it->second;
  if (j.state == JobState::COMPLETED || j.state == JobState::FAILED || j.state == JobState::CANCELLED) return false;
  const double t = now();
  account(j, t);
  j.state = JobState::CANCELLED;
  j.finished_at = t;
  pending_.erase(std::remove(pending_.begin(), pending_.end(), id), pending_.end());
  return true;
}

bool Scheduler::complete(uint64_t id, bool ok, const std::string& reason) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = jobs_.find(id);
  if (it == jobs_.end() || it->second.state != JobState::RUNNING) return false;
  Job& j = it->second;
  const double t = now();
  account(j, t);
  j.state = ok ? JobState::COMPLETED : JobState::FAILED;
  j.finished_at = t;
  j.reason = reason;
  return true;
}

uint64_t Scheduler::reserved_on(int node) const {
  uint64_t r = 0;
  for (auto& kv : jobs_)
    if (kv.second.state == JobState::RUNNING &&
        std::find(kv.second.nodes.begin(), kv.second.nodes.end(), node) != kv.second.nodes.end())
      r += kv.second.spec.memory_per_node;
  return r;
}

int Scheduler::effective_priority(const Job& j, double total_usage, double total_weight) const {
  int p = static_cast<int>(j.spec.priority);
  if (j.spec.priority == JobPriority::LOW && total_usage > 0) {
    auto wi = weight_.find(j.spec.tenant);
    const double w = wi == weight_.end() ? 1.0 : wi->second;
    auto ui = usage_.find(j.spec.tenant);
    const double used = ui == usage_.end() ? 0.0 : ui->second;
    // below its fair share of what has been consumed so far: treat as NORMAL
    if (used < total_usage * (w / total_weight)) p = static_cast<int>(JobPriority::NORMAL);
  }
  return p;
}

TickResult Scheduler::schedule_tick(const std::vector<NodeLoad>& nodes) {
  std::lock_guard<std::mutex> g(mu_);
  TickResult res;
  const double t = now();

  double total_usage = 0, total_weight = 0;
  std::map<std::string, bool> tenants;
  for (auto& kv : jobs_) tenants[kv.second.spec.tenant] = true;
  for (auto& kv : usage_) total_usage += kv.second;
  for (auto& kv : tenants) {
    auto wi = weight_.find(kv.first);
    total_weight += wi == weight_.end() ? 1.0 : wi->second;
  }
  if (total_weight <= 0) total_weight = 1;

  // Dispatch order: requeued jobs keep their place at the front; the rest by
  // effective priority (high first), then first come first served.
  std::vector<uint64_t> order(pending_.begin(), pending_.end());
  std::stable_sort(order.begin(), order.end(), [&](uint64_t a, uint64_t b) {
    const Job& ja = jobs_.at(a);
    const Job& jb = jobs_.at(b);
    const bool ra = ja.state == JobState::RESCHEDULING, rb = jb.state == JobState::RESCHEDULING;
    if (ra != rb) return ra;
    const int pa = effective_priority(ja, total_usage, total_weight), pb = effective_priority(jb, total_usage, total_weight);
    if (pa != pb) return pa > pb;
    return ja.submit_seq < jb.submit_seq;
  });

  // Free memory per online node after what running jobs have reserved.
  std::map<int, int64_t> free_mem;
  for (auto& n : nodes)
    if (n.online)
      free_mem[n.node_id] = static_cast<int64_t>(n.memory_total) - static_cast<int64_t>(n.memory_used) -
                            static_cast<int64_t>(reserved_on(n.node_id));

  auto try_place = [&](const Job& j, std::vector<int>* out) {
    out->clear();
    for (auto& kv : free_mem) {
      if (kv.second >= static_cast<int64_t>(j.spec.memory_per_node)) out->push_back(kv.first);
      if (static_cast<int>(out->size()) == j.spec.nodes_required) return true;
    }
    return false;
  };
  auto start = [&](Job& j, const std::vector<int>& where) {
    j.state = JobState::RUNNING;
    j.nodes = where;
    j.started_at = t;
    for (int n : where) free_mem[n] -= static_cast<int64_t>(j.spec.memory_per_node);
    pending_.erase(std::remove(pending_.begin(), pending_.end(), j.id), pending_.end());
    res.started.push_back({j.id, where});
  };

  for (uint64_t id : order) {
    Job& j = jobs_.at(id);
    std::vector<int> where;
    if (try_place(j, &where)) {
      start(j, where);
      continue;
    }
    // HIGH and CRITICAL jobs may push LOW jobs back to the queue.
    if (j.spec.priority >= JobPriority::HIGH) {
      std::vector<uint64_t> victims;
      for (auto& kv : jobs_)
        if (kv.second.state == JobState::RUNNING && kv.second.spec.priority == JobPriority::LOW) victims.push_back(kv.first);
      // youngest first: the least work is lost
      std::sort(victims.begin(), victims.end(), [&](uint64_t a, uint64_t b) { return jobs_.at(a).started_at > jobs_.at(b).started_at; });
      std::vector<uint64_t> taken;
      for (uint64_t v : victims) {
        Job& vj = jobs_.at(v);
        for (int n : vj.nodes)
          if (free_mem.count(n)) free_mem[n] += static_cast<int64_t>(vj.spec.memory_per_node);
        taken.push_back(v);
        if (try_place(j, &where)) break;
      }
      if (!where.empty() && static_cast<int>(where.size()) == j.spec.nodes_required) {
        for (uint64_t v : taken) {
          Job& vj = jobs_.at(v);
          account(vj, t);
          vj.state = JobState::PENDING;
          vj.nodes.clear();
          vj.started_at = 0;
          ++vj.preemptions;
          vj.reason = "preempted by job " + std::to_string(j.id);
          pending_.push_back(v);
          res.preempted.push_back(v);
        }
        start(j, where);
      } else {
        // could not make room: give the memory back on paper
        for (uint64_t v : taken)
          for (int n : jobs_.at(v).nodes)
            if (free_mem.count(n)) free_mem[n] -= static_cast<int64_t>(jobs_.at(v).spec.memory_per_node);
      }
    }
  }
  return res;
}

std::vector<uint64_t> Scheduler::evict_node(int node_id) {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<uint64_t> touched;
  const double t = now();
  for (auto& kv : jobs_) {
    Job& j = kv.second;
    if (j.state != JobState::RUNNING) continue;
    if (std::find(j.nodes.begin(), j.nodes.end(), node_id) == j.nodes.end()) continue;
    account(j, t);
    if (j.nodes.size() <= 1) {
      j.state = JobState::FAILED;
      j.finished_at = t;
      j.reason = "node " + std::to_string(node_id) + " went offline";
    } else {
      j.state = JobState::RESCHEDULING;
      j.reason = "node " + std::to_string(node_id) + " went offline; requeued";
      j.nodes.clear();
      j.started_at = 0;
      pending_.push_front(j.id);
    }
    touched.push_back(j.id);
  }
  return touched;
}

bool Scheduler::get(uint64_t id, Job* out) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = jobs_.find(id);
  if (it == jobs_.end()) return false;
  *out = it->second;
  return true;
}

std::vector<Job> Scheduler::jobs() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<Job> out;
  for (auto& kv : jobs_) out.push_back(kv.second);
  return out;
}

std::vector<Job> Scheduler::queue() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<Job> out;
  for (uint64_t id : pending_) out.push_back(jobs_.at(id));
  return out;
}

double Scheduler::tenant_node_seconds(const std::string& tenant) const {
  std::lock_guard<std::mutex> g(mu_);
  double u = 0;
  auto it = usage_.find(tenant);
  if (it != usage_.end()) u = it->second;
  const double t = now();
  for (auto& kv : jobs_)
    if (kv.second.state == JobState::RUNNING && kv.second.spec.tenant == tenant)
      u += (t - kv.second.started_at) * static_cast<double>(kv.second.nodes.size());
  return u;
}

void Scheduler::set_tenant_weight(const std::string& tenant, double weight) {
  std::lock_guard<std::mutex> g(mu_);
  weight_[tenant] = weight;
}

size_t Scheduler::running_count() const {
  std::lock_guard<std::mutex> g(mu_);
  size_t n = 0;
  for (auto& kv : jobs_) n += kv.second.state == JobState::RUNNING;
  return n;
}

}  // namespace mccl
