// Multi-tenant job scheduler of the cluster manager (host only, no GPU calls).
//
// Parity: the reference's Scheduler has priorities LOW..CRITICAL, job states
// PENDING / RUNNING / COMPLETED / FAILED / RESCHEDULING, submit / cancel /
// complete, a schedule_tick that orders by priority then first-come-first-
// served, bumps LOW jobs of tenants that are below their fair share to NORMAL,
// places first-fit by per-node free memory, lets HIGH and CRITICAL jobs
// preempt LOW ones, evict_node that fails single-node jobs and requeues
// multi-node jobs at the front, and node-seconds accounting per tenant
// (csrc/runtime/Scheduler.hpp:12-104, Scheduler.cpp:29-281).  A "node" here is
// one GPU rank of the box.
#pragma once

#include <chrono>
#include <cstdint>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace mccl {

enum class JobPriority : int { LOW = 0, NORMAL = 1, HIGH = 2, CRITICAL = 3 };
enum class JobState : int { PENDING = 0, RUNNING, COMPLETED, FAILED, RESCHEDULING, CANCELLED };

const char* job_state_name(JobState s);
const char* job_priority_name(JobPriority p);

struct JobSpec {
  std::string name;
  std::string tenant = "default";
  JobPriority priority = JobPriority::NORMAL;
  int nodes_required = 1;
  uint64_t memory_per_node = 0;  // bytes
  std::string command;           // opaque to the scheduler
};

struct Job {
  uint64_t id = 0;
  JobSpec spec;
  JobState state = JobState::PENDING;
  std::vector<int> nodes;        // where it runs (RUNNING) or last ran
  uint64_t submit_seq = 0;       // FCFS order
  double submitted_at = 0, started_at = 0, finished_at = 0;  // seconds, scheduler clock
  int preemptions = 0;
  std::string reason;            // why it failed / was requeued
};

struct NodeLoad {
  int node_id = 0;
  bool online = true;
  uint64_t memory_total = 0;
  uint64_t memory_used = 0;      // by things the scheduler does not know about
};

struct Placement {
  uint64_t job_id = 0;
  std::vector<int> nodes;
};

struct TickResult {
  std::vector<Placement> started;
  std::vector<uint64_t> preempted;  // jobs moved back to the queue to make room
};

class Scheduler {
 public:
  using Clock = double (*)();  // seconds; injectable for tests
  explicit Scheduler(Clock clock = nullptr);

  uint64_t submit(const JobSpec& spec);
  bool cancel(uint64_t id);
  // Marks a RUNNING job COMPLETED (ok) or FAILED.
  bool complete(uint64_t id, bool ok, const std::string& reason = "");
  TickResult schedule_tick(const std::vector<NodeLoad>& nodes);
  // Node went away: single-node jobs on it fail, multi-node jobs are requeued first in line.
  std::vector<uint64_t> evict_node(int node_id);

  bool get(uint64_t id, Job* out) const;
  std::vector<Job> jobs() const;           // every known job, by id
  std::vector<Job> queue() const;          // pending jobs in dispatch order
  double tenant_node_seconds(const std::string& tenant) const;
  // Share a tenant is entitled to (weights default to 1).
  void set_tenant_weight(const std::string& tenant, double weight);
  size_t running_count() const;

 private:
  double now() const;
  void account(Job& j, double until);
  int effective_priority(const Job& j, double total_usage, double total_weight) const;
  uint64_t reserved_on(int node) const;

  Clock clock_;
  mutable std::mutex mu_;
  uint64_t next_id_ = 1, next_seq_ = 1;
  std::map<uint64_t, Job> jobs_;
  std::deque<uint64_t> pending_;           // ids; requeued jobs are pushed to the front
  std::map<std::string, double> usage_;    // tenant → node-seconds
  std::map<std::string, double> weight_;
};

}  // namespace mccl
