// Per-operation metrics with a percentile summary.
//
// Parity: the reference's Metrics class records, per op, a sequence number,
// name, byte count, start / execute-start / end stamps and sync / network /
// reduce phase times, keeps at most 10 000 records and summarises them into
// totals, avg / p50 / p99 latency, peak Gbps and phase averages
// (csrc/runtime/Metrics.hpp:14-111, Metrics.cpp:69-137).  Here the phases of
// a GPU collective are queue wait (submit → launch), device time (CUDA event
// pair around the kernels) and host time; CPU collectives keep the
// sync / network / reduce split.  Python reads the summary through
// mccl.get_metrics().
//
// Tracing: with MCCL_TRACE=<path> every finished op is appended to <path>.<pid>
// as one Chrome-trace event per line ({"name","ph":"X","ts","dur","pid","tid",
// "args":{bytes,algo,queue_wait_ms,device_ms,...}}), which chrome://tracing and
// Perfetto load after wrapping the lines in [ ].  With MCCL_NVTX=1 the same ops
// are bracketed by NVTX ranges (begin at submit, end at completion) so that they
// line up with the kernels in a timeline profiler.  The reference has only
// os_signpost calls for Instruments (csrc/metal/MPSInterop.mm:338-349).
#pragma once

#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace mccl {

struct OpMetric {
  uint64_t seq = 0;
  std::string name;
  std::string algo;
  uint64_t bytes = 0;
  double start_us = 0, execute_start_us = 0, end_us = 0;
  double sync_ms = 0, network_ms = 0, reduce_ms = 0, device_ms = 0;
  bool failed = false;
  uint64_t nvtx_id = 0;
  double latency_ms() const { return (end_us - start_us) / 1e3; }
  double queue_wait_ms() const { return (execute_start_us - start_us) / 1e3; }
  double execution_ms() const { return (end_us - execute_start_us) / 1e3; }
};

struct MetricsSummary {
  uint64_t total_ops = 0, total_bytes = 0, total_errors = 0;
  uint64_t transport_bytes_sent = 0, transport_bytes_received = 0;
  double avg_latency_ms = 0, p50_latency_ms = 0, p99_latency_ms = 0;
  double peak_gbps = 0;
  double avg_sync_ms = 0, avg_network_ms = 0, avg_reduce_ms = 0, avg_device_ms = 0;
  double avg_queue_wait_ms = 0, avg_execution_ms = 0;
  std::map<std::string, uint64_t> ops_by_name;
  std::map<std::string, uint64_t> bytes_by_algo;
};

class Metrics {
 public:
  static constexpr size_t kHistoryCap = 10000;

  static double now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
  }

  static Metrics& global() {
    static Metrics m;
    return m;
  }

  // Returns the sequence number of the new in-flight record.
  uint64_t op_start(const std::string& name, uint64_t bytes, const std::string& algo = "") {
    std::lock_guard<std::mutex> g(mu_);
    OpMetric m;
    m.seq = next_seq_++;
    m.name = name;
    m.algo = algo;
    m.bytes = bytes;
    m.start_us = m.execute_start_us = now_us();
    inflight_[m.seq] = m;
    if (nvtx_begin_) m.nvtx_id = nvtx_begin_(name.c_str());
    inflight_[m.seq].nvtx_id = m.nvtx_id;
    return m.seq;
  }
  // Installed by the CUDA side (the host-only build has no NVTX): begin returns a range id, end closes it.
  void set_nvtx(uint64_t (*begin)(const char*), void (*end)(uint64_t)) {
    std::lock_guard<std::mutex> g(mu_);
    nvtx_begin_ = begin;
    nvtx_end_ = end;
  }
  // Appends finished ops to `path`.<pid>; an empty path turns tracing off.
  void set_trace(const std::string& path) {
    std::lock_guard<std::mutex> g(mu_);
    if (trace_) {
      std::fclose(trace_);
      trace_ = nullptr;
    }
    if (!path.empty()) trace_ = std::fopen((path + "." + std::to_string(static_cast<long>(getpid()))).c_str(), "a");
  }
  void op_execute_start(uint64_t seq) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = inflight_.find(seq);
    if (it != inflight_.end()) it->second.execute_start_us = now_us();
  }
  // phase ∈ {"sync","network","reduce","device"}; times add up within an op.
  void record_phase(uint64_t seq, const char* phase, double ms) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = inflight_.find(seq);
    if (it == inflight_.end()) return;
    switch (phase[0]) {
      case 's': it->second.sync_ms += ms; break;
      case 'n': it->second.network_ms += ms; break;
      case 'r': it->second.reduce_ms += ms; break;
      default: it->second.device_ms += ms; break;
    }
  }
  void op_end(uint64_t seq, bool failed = false) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = inflight_.find(seq);
    if (it == inflight_.end()) return;
    it->second.end_us = now_us();
    it->second.failed = failed;
    if (failed) ++errors_;
    if (nvtx_end_ && it->second.nvtx_id) nvtx_end_(it->second.nvtx_id);
    if (!trace_checked_) {
      trace_checked_ = true;
      const char* tp = std::getenv("MCCL_TRACE");
      if (tp && *tp && !trace_) trace_ = std::fopen((std::string(tp) + "." + std::to_string(static_cast<long>(getpid()))).c_str(), "a");
    }
    if (trace_) {
      const OpMetric& m = it->second;
      std::fprintf(trace_,
                   "{\"name\":\"%s\",\"ph\":\"X\",\"ts\":%.3f,\"dur\":%.3f,\"pid\":%ld,\"tid\":0,\"args\":{\"seq\":%llu,\"bytes\":%llu,"
                   "\"algo\":\"%s\",\"queue_wait_ms\":%.4f,\"device_ms\":%.4f,\"sync_ms\":%.4f,\"network_ms\":%.4f,\"reduce_ms\":%.4f,"
                   "\"failed\":%s}},\n",
                   m.name.c_str(), m.start_us, m.end_us - m.start_us, static_cast<long>(getpid()),
                   static_cast<unsigned long long>(m.seq), static_cast<unsigned long long>(m.bytes), m.algo.c_str(), m.queue_wait_ms(),
                   m.device_ms, m.sync_ms, m.network_ms, m.reduce_ms, m.failed ? "true" : "false");
      std::fflush(trace_);
    }
    history_.push_back(it->second);
    if (history_.size() > kHistoryCap) history_.pop_front();
    ++total_ops_;
    total_bytes_ += it->second.bytes;
    inflight_.erase(it);
  }
  void record_transport_bytes(uint64_t sent, uint64_t received) {
    std::lock_guard<std::mutex> g(mu_);
    tx_ += sent;
    rx_ += received;
  }
  void record_error() {
    std::lock_guard<std::mutex> g(mu_);
    ++errors_;
  }
  void reset() {
    std::lock_guard<std::mutex> g(mu_);
    history_.clear();
    inflight_.clear();
    total_ops_ = total_bytes_ = errors_ = tx_ = rx_ = 0;
  }
  std::vector<OpMetric> history() const {
    std::lock_guard<std::mutex> g(mu_);
    return std::vector<OpMetric>(history_.begin(), history_.end());
  }

  MetricsSummary summarize() const {
    std::lock_guard<std::mutex> g(mu_);
    MetricsSummary s;
    s.total_ops = total_ops_;
    s.total_bytes = total_bytes_;
    s.total_errors = errors_;
    s.transport_bytes_sent = tx_;
    s.transport_bytes_received = rx_;
    if (history_.empty()) return s;
    std::vector<double> lat;
    lat.reserve(history_.size());
    for (auto& m : history_) {
      double l = m.latency_ms();
      lat.push_back(l);
      s.avg_latency_ms += l;
      s.avg_sync_ms += m.sync_ms;
      s.avg_network_ms += m.network_ms;
      s.avg_reduce_ms += m.reduce_ms;
      s.avg_device_ms += m.device_ms;
      s.avg_queue_wait_ms += m.queue_wait_ms();
      s.avg_execution_ms += m.execution_ms();
      double busy_ms = m.device_ms > 0 ? m.device_ms : m.execution_ms();
      if (busy_ms > 0 && m.bytes > 0) s.peak_gbps = std::max(s.peak_gbps, m.bytes * 8.0 / (busy_ms * 1e6));
      ++s.ops_by_name[m.name];
      if (!m.algo.empty()) s.bytes_by_algo[m.algo] += m.bytes;
    }
    double n = static_cast<double>(history_.size());
    s.avg_latency_ms /= n;
    s.avg_sync_ms /= n;
    s.avg_network_ms /= n;
    s.avg_reduce_ms /= n;
    s.avg_device_ms /= n;
    s.avg_queue_wait_ms /= n;
    s.avg_execution_ms /= n;
    std::sort(lat.begin(), lat.end());
    s.p50_latency_ms = lat[lat.size() / 2];
    s.p99_latency_ms = lat[std::min(lat.size() - 1, static_cast<size_t>(lat.size() * 0.99))];
    return s;
  }

 private:
  mutable std::mutex mu_;
  uint64_t next_seq_ = 1;
  std::map<uint64_t, OpMetric> inflight_;
  std::deque<OpMetric> history_;
  uint64_t total_ops_ = 0, total_bytes_ = 0, errors_ = 0, tx_ = 0, rx_ = 0;
  std::FILE* trace_ = nullptr;
  bool trace_checked_ = false;
  uint64_t (*nvtx_begin_)(const char*) = nullptr;
  void (*nvtx_end_)(uint64_t) = nullptr;
};

}  // namespace mccl
