// FIFO progress engine.
//
// Role: runs host-side collective bodies (TCP transfers, CPU reductions)
// strictly in submission order on one worker thread, so that every rank
// consumes the per-peer byte streams in the same order.  Parity: the
// reference ships a single-thread unbounded FIFO whose shutdown drains the
// queue (csrc/backend/Progress.cpp:15-42) and an older engine with a bounded
// queue, sequence numbers, completion/error callbacks and a metrics hook
// (csrc/runtime/ProgressEngine.cpp:46-153); this class merges the two.  An
// exception thrown by a task goes to its on_error callback and does not stop
// the worker.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <exception>
#include <functional>
#include <mutex>
#include <string>
#include <thread>

namespace mccl {

struct ProgressTask {
  std::string name;
  uint64_t bytes = 0;
  std::function<void()> execute;
  std::function<void()> on_complete;                    // optional
  std::function<void(std::exception_ptr)> on_error;     // optional
  uint64_t metric_seq = 0;                              // 0 = not tracked
};

class Progress {
 public:
  explicit Progress(size_t max_queue_depth = 1024, const char* thread_name = "mccl_engine");
  ~Progress();
  Progress(const Progress&) = delete;
  Progress& operator=(const Progress&) = delete;

  // Enqueues and returns the task's engine sequence number.  Blocks while the
  // queue holds max_queue_depth tasks.  After shutdown the task is rejected
  // through its on_error callback.
  uint64_t submit(ProgressTask task);
  // Shorthand for fire-and-forget work.
  uint64_t submit(std::function<void()> fn);

  // Blocks until every task submitted so far has finished.
  void drain();
  // Idempotent; runs what is already queued, then joins the worker.
  void shutdown();

  uint64_t submitted() const { return next_seq_.load() - 1; }
  uint64_t completed() const { return completed_.load(); }
  size_t depth() const;

 private:
  void run(const char* thread_name);
  struct Slot {
    uint64_t seq;
    ProgressTask task;
  };
  const size_t max_depth_;
  mutable std::mutex mu_;
  std::condition_variable cv_work_, cv_space_, cv_idle_;
  std::deque<Slot> queue_;
  bool stopping_ = false;
  bool busy_ = false;
  std::atomic<uint64_t> next_seq_{1};
  std::atomic<uint64_t> completed_{0};
  std::thread worker_;
};

}  // namespace mccl
