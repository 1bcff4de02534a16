#include "progress.hpp"

#include <pthread.h>

#include <stdexcept>

#include "../core/log.hpp"
#include "metrics.hpp"

namespace mccl {

Progress::Progress(size_t max_queue_depth, const char* thread_name)
    : max_depth_(max_queue_depth ? max_queue_depth : 1), worker_([this, thread_name] { run(thread_name); }) {}

Progress::~Progress() { shutdown(); }

uint64_t Progress::submit(std::function<void()> fn) {
  ProgressTask t;
  t.name = "task";
  t.execute = std::move(fn);
  return submit(std::move(t));
}

uint64_t Progress::submit(ProgressTask task) {
  std::unique_lock<std::mutex> g(mu_);
  cv_space_.wait(g, [&] { return stopping_ || queue_.size() < max_depth_; });
  if (stopping_) {
    g.unlock();
    if (task.on_error)
      task.on_error(std::make_exception_ptr(std::runtime_error("mccl: progress engine is shut down")));
    return 0;
  }
  uint64_t seq = next_seq_.fetch_add(1);
  queue_.push_back(Slot{seq, std::move(task)});
  g.unlock();
  cv_work_.notify_one();
  return seq;
}

size_t Progress::depth() const {
  std::lock_guard<std::mutex> g(mu_);
  return queue_.size();
}

void Progress::drain() {
  std::unique_lock<std::mutex> g(mu_);
  cv_idle_.wait(g, [&] { return queue_.empty() && !busy_; });
}

void Progress::shutdown() {
  {
    std::lock_guard<std::mutex> g(mu_);
    if (stopping_ && !worker_.joinable()) return;
    stopping_ = true;
  }
  cv_work_.notify_all();
  cv_space_.notify_all();
  if (worker_.joinable()) {
    if (worker_.get_id() == std::this_thread::get_id())
      worker_.detach();
    else
      worker_.join();
  }
}

void Progress::run(const char* thread_name) {
  pthread_setname_np(pthread_self(), thread_name);
  for (;;) {
    Slot slot;
    {
      std::unique_lock<std::mutex> g(mu_);
      cv_work_.wait(g, [&] { return stopping_ || !queue_.empty(); });
      if (queue_.empty()) {
        // stopping_ and nothing left: the queue has been drained.
        cv_idle_.notify_all();
        return;
      }
      slot = std::move(queue_.front());
      queue_.pop_front();
      busy_ = true;
    }
    cv_space_.notify_one();
    ProgressTask& t = slot.task;
    if (t.metric_seq) Metrics::global().op_execute_start(t.metric_seq);
    bool failed = false;
    try {
      if (t.execute) t.execute();
      if (t.on_complete) t.on_complete();
    } catch (...) {
      failed = true;
      if (t.on_error) {
        try {
          t.on_error(std::current_exception());
        } catch (...) {
          MCCL_ERROR("progress: on_error callback of '" << t.name << "' threw");
        }
      } else {
        MCCL_WARN("progress: task '" << t.name << "' (seq " << slot.seq << ") threw and has no error callback");
      }
    }
    if (t.metric_seq) Metrics::global().op_end(t.metric_seq, failed);
    completed_.fetch_add(1);
    {
      std::lock_guard<std::mutex> g(mu_);
      busy_ = false;
      if (queue_.empty()) cv_idle_.notify_all();
    }
  }
}

}  // namespace mccl
