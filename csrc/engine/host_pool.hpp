// Reusable host staging buffers.
//
// Parity: the reference's MemoryPool hands out page-aligned host buffers,
// reuses the best-fitting free one, over-allocates by 25 % (at most 256 MB of
// slack) to absorb slightly larger later requests, and wraps them in an RAII
// PooledBuffer (csrc/runtime/MemoryPool.cpp:25-126).  This pool does the same
// and can pin its buffers for DMA through a pair of hooks (the CUDA build
// installs cudaHostRegister / cudaHostUnregister); without hooks the buffers
// are plain aligned host memory, which is what the CPU-tensor path needs.
#pragma once

#include <cstddef>
#include <cstdlib>
#include <functional>
#include <mutex>
#include <vector>

#include "../core/errors.hpp"

namespace mccl {

class HostPool;

class PooledBuffer {
 public:
  PooledBuffer() = default;
  PooledBuffer(HostPool* pool, void* ptr, size_t capacity, size_t size)
      : pool_(pool), ptr_(ptr), capacity_(capacity), size_(size) {}
  PooledBuffer(PooledBuffer&& o) noexcept { *this = std::move(o); }
  PooledBuffer& operator=(PooledBuffer&& o) noexcept;
  PooledBuffer(const PooledBuffer&) = delete;
  PooledBuffer& operator=(const PooledBuffer&) = delete;
  ~PooledBuffer() { release(); }
  void release();
  void* data() const { return ptr_; }
  template <typename T>
  T* as() const { return static_cast<T*>(ptr_); }
  size_t size() const { return size_; }
  size_t capacity() const { return capacity_; }
  explicit operator bool() const { return ptr_ != nullptr; }

 private:
  HostPool* pool_ = nullptr;
  void* ptr_ = nullptr;
  size_t capacity_ = 0, size_ = 0;
};

class HostPool {
 public:
  using PinHook = std::function<bool(void*, size_t)>;
  using UnpinHook = std::function<void(void*)>;

  explicit HostPool(size_t alignment = 4096) : alignment_(alignment) {}
  ~HostPool() { trim(); }

  void set_pin_hooks(PinHook pin, UnpinHook unpin) {
    std::lock_guard<std::mutex> g(mu_);
    pin_ = std::move(pin);
    unpin_ = std::move(unpin);
  }

  PooledBuffer acquire(size_t nbytes) {
    if (nbytes == 0) nbytes = 1;
    std::lock_guard<std::mutex> g(mu_);
    // best fit among free blocks
    int best = -1;
    for (size_t i = 0; i < free_.size(); ++i)
      if (free_[i].cap >= nbytes && (best < 0 || free_[i].cap < free_[best].cap)) best = static_cast<int>(i);
    if (best >= 0) {
      Block b = free_[best];
      free_.erase(free_.begin() + best);
      ++hits_;
      return PooledBuffer(this, b.ptr, b.cap, nbytes);
    }
    size_t slack = nbytes / 4;
    if (slack > (size_t(256) << 20)) slack = size_t(256) << 20;
    size_t cap = round_up(nbytes + slack);
    void* p = nullptr;
    MCCL_CHECK(posix_memalign(&p, alignment_, cap) == 0 && p, "host pool: allocation of " << cap << " bytes failed");
    if (pin_ && !pin_(p, cap)) { /* unpinned buffers still work, only slower */ }
    ++misses_;
    allocated_ += cap;
    return PooledBuffer(this, p, cap, nbytes);
  }

  // Frees every cached block.
  void trim() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& b : free_) {
      if (unpin_) unpin_(b.ptr);
      std::free(b.ptr);
      allocated_ -= b.cap;
    }
    free_.clear();
  }

  size_t cached_blocks() const {
    std::lock_guard<std::mutex> g(mu_);
    return free_.size();
  }
  size_t allocated_bytes() const { return allocated_; }
  size_t hits() const { return hits_; }
  size_t misses() const { return misses_; }

  static HostPool& staging() {
    static HostPool pool(16384);
    return pool;
  }

 private:
  friend class PooledBuffer;
  struct Block {
    void* ptr;
    size_t cap;
  };
  size_t round_up(size_t n) const { return (n + alignment_ - 1) / alignment_ * alignment_; }
  void give_back(void* p, size_t cap) {
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back({p, cap});
  }
  size_t alignment_;
  mutable std::mutex mu_;
  std::vector<Block> free_;
  PinHook pin_;
  UnpinHook unpin_;
  size_t allocated_ = 0, hits_ = 0, misses_ = 0;
};

inline PooledBuffer& PooledBuffer::operator=(PooledBuffer&& o) noexcept {
  if (this != &o) {
    release();
    pool_ = o.pool_;
    ptr_ = o.ptr_;
    capacity_ = o.capacity_;
    size_ = o.size_;
    o.pool_ = nullptr;
    o.ptr_ = nullptr;
    o.capacity_ = o.size_ = 0;
  }
  return *this;
}

inline void PooledBuffer::release() {
  if (pool_ && ptr_) pool_->give_back(ptr_, capacity_);
  pool_ = nullptr;
  ptr_ = nullptr;
  capacity_ = size_ = 0;
}

}  // namespace mccl
