#include "timeline.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "errors.hpp"
#include "../symm/cu_driver.hpp"

namespace mccl {

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
TimelineBuf* g_buf[kMaxDevices] = {};
int g_cap[kMaxDevices] = {};
bool g_on[kMaxDevices] = {};

int current_device() {
  int dev = 0;
  MCCL_CUDA_CHECK(cudaGetDevice(&dev));
  MCCL_CHECK(dev >= 0 && dev < kMaxDevices, "timeline: device index " << dev << " out of range");
  return dev;
}
}  // namespace

void timeline_enable(int capacity, int every, int detail) {
  const int dev = current_device();
  capacity = std::max(capacity, 64);
  every = std::max(every, 1);
  std::lock_guard<std::mutex> g(g_mu);
  if (g_buf[dev] != nullptr && g_cap[dev] < capacity) {
    MCCL_CUDA_CHECK(cudaDeviceSynchronize());
    MCCL_CUDA_CHECK(cudaFree(g_buf[dev]));
    g_buf[dev] = nullptr;
  }
  if (g_buf[dev] == nullptr) {
    void* p = nullptr;
    MCCL_CUDA_CHECK(cudaMalloc(&p, sizeof(TimelineBuf) + sizeof(TimelineRec) * static_cast<size_t>(capacity)));
    g_buf[dev] = static_cast<TimelineBuf*>(p);
    g_cap[dev] = capacity;
  }
  TimelineBuf head{};
  head.cap = static_cast<uint32_t>(g_cap[dev]);
  head.count = 0;
  head.every = static_cast<uint32_t>(every);
  head.detail = static_cast<uint32_t>(detail);
  MCCL_CUDA_CHECK(cudaMemcpy(g_buf[dev], &head, offsetof(TimelineBuf, rec), cudaMemcpyHostToDevice));
  g_on[dev] = true;
}

void timeline_disable() {
  const int dev = current_device();
  std::lock_guard<std::mutex> g(g_mu);
  g_on[dev] = false;  // the buffer stays: captured graphs may still hold its address
}

TimelineBuf* timeline_device_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  return g_on[dev] ? g_buf[dev] : nullptr;
}

std::vector<TimelineRec> timeline_drain() {
  const int dev = current_device();
  std::lock_guard<std::mutex> g(g_mu);
  std::vector<TimelineRec> out;
  if (g_buf[dev] == nullptr) return out;
  MCCL_CUDA_CHECK(cudaDeviceSynchronize());
  TimelineBuf head{};
  MCCL_CUDA_CHECK(cudaMemcpy(&head, g_buf[dev], offsetof(TimelineBuf, rec), cudaMemcpyDeviceToHost));
  const uint32_t n = std::min(head.count, head.cap);
  out.resize(n);
  if (n)
    MCCL_CUDA_CHECK(cudaMemcpy(out.data(), reinterpret_cast<char*>(g_buf[dev]) + offsetof(TimelineBuf, rec),
                               sizeof(TimelineRec) * n, cudaMemcpyDeviceToHost));
  const uint32_t zero = 0;
  MCCL_CUDA_CHECK(cudaMemcpy(reinterpret_cast<char*>(g_buf[dev]) + offsetof(TimelineBuf, count), &zero, sizeof(zero),
                             cudaMemcpyHostToDevice));
  std::sort(out.begin(), out.end(), [](const TimelineRec& a, const TimelineRec& b) { return a.t0 < b.t0; });
  return out;
}

}  // namespace mccl
