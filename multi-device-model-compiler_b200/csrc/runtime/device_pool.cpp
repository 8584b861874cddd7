#include "device_pool.h"

namespace mdc {

// Size classes: 512 B granules up to 1 MiB, 2 MiB granules above (the driver's own
// allocation granularity for large blocks), so freed blocks are reusable by near sizes.
size_t DevicePool::round_size(size_t bytes) {
  if (bytes == 0) bytes = 1;
  const size_t small = 512, large = size_t(2) << 20;
  if (bytes <= (size_t(1) << 20)) return (bytes + small - 1) / small * small;
  return (bytes + large - 1) / large * large;
}

cudaEvent_t DevicePool::take_event() {
  if (!spare_events_.empty()) {
    cudaEvent_t e = spare_events_.back();
    spare_events_.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  return e;
}

void *DevicePool::alloc(size_t bytes, cudaStream_t stream, cudaError_t *err) {
  *err = cudaSuccess;
  const size_t size = round_size(bytes);
  std::lock_guard<std::mutex> lock(mu_);
  // Best fit among cached blocks, but never waste more than half of a block.
  auto it = free_.lower_bound(size);
  if (it != free_.end() && it->first <= size * 2) {
    Block b = it->second;
    free_.erase(it);
    if (b.stream != stream && b.ready) {
      // ordered after the last use on the other stream, without blocking the host
      cudaError_t e = cudaStreamWaitEvent(stream, b.ready, 0);
      if (e != cudaSuccess) *err = e;
    }
    if (b.ready) {
      spare_events_.push_back(b.ready);
      b.ready = nullptr;
    }
    live_[b.ptr] = b;
    in_use_ += b.size;
    return b.ptr;
  }
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, size);
  if (e == cudaErrorMemoryAllocation) {
    (void)cudaGetLastError();
    // return every cached block to the driver and retry once
    for (auto &kv : free_) {
      if (kv.second.ready) {
        cudaEventSynchronize(kv.second.ready);
        spare_events_.push_back(kv.second.ready);
      }
      cudaFree(kv.second.ptr);
      reserved_ -= kv.second.size;
    }
    free_.clear();
    e = cudaMalloc(&p, size);
  }
  if (e != cudaSuccess) {
    *err = e;
    (void)cudaGetLastError();
    return nullptr;
  }
  Block b;
  b.ptr = p;
  b.size = size;
  b.stream = stream;
  live_[p] = b;
  reserved_ += size;
  in_use_ += size;
  return p;
}

bool DevicePool::free(void *ptr, cudaStream_t stream, cudaError_t *err) {
  *err = cudaSuccess;
  if (!ptr) return true;
  std::lock_guard<std::mutex> lock(mu_);
  auto it = live_.find(ptr);
  if (it == live_.end()) return false;
  Block b = it->second;
  live_.erase(it);
  b.stream = stream;
  b.ready = take_event();
  cudaError_t e = cudaEventRecord(b.ready, stream);
  if (e != cudaSuccess) *err = e;
  in_use_ -= b.size;
  free_.emplace(b.size, b);
  return true;
}

void DevicePool::trim() {
  std::lock_guard<std::mutex> lock(mu_);
  for (auto &kv : free_) {
    if (kv.second.ready) {
      cudaEventSynchronize(kv.second.ready);
      spare_events_.push_back(kv.second.ready);
    }
    cudaFree(kv.second.ptr);
    reserved_ -= kv.second.size;
  }
  free_.clear();
}

}  // namespace mdc
