// Caching, stream-ordered device memory pool behind mgpuMemAlloc / mgpuMemFree[Async].
//
// The reference allocates with a synchronous cuMemAlloc / cuMemFree on every call of a
// lowered graph (lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:204-213) and its fused layer
// issues about twenty cuMemAllocAsync per call (lib/Kernels/GPU/LLM.cu:35-154).  Here blocks
// are cached by size class and handed back without touching the driver.  A free records an
// event on the freeing stream; a later allocation on a different stream makes that stream
// wait for the event before the block is reused, so reuse is always ordered after the last
// use without any host synchronisation.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace mdc {

class DevicePool {
public:
  // Returns nullptr (and leaves *err set) when the driver is out of memory even after
  // every cached block has been returned to it.
  void *alloc(size_t bytes, cudaStream_t stream, cudaError_t *err);
  // Returns false if ptr did not come from this pool.
  bool free(void *ptr, cudaStream_t stream, cudaError_t *err);
  void trim();
  uint64_t reserved_bytes() const { return reserved_; }
  uint64_t in_use_bytes() const { return in_use_; }

  static size_t round_size(size_t bytes);

private:
  struct Block {
    void *ptr = nullptr;
    size_t size = 0;
    cudaStream_t stream = nullptr;  // stream of the last free
    cudaEvent_t ready = nullptr;    // recorded at the last free
  };
  cudaEvent_t take_event();

  std::mutex mu_;
  std::multimap<size_t, Block> free_;          // size -> cached block
  std::unordered_map<void *, Block> live_;     // blocks handed out
  std::vector<cudaEvent_t> spare_events_;
  uint64_t reserved_ = 0;
  uint64_t in_use_ = 0;
};

}  // namespace mdc
