// Shared host-side helpers of the operator library: status reporting through the runtime
// library's sticky error, launch accounting, device queries and the element-type enum.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "mdc_gpu_ops.h"
#include "mdc_gpu_runtime.h"

#define MDC_API extern "C" __attribute__((visibility("default")))
#define MDC_CXX_API __attribute__((visibility("default")))

namespace mdc {

extern std::atomic<uint64_t> g_launch_count;

inline bool check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return true;
  char msg[256];
  snprintf(msg, sizeof(msg), "%s: %s", what, cudaGetErrorName(e));
  mgpuSetLastError(static_cast<int32_t>(e), msg);
  (void)cudaGetLastError();
  return false;
}

inline void fail(const char *what) { mgpuSetLastError(-1, what); }

// Call after every <<<>>> launch: counts it and turns a launch failure into the status.
inline bool launched(const char *what) {
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return check_cuda(cudaGetLastError(), what);
}

struct DeviceInfo {
  int device = -1;
  int sms = 0;
  int cc_major = 0, cc_minor = 0;
  bool ok = false;
};
// Properties of the current device; ok == false (with the status set) if there is no
// usable CUDA device or it is not compute capability 10.x.
const DeviceInfo &device_info();

inline size_t dtype_size(int32_t dtype) { return dtype == MGPU_DTYPE_F32 ? 4 : 2; }
inline bool dtype_is16(int32_t dtype) { return dtype == MGPU_DTYPE_F16 || dtype == MGPU_DTYPE_BF16; }

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// Optional per-launch timing: while profiling is on (mgpuOpsProfileBegin), every launch
// site brackets its kernel with two CUDA events on the launching stream; mgpuOpsProfileEnd
// sums the elapsed times per kernel category.  Off by default (no events, no overhead).
enum ProfileCategory : int { kCatGemm = 0, kCatAttention = 1, kCatLayerNorm = 2, kCatElementwise = 3, kNumCategories = 4 };
extern bool g_profiling;
void profile_mark(int category, cudaStream_t stream, bool begin);
struct ProfileScope {
  int cat;
  cudaStream_t stream;
  ProfileScope(int c, cudaStream_t s) : cat(c), stream(s) {
    if (g_profiling) profile_mark(cat, stream, true);
  }
  ~ProfileScope() {
    if (g_profiling) profile_mark(cat, stream, false);
  }
};

// Device slot the tensor-core kernels write a non-zero code into when one of their bounded
// waits gives up; checked (and turned into the status) by mgpuOpsCheckDeviceStatus().
uint32_t *device_error_slot();

}  // namespace mdc

// Reads the device error slot (synchronises the stream); 0 = no kernel reported a problem.
MDC_API uint32_t mgpuOpsCheckDeviceStatus(void *stream);
