// Shared host-side helpers of the operator library: status reporting through the runtime
// library's sticky error, launch accounting, device queries and the element-type enum.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
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

// Launch helper for the kernels of the layer chain.  With programmatic dependent launch the
// front end may set the next kernel up (and start its CTAs on SMs the previous kernel has
// already left) while the previous kernel drains; each such kernel calls pdl_wait() (device,
// ptx_sm100.cuh / below) before it touches global memory, which orders it after the whole
// previous grid.  MDC_PDL=0 turns the attribute off (plain stream order).
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                int cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
// Blocks until the grid this one was made dependent on has completed and its writes are
// visible; returns at once for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the NEXT kernel of the chain be set up now: once every CTA of this grid has executed
// this (or exited), the dependent grid's CTAs are placed on whatever SM resources are free
// and run their prologue (barrier init, tensor-memory allocation, descriptor prefetch) up to
// their own pdl_wait(), which still holds them until this whole grid has finished and its
// writes are visible.  Called first thing in every chain kernel, so nothing of the next
// kernel's launch and set-up latency is left exposed between two kernels.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

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

// fp32 [R, C] -> 16-bit [R, Cp] with zero padding of the columns C..Cp (elementwise.cu)
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype, cudaStream_t s);

// Packed 16-bit [N, Kp] form of an fp32 [K, N] weight, from the constant cache when the weight
// is a copy of a registered constant (defined in ops_init.cu).
void *packed_weight(const float *w, int64_t K, int64_t N, int32_t dtype, void *stream, bool *cached);

// Device slot the tensor-core kernels write a non-zero code into when one of their bounded
// waits gives up; checked (and turned into the status) by mgpuOpsCheckDeviceStatus().
uint32_t *device_error_slot();

}  // namespace mdc

// Reads the device error slot (synchronises the stream); 0 = no kernel reported a problem.
MDC_API uint32_t mgpuOpsCheckDeviceStatus(void *stream);
