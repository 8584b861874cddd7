// Helpers for the hand-written "lowered graph" modules.  Each module exports
// _mlir_ciface_main_graph and performs, in order, the runtime calls that the reference
// compiler's GPU pipeline emits for that graph: a data stream and a kernel stream linked
// by events (lib/Dialect/Device/Transform/AsyncDependencyConvert.cpp:45-139), device
// allocations and host->device copies of every operand
// (lib/Dialect/Device/Transform/DeviceDataCopyGeneration.cpp:26-70), the op call
// (lib/Conversion/ConvertDeviceToLLVM/ConvertDeviceToLLVM.cpp:410-455 or
// lib/Dialect/Device/IR/GPUOffloadingAttr.cpp:255-313 for generated kernels), the copy
// back, the frees and the stream teardown (ConvertDeviceToLLVM.cpp:337-358).  Shapes are
// read from the memref descriptors, so one module serves any batch size.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "mdc_gpu_ops.h"
#include "mdc_gpu_runtime.h"

template <int N>
struct MemRef {
  float *allocated;
  float *aligned;
  intptr_t offset;
  intptr_t sizes[N];
  intptr_t strides[N];
  int64_t count() const {
    int64_t n = 1;
    for (int i = 0; i < N; ++i) n *= sizes[i];
    return n;
  }
  float *data() const { return aligned + offset; }
};

// The callee owns the allocation of the result (64-byte aligned, examples/add.ll:9-23).
template <int N>
inline float *alloc_result(MemRef<N> *out, const intptr_t *sizes) {
  int64_t n = 1;
  for (int i = N - 1; i >= 0; --i) {
    out->sizes[i] = sizes[i];
    out->strides[i] = n;
    n *= sizes[i];
  }
  size_t bytes = (static_cast<size_t>(n) * sizeof(float) + 63) / 64 * 64;
  float *p = static_cast<float *>(aligned_alloc(64, bytes ? bytes : 64));
  out->allocated = out->aligned = p;
  out->offset = 0;
  return p;
}

struct GraphStreams {
  mgpu_stream_t data, kernel;
  mgpu_event_t data_ev, kernel_ev;
  GraphStreams() {
    data = mgpuStreamCreate();
    data_ev = mgpuEventCreateWithStream(data);
    kernel = mgpuStreamCreate();
    kernel_ev = mgpuEventCreateWithStream(kernel);
  }
  // device.record + device.wait: `to` continues after everything queued on `from`
  void data_to_kernel() { mgpuEventRecord(data_ev, data); mgpuStreamWaitEvent(kernel, data_ev); }
  void kernel_to_data() { mgpuEventRecord(kernel_ev, kernel); mgpuStreamWaitEvent(data, kernel_ev); }
  void end() {
    mgpuEventDestroy(data_ev);
    mgpuStreamSynchronize(data);
    mgpuStreamDestroy(data);
    mgpuEventDestroy(kernel_ev);
    mgpuStreamSynchronize(kernel);
    mgpuStreamDestroy(kernel);
  }
};

inline float *upload(const float *host, int64_t n, mgpu_stream_t s) {
  float *dev = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>(n) * sizeof(float), s));
  if (dev) mgpuMemcpy(dev, const_cast<float *>(host), static_cast<size_t>(n) * sizeof(float), s);
  return dev;
}

#define MDC_GRAPH_EXPORT extern "C" __attribute__((visibility("default")))
