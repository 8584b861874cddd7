// Library lifetime (gpuOpsInit / gpuOpsDeinit), the reference's mgpuMatmul entry point on
// top of the tensor-core Gemm.
#include "ops_common.h"

namespace mdc {
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s);
}

namespace mdc {
// The packed ([N, Kp], 16-bit) form of the fp32 weight w [K, N] on `stream`.  *cached = true:
// the buffer belongs to the constant cache (w is a copy of a registered constant; packed at
// the first use, reused afterwards) and must not be freed; false: a pool block the caller
// frees after its last use.  nullptr when out of memory.
void *packed_weight(const float *w, int64_t K, int64_t N, int32_t dtype, void *stream, bool *cached) {
  *cached = false;
  const int64_t Kp = (K + 7) / 8 * 8;
  const uint64_t bytes = static_cast<uint64_t>(N) * Kp * 2;
  if (const void *key = mgpuConstantSourceOf(w)) {
    // one packed form per (shape, element type) of a constant
    const uint64_t tag = (static_cast<uint64_t>(K) * 0x9E3779B97F4A7C15ull) ^ (static_cast<uint64_t>(N) << 20) ^
                         (static_cast<uint64_t>(dtype) << 60) ^ 0x5041434bull;
    int32_t needs_fill = 0;
    if (void *buf = mgpuConstantDerived(key, tag, bytes, stream, &needs_fill)) {
      if (needs_fill) {
        mgpuPackWeight(w, buf, K, N, dtype, stream);
        mgpuConstantDerivedReady(key, tag, stream);
      }
      *cached = true;
      return buf;
    }
  }
  void *buf = mgpuMemAllocAsync(bytes, stream);
  if (buf) mgpuPackWeight(w, buf, K, N, dtype, stream);
  return buf;
}
}  // namespace mdc

using namespace mdc;

// ---- lifetime: lib/Kernels/GPU/Ops.cu:43-55, lib/Kernels/GPU/LLM.cu:14-24 ----
// The reference creates a cuBLASLt handle, a 16 MiB workspace, a cuDNN handle and a copy
// stream here.  This library keeps no library handles: init only checks that the device
// is a B200-class GPU and allocates the 4-byte device status word.
MDC_API int32_t mgpuOpsInit(void) {
  if (!device_info().ok) return -1;
  return device_error_slot() ? 0 : -1;
}
MDC_API void mgpuOpsDeinit(void) {}

MDC_CXX_API void gpuOpsInit() { mgpuOpsInit(); }
MDC_CXX_API void gpuOpsDeinit() { mgpuOpsDeinit(); }
MDC_CXX_API void gpuLLMOpsInit() {}
MDC_CXX_API void gpuLLMOpsDeinit() {}
// include/multi-device-model-compiler/Kernels/GPU/Ops.h:20; the reference throws
// std::logic_error (Ops.cu:21-27), this one records the status and returns.
MDC_CXX_API void checkCudaStatus(cudaError_t status) { check_cuda(status, "checkCudaStatus"); }

// ---- mgpuMatmul: fp32 at the boundary, fp16 tensor-core math, fp32 accumulate ----
// input [M,K] and weight [K,N] are converted on every call (the caller may have rewritten
// them since the last one): input by a cast, weight by the cast + transpose that gives the
// Gemm its K-contiguous operand.  Scratch comes from the runtime's device pool.
// Exception: a weight buffer that the runtime knows to be an unmodified copy of a registered
// constant (mgpuRegisterConstant + mgpuMemcpy, what a lowered graph does with its weights on
// every call) is packed once; the packed copy lives with the registration.
MDC_API void mgpuMatmul(float *input, float *weight, float *bias, float *output, int64_t M, int64_t N,
                        int64_t K, void *stream) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) { fail("mgpuMatmul: K must be positive"); return; }
  if (!device_info().ok) return;
  const int64_t Kp = (K + 7) / 8 * 8;
  void *a16 = mgpuMemAllocAsync(static_cast<uint64_t>(M) * Kp * 2, stream);
  bool w_cached = false;
  void *w16 = packed_weight(weight, K, N, MGPU_DTYPE_F16, stream, &w_cached);
  if (a16 && w16) {
    cast_rows_padded(input, a16, M, K, Kp, MGPU_DTYPE_F16, as_stream(stream));
    mgpuMatmulEx16(a16, w16, bias, nullptr, output, M, N, Kp, MGPU_DTYPE_F16, MGPU_DTYPE_F32,
                   MGPU_ACT_NONE, stream);
  }
  if (a16) mgpuMemFreeAsync(a16, stream);
  if (w16 && !w_cached) mgpuMemFreeAsync(w16, stream);
}
