// Library lifetime (gpuOpsInit / gpuOpsDeinit), the reference's mgpuMatmul entry point on
// top of the tensor-core Gemm.
#include "ops_common.h"

namespace mdc {
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s);
}

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
MDC_API void mgpuMatmul(float *input, float *weight, float *bias, float *output, int64_t M, int64_t N,
                        int64_t K, void *stream) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) { fail("mgpuMatmul: K must be positive"); return; }
  if (!device_info().ok) return;
  const int64_t Kp = (K + 7) / 8 * 8;
  void *a16 = mgpuMemAllocAsync(static_cast<uint64_t>(M) * Kp * 2, stream);
  void *w16 = mgpuMemAllocAsync(static_cast<uint64_t>(N) * Kp * 2, stream);
  if (a16 && w16) {
    cast_rows_padded(input, a16, M, K, Kp, MGPU_DTYPE_F16, as_stream(stream));
    mgpuPackWeight(weight, w16, K, N, MGPU_DTYPE_F16, stream);
    mgpuMatmulEx16(a16, w16, bias, nullptr, output, M, N, Kp, MGPU_DTYPE_F16, MGPU_DTYPE_F32,
                   MGPU_ACT_NONE, stream);
  }
  if (a16) mgpuMemFreeAsync(a16, stream);
  if (w16) mgpuMemFreeAsync(w16, stream);
}
