/* C++-linkage entry points of libMultiDeviceGPUOps.so: the reference declares these as
 * function templates (include/multi-device-model-compiler/Kernels/GPU/Ops.h:15-20,51-74 and
 * Kernels/GPU/Utils.h:6-8) and instantiates them for the listed types; other translation units
 * of the reference (lib/Kernels/GPU/LLM.cu) call them by their mangled names.  The library
 * exports the same instantiations:
 *   mgpuMatmulEx<half>, mgpuMatmulEx<float>          Ops.h:51-55   (lib/Kernels/GPU/Ops.cu:136-234)
 *   mgpuLayerNorm<half>                              Ops.h:57-61   (LayerNorm.cu:410-436)
 *   mgpuAddResidualPreLayerNorm<half>                Ops.h:63-68   (LayerNorm.cu:438-466)
 *   mgpuAddFusedQKVBiasTranspose<half>               Ops.h:70-74   (Transpose.cu:72-85)
 *   invokeCudaCast<half, float>, <float, half>       Utils.h:6-8   (Utils.cu:38-103)
 *   gpuOpsInit / gpuOpsDeinit / gpuLLMOpsInit / gpuLLMOpsDeinit / checkCudaStatus   Ops.h:15-20
 * Differences: nothing throws (failures set the sticky status, mgpuGetLastError);
 * mgpuMatmulEx refuses ReLU combined with a residual; mgpuMatmulEx<half> needs K % 8 == 0. */
#ifndef MDC_GPU_OPS_CXX_H_
#define MDC_GPU_OPS_CXX_H_

#include <cstddef>
#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

void gpuOpsInit();
void gpuOpsDeinit();
void gpuLLMOpsInit();
void gpuLLMOpsDeinit();
void checkCudaStatus(cudaError_t status);

template <typename T>
void mgpuMatmulEx(T *input, T *weight, T *bias, T *output, T *residual, int64_t M, int64_t N, int64_t K,
                  bool hasBias, bool hasRelu, bool hasResidual, cudaStream_t stream);

template <typename T>
void mgpuLayerNorm(const T *input, const T *gamma, const T *beta, T *output, const float layernorm_eps,
                   const int m, const int n, float *scale, cudaStream_t stream);

template <typename T>
void mgpuAddResidualPreLayerNorm(const T *input, const T *residual, const T *gamma, const T *beta, T *output,
                                 T *normed_output, const float layernorm_eps, int m, int n, float *scale,
                                 cudaStream_t stream);

template <typename T>
void mgpuAddFusedQKVBiasTranspose(T *q_buf, T *k_buf, T *v_buf, T *QKV, const T *qkv_bias, const int batch_size,
                                  const int seq_len, const int token_num, const int head_num,
                                  const int size_per_head, cudaStream_t stream);

template <typename T_OUT, typename T_IN>
void invokeCudaCast(T_OUT *dst, T_IN const *const src, const size_t size, cudaStream_t stream);

#endif
