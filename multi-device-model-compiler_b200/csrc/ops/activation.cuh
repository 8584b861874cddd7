// Activation functions shared by the elementwise kernels and the Gemm epilogue.
// ReLU is what the reference layer applies (lib/Kernels/GPU/LLM.cu:119-121, epilogue
// RELU_BIAS of lib/Kernels/GPU/Ops.cu:152-159); GELU in its exact erf form and in the tanh
// approximation are additions for the encoder configurations.
#pragma once

#include <cuda_runtime.h>

namespace mdc {

enum : int { kActNone = 0, kActRelu = 1, kActGeluErf = 2, kActGeluTanh = 3 };

__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
  case kActRelu:
    return v > 0.f ? v : 0.f;
  case kActGeluErf:
    return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
  case kActGeluTanh: {
    const float u = 0.79788456080286535588f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(u));
  }
  default:
    return v;
  }
}

template <int ACT>
__device__ __forceinline__ float act_apply_t(float v) {
  return act_apply(v, ACT);
}

}  // namespace mdc
