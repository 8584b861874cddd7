// Hand-written elementwise kernels (fp32): Add, bias add, ReLU / GELU, and the element
// type casts.  They stand in for the scalar one-element-per-thread kernels the reference
// compiler generates (lib/Dialect/Device/Transform/TilingScfParallelDevice.cpp:31-84) and
// for the shared-memory-staged cast kernels of lib/Kernels/GPU/Utils.cu:16-83.
//
// All are HBM-bound: each thread moves 128 bits per access, UNROLL accesses are issued
// before the first use so enough bytes are in flight per SM, and the grid is a multiple of
// the SM count walked with a grid stride.  Unaligned pointers and tails take a scalar path.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "activation.cuh"

namespace mdc {

constexpr int kEwBlock = 256;
constexpr int kEwUnroll = 4;

__device__ __forceinline__ bool aligned16(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// c = a + b.  IEEE fp32 add, no contraction possible: bit-exact with the CPU loop.
__global__ void __launch_bounds__(kEwBlock)
mdc_add_f32(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ c,
            int64_t n) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (aligned16(a) && aligned16(b) && aligned16(c)) {
    const int64_t nvec = n >> 2;
    const float4 *a4 = reinterpret_cast<const float4 *>(a);
    const float4 *b4 = reinterpret_cast<const float4 *>(b);
    float4 *c4 = reinterpret_cast<float4 *>(c);
    int64_t i = tid;
    for (; i + (kEwUnroll - 1) * nthreads < nvec; i += kEwUnroll * nthreads) {
      float4 va[kEwUnroll], vb[kEwUnroll];
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        va[u] = __ldcs(a4 + i + u * nthreads);
        vb[u] = __ldcs(b4 + i + u * nthreads);
      }
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        float4 r;
        r.x = __fadd_rn(va[u].x, vb[u].x);
        r.y = __fadd_rn(va[u].y, vb[u].y);
        r.z = __fadd_rn(va[u].z, vb[u].z);
        r.w = __fadd_rn(va[u].w, vb[u].w);
        __stcs(c4 + i + u * nthreads, r);
      }
    }
    for (; i < nvec; i += nthreads) {
      const float4 va = a4[i], vb = b4[i];
      float4 r;
      r.x = __fadd_rn(va.x, vb.x);
      r.y = __fadd_rn(va.y, vb.y);
      r.z = __fadd_rn(va.z, vb.z);
      r.w = __fadd_rn(va.w, vb.w);
      c4[i] = r;
    }
    for (int64_t j = (nvec << 2) + tid; j < n; j += nthreads) c[j] = __fadd_rn(a[j], b[j]);
  } else {
    for (int64_t j = tid; j < n; j += nthreads) c[j] = __fadd_rn(a[j], b[j]);
  }
}

// y[r, j] = x[r, j] + bias[j]
__global__ void __launch_bounds__(kEwBlock)
mdc_bias_add_f32(const float *__restrict__ x, const float *__restrict__ bias,
                 float *__restrict__ y, int64_t rows, int64_t cols) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n = rows * cols;
  if ((cols & 3) == 0 && aligned16(x) && aligned16(y) && aligned16(bias)) {
    const int64_t nvec = n >> 2;
    const int64_t cvec = cols >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *b4 = reinterpret_cast<const float4 *>(bias);
    float4 *y4 = reinterpret_cast<float4 *>(y);
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const float4 v = __ldcs(x4 + i);
      const float4 bv = __ldg(b4 + (i % cvec));
      float4 r;
      r.x = __fadd_rn(v.x, bv.x);
      r.y = __fadd_rn(v.y, bv.y);
      r.z = __fadd_rn(v.z, bv.z);
      r.w = __fadd_rn(v.w, bv.w);
      __stcs(y4 + i, r);
    }
  } else {
    for (int64_t j = tid; j < n; j += nthreads) y[j] = __fadd_rn(x[j], bias[j % cols]);
  }
}

template <int ACT>
__device__ __forceinline__ void activation_body(const float *__restrict__ x, float *__restrict__ y,
                                                int64_t n) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (aligned16(x) && aligned16(y)) {
    const int64_t nvec = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    float4 *y4 = reinterpret_cast<float4 *>(y);
    int64_t i = tid;
    for (; i + (kEwUnroll - 1) * nthreads < nvec; i += kEwUnroll * nthreads) {
      float4 v[kEwUnroll];
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) v[u] = __ldcs(x4 + i + u * nthreads);
#pragma unroll
      for (int u = 0; u < kEwUnroll; ++u) {
        float4 r;
        r.x = act_apply_t<ACT>(v[u].x);
        r.y = act_apply_t<ACT>(v[u].y);
        r.z = act_apply_t<ACT>(v[u].z);
        r.w = act_apply_t<ACT>(v[u].w);
        __stcs(y4 + i + u * nthreads, r);
      }
    }
    for (; i < nvec; i += nthreads) {
      const float4 v = x4[i];
      float4 r;
      r.x = act_apply_t<ACT>(v.x);
      r.y = act_apply_t<ACT>(v.y);
      r.z = act_apply_t<ACT>(v.z);
      r.w = act_apply_t<ACT>(v.w);
      y4[i] = r;
    }
    for (int64_t j = (nvec << 2) + tid; j < n; j += nthreads) y[j] = act_apply_t<ACT>(x[j]);
  } else {
    for (int64_t j = tid; j < n; j += nthreads) y[j] = act_apply_t<ACT>(x[j]);
  }
}

__global__ void __launch_bounds__(kEwBlock)
mdc_relu_f32(const float *__restrict__ x, float *__restrict__ y, int64_t n) {
  activation_body<kActRelu>(x, y, n);
}
__global__ void __launch_bounds__(kEwBlock)
mdc_gelu_erf_f32(const float *__restrict__ x, float *__restrict__ y, int64_t n) {
  activation_body<kActGeluErf>(x, y, n);
}
__global__ void __launch_bounds__(kEwBlock)
mdc_gelu_tanh_f32(const float *__restrict__ x, float *__restrict__ y, int64_t n) {
  activation_body<kActGeluTanh>(x, y, n);
}

// Grid for a grid-stride kernel over nvec 128-bit items: enough blocks to cover the
// data once at kEwUnroll items per thread, capped at 8 resident blocks per SM.
inline int ew_grid(int64_t n_items, int num_sms) {
  int64_t per_block = static_cast<int64_t>(kEwBlock) * kEwUnroll;
  int64_t blocks = (n_items + per_block - 1) / per_block;
  int64_t cap = static_cast<int64_t>(num_sms) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace mdc
