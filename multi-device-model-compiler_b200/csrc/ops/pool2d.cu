// mgpuPool2d (reference: lib/Kernels/GPU/Ops.cu:342-374, CPU twin lib/Kernels/CPU/Ops.cpp:161-210).
// fp32 NCHW tensors.  One thread per output element, window read straight from global memory
// (adjacent threads read adjacent windows, so every line is fetched from HBM once and
// re-served by L1/L2).  method 0 = max over the in-bounds elements, 1 = average with the
// padding counted (divisor = window elements inside the padded extent = KH*KW for every
// window that fits).
#include <type_traits>

#include "ops_common.h"

namespace mdc {
namespace {

struct PoolGeom {
  int C, H, W, OH, OW, KH, KW, PHL, PWL, PHR, PWR, SH, SW;
  int64_t total;  // N*C*OH*OW
};

template <bool AVG>
__global__ void __launch_bounds__(256) pool2d_kernel(const float *__restrict__ x, float *__restrict__ out, PoolGeom g) {
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < g.total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int ow = int(idx % g.OW);
    const int64_t t = idx / g.OW;
    const int oh = int(t % g.OH);
    const int64_t plane = t / g.OH;  // n*C + c
    const float *src = x + plane * g.H * g.W;
    const int ih0 = oh * g.SH - g.PHL, iw0 = ow * g.SW - g.PWL;
    const int ih_lo = max(ih0, 0), ih_hi = min(ih0 + g.KH, g.H);
    const int iw_lo = max(iw0, 0), iw_hi = min(iw0 + g.KW, g.W);
    float acc = AVG ? 0.f : -INFINITY;
    for (int ih = ih_lo; ih < ih_hi; ++ih)
      for (int iw = iw_lo; iw < iw_hi; ++iw) {
        const float v = __ldg(src + int64_t(ih) * g.W + iw);
        acc = AVG ? acc + v : fmaxf(acc, v);
      }
    if (AVG) {
      // padding counts, anything beyond the padded extent does not
      const int rows = min(ih0 + g.KH, g.H + g.PHR) - ih0;
      const int cols = min(iw0 + g.KW, g.W + g.PWR) - iw0;
      acc /= float(max(rows * cols, 1));
    }
    out[idx] = acc;
  }
}

// Non-overlapping windows without padding whose rows are one aligned vector (KW == SW == VEC,
// W a multiple of VEC): each window row is a single 8- or 16-byte load.
template <bool AVG, int VEC>
__global__ void __launch_bounds__(256) pool2d_tiled_kernel(const float *__restrict__ x, float *__restrict__ out,
                                                           PoolGeom g) {
  using V = typename std::conditional<VEC == 4, float4, float2>::type;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < g.total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int ow = int(idx % g.OW);
    const int64_t t = idx / g.OW;
    const int oh = int(t % g.OH);
    const int64_t plane = t / g.OH;
    const float *src = x + (plane * g.H + int64_t(oh) * g.SH) * g.W + ow * VEC;
    float acc = AVG ? 0.f : -INFINITY;
    for (int kh = 0; kh < g.KH; ++kh) {
      const V v = __ldg(reinterpret_cast<const V *>(src + int64_t(kh) * g.W));
      if constexpr (VEC == 4) {
        acc = AVG ? acc + v.x + v.y + v.z + v.w : fmaxf(fmaxf(acc, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
      } else {
        acc = AVG ? acc + v.x + v.y : fmaxf(acc, fmaxf(v.x, v.y));
      }
    }
    out[idx] = AVG ? acc / float(g.KH * VEC) : acc;
  }
}

int grid_for(int64_t items, int per_block) {
  const int64_t blocks = (items + per_block - 1) / per_block;
  const int64_t cap = int64_t(device_info().sms) * 16;
  return int(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace
}  // namespace mdc

using namespace mdc;

MDC_API void mgpuPool2d(float *input, float *output, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OH,
                        int64_t OW, int64_t KH, int64_t KW, int64_t PHL, int64_t PWL, int64_t PHR, int64_t PWR,
                        int64_t SH, int64_t SW, int64_t method, void *stream) {
  if (N <= 0 || C <= 0 || OH <= 0 || OW <= 0) return;
  if (H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || SH <= 0 || SW <= 0 || PHL < 0 || PWL < 0 || PHR < 0 || PWR < 0) {
    fail("mgpuPool2d: sizes and strides must be positive, paddings non-negative");
    return;
  }
  if (method != 0 && method != 1) { fail("mgpuPool2d: method must be 0 (max) or 1 (average)"); return; }
  if ((OH - 1) * SH + KH > H + PHL + PHR || (OW - 1) * SW + KW > W + PWL + PWR) {
    fail("mgpuPool2d: output extent does not fit the padded input");
    return;
  }
  // a window that lies wholly in the padding has no defined maximum
  if (method == 0 && (PHL >= KH || PWL >= KW || (OH - 1) * SH - PHL >= H || (OW - 1) * SW - PWL >= W)) {
    fail("mgpuPool2d: a window lies entirely inside the padding");
    return;
  }
  if (H * W > INT32_MAX || OH > INT32_MAX || OW > INT32_MAX) {
    fail("mgpuPool2d: shape exceeds this library's index range");
    return;
  }
  if (!device_info().ok) return;
  PoolGeom g;
  g.C = int(C), g.H = int(H), g.W = int(W), g.OH = int(OH), g.OW = int(OW), g.KH = int(KH), g.KW = int(KW);
  g.PHL = int(PHL), g.PWL = int(PWL), g.PHR = int(PHR), g.PWR = int(PWR), g.SH = int(SH), g.SW = int(SW);
  g.total = N * C * OH * OW;
  cudaStream_t s = as_stream(stream);
  const int grid = grid_for(g.total, 256);
  const bool tiled = PHL == 0 && PWL == 0 && KW == SW && (KW == 4 || KW == 2) && W % KW == 0 &&
                     (OH - 1) * SH + KH <= H && OW * KW <= W &&
                     reinterpret_cast<uintptr_t>(input) % (KW * 4) == 0;
  if (tiled && KW == 4) {
    if (method == 1) pool2d_tiled_kernel<true, 4><<<grid, 256, 0, s>>>(input, output, g);
    else pool2d_tiled_kernel<false, 4><<<grid, 256, 0, s>>>(input, output, g);
  } else if (tiled) {
    if (method == 1) pool2d_tiled_kernel<true, 2><<<grid, 256, 0, s>>>(input, output, g);
    else pool2d_tiled_kernel<false, 2><<<grid, 256, 0, s>>>(input, output, g);
  } else if (method == 1) {
    pool2d_kernel<true><<<grid, 256, 0, s>>>(input, output, g);
  } else {
    pool2d_kernel<false><<<grid, 256, 0, s>>>(input, output, g);
  }
  check_cuda(cudaGetLastError(), "launch pool2d");
  launched("mdc_pool2d");
}
