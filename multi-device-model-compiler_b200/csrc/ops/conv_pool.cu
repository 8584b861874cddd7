// mgpuConv2d and mgpuPool2d (reference: lib/Kernels/GPU/Ops.cu:238-374, CPU twins
// lib/Kernels/CPU/Ops.cpp:83-210).  fp32 NCHW tensors at the boundary, OIHW filters.
//
// Convolution = gather + tensor-core Gemm + scatter:
//   1. im2col_kernel gathers the input patches into a 16-bit matrix col[N*OH*OW, Kp]
//      (k = (ic*KH + kh)*KW + kw, the order the OIHW filter is already stored in, so the
//      filter only needs a cast, not a transpose);
//   2. the tcgen05 Gemm computes y[N*OH*OW, OC] = col * filter^T + bias in fp32 (ReLU fused
//      there when nothing is added afterwards);
//   3. nhwc_to_nchw_kernel transposes each image's [OH*OW, OC] block into [OC, OH*OW] through
//      shared memory, adding postAdd and applying ReLU on the way.
// The filter is applied as a cross-correlation (ONNX Conv, oneDNN convolution_forward).
// The reference's GPU path asks cuDNN for CUDNN_CONVOLUTION (a flipped filter, Ops.cu:258),
// which disagrees with its own CPU path; this library follows the CPU path and ONNX.
// With both flags set the result is relu(conv + bias + postAdd), cuDNN's fused form
// (Ops.cu:334-337).
//
// Pooling: one thread per output element, window read straight from global memory (adjacent
// threads read adjacent windows, so every line is fetched from HBM once and re-served by
// L1/L2).  method 0 = max over the in-bounds elements, 1 = average with the padding counted
// (divisor = window elements inside the padded extent = KH*KW for every window that fits).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ops_common.h"

namespace mdc {
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s);

namespace {

struct ConvGeom {
  int N, IC, H, W, OC, KH, KW, OH, OW, PHL, PWL, SH, SW, DH, DW;
  int K, Kp;      // IC*KH*KW and its multiple-of-8 padding
  int64_t M;      // N*OH*OW
};

// One thread per 8 consecutive k of one output pixel: a single 16-byte store, coalesced
// along k; the scattered 4-byte reads hit L1/L2 (the input is KH*KW times smaller than col).
__global__ void __launch_bounds__(256) im2col_kernel(const float *__restrict__ x, __half *__restrict__ col,
                                                     ConvGeom g) {
  const int groups = g.Kp >> 3;
  const int64_t total = g.M * groups;
  const int khw = g.KH * g.KW;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total;
       idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t m = idx / groups;
    const int k0 = int(idx - m * groups) << 3;
    const int ow = int(m % g.OW);
    const int64_t t = m / g.OW;
    const int oh = int(t % g.OH);
    const int n = int(t / g.OH);
    int ic = k0 / khw;
    int r = k0 - ic * khw;
    int kh = r / g.KW;
    int kw = r - kh * g.KW;
    const int ih0 = oh * g.SH - g.PHL, iw0 = ow * g.SW - g.PWL;
    const float *img = x + int64_t(n) * g.IC * g.H * g.W;
    __align__(16) __half v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float val = 0.f;
      if (k0 + j < g.K) {
        const int ih = ih0 + kh * g.DH, iw = iw0 + kw * g.DW;
        if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) val = __ldg(img + (int64_t(ic) * g.H + ih) * g.W + iw);
      }
      v[j] = __float2half_rn(val);
      if (++kw == g.KW) {
        kw = 0;
        if (++kh == g.KH) kh = 0, ++ic;
      }
    }
    *reinterpret_cast<uint4 *>(col + m * g.Kp + k0) = *reinterpret_cast<const uint4 *>(v);
  }
}

// y[n][p][oc] -> out[n][oc][p] (+ add[n][oc][p]) (ReLU); 32x32 tiles, block (32, 8).
template <bool ADD, bool RELU>
__global__ void __launch_bounds__(256) nhwc_to_nchw_kernel(const float *__restrict__ y, const float *__restrict__ add,
                                                           float *__restrict__ out, int P, int OC) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const float *src = y + int64_t(n) * P * OC;
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int p = p0 + i, c = c0 + threadIdx.x;
    if (p < P && c < OC) tile[i][threadIdx.x] = src[int64_t(p) * OC + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, p = p0 + threadIdx.x;
    if (c < OC && p < P) {
      const int64_t o = (int64_t(n) * OC + c) * P + p;
      float v = tile[threadIdx.x][i];
      if (ADD) v += add[o];
      if (RELU) v = fmaxf(v, 0.f);
      out[o] = v;
    }
  }
}

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

int grid_for(int64_t items, int per_block) {
  const int64_t blocks = (items + per_block - 1) / per_block;
  const int64_t cap = int64_t(device_info().sms) * 16;
  return int(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace
}  // namespace mdc

using namespace mdc;

MDC_API void mgpuConv2d(float *input, float *weight, float *bias, float *output, float *postAdd, int64_t N,
                        int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH, int64_t KW, int64_t OH,
                        int64_t OW, int64_t PHL, int64_t PWL, int64_t PHR, int64_t PWR, int64_t SH, int64_t SW,
                        int64_t DH, int64_t DW, bool hasPostAdd, bool hasContainRelu, void *stream) {
  if (N <= 0 || OC <= 0 || OH <= 0 || OW <= 0) return;
  if (IC <= 0 || H <= 0 || W <= 0 || KH <= 0 || KW <= 0 || SH <= 0 || SW <= 0 || DH <= 0 || DW <= 0 ||
      PHL < 0 || PWL < 0 || PHR < 0 || PWR < 0) {
    fail("mgpuConv2d: sizes, strides and dilations must be positive, paddings non-negative");
    return;
  }
  // the caller's output extent must be the one its geometry produces
  if ((OH - 1) * SH + (KH - 1) * DH + 1 > H + PHL + PHR || (OW - 1) * SW + (KW - 1) * DW + 1 > W + PWL + PWR) {
    fail("mgpuConv2d: output extent does not fit the padded input");
    return;
  }
  if (hasPostAdd && !postAdd) { fail("mgpuConv2d: hasPostAdd without a postAdd tensor"); return; }
  const int64_t M = N * OH * OW, K = IC * KH * KW;
  if (M > INT32_MAX || K > (1 << 24) || OC > (1 << 24) || N > 65535 || H * W > INT32_MAX) {
    fail("mgpuConv2d: shape exceeds this library's index range");
    return;
  }
  if (!device_info().ok) return;
  cudaStream_t s = as_stream(stream);
  ConvGeom g;
  g.N = int(N), g.IC = int(IC), g.H = int(H), g.W = int(W), g.OC = int(OC), g.KH = int(KH), g.KW = int(KW);
  g.OH = int(OH), g.OW = int(OW), g.PHL = int(PHL), g.PWL = int(PWL), g.SH = int(SH), g.SW = int(SW);
  g.DH = int(DH), g.DW = int(DW), g.K = int(K), g.Kp = int((K + 7) / 8 * 8), g.M = M;

  void *col = mgpuMemAllocAsync(uint64_t(M) * g.Kp * 2, stream);
  void *w16 = mgpuMemAllocAsync(uint64_t(OC) * g.Kp * 2, stream);
  void *y = mgpuMemAllocAsync(uint64_t(M) * OC * 4, stream);
  if (col && w16 && y) {
    im2col_kernel<<<grid_for(M * (g.Kp / 8), 256), 256, 0, s>>>(input, static_cast<__half *>(col), g);
    check_cuda(cudaGetLastError(), "launch im2col");
    launched("mdc_im2col");
    cast_rows_padded(weight, w16, OC, K, g.Kp, MGPU_DTYPE_F16, s);
    const bool relu_in_gemm = hasContainRelu && !hasPostAdd;
    mgpuMatmulEx16(col, w16, bias, nullptr, y, M, OC, g.Kp, MGPU_DTYPE_F16, MGPU_DTYPE_F32,
                   relu_in_gemm ? MGPU_ACT_RELU : MGPU_ACT_NONE, stream);
    const int P = int(OH * OW);
    const dim3 grid((P + 31) / 32, (unsigned(OC) + 31) / 32, unsigned(N)), block(32, 8);
    float *yf = static_cast<float *>(y);
    if (hasPostAdd && hasContainRelu) nhwc_to_nchw_kernel<true, true><<<grid, block, 0, s>>>(yf, postAdd, output, P, int(OC));
    else if (hasPostAdd) nhwc_to_nchw_kernel<true, false><<<grid, block, 0, s>>>(yf, postAdd, output, P, int(OC));
    else nhwc_to_nchw_kernel<false, false><<<grid, block, 0, s>>>(yf, nullptr, output, P, int(OC));
    check_cuda(cudaGetLastError(), "launch nhwc_to_nchw");
    launched("mdc_nhwc_to_nchw");
  }
  if (col) mgpuMemFreeAsync(col, stream);
  if (w16) mgpuMemFreeAsync(w16, stream);
  if (y) mgpuMemFreeAsync(y, stream);
}

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
  if (method == 1) pool2d_kernel<true><<<grid, 256, 0, s>>>(input, output, g);
  else pool2d_kernel<false><<<grid, 256, 0, s>>>(input, output, g);
  check_cuda(cudaGetLastError(), "launch pool2d");
  launched("mdc_pool2d");
}
