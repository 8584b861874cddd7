// The C++-linkage template entry points that sibling translation units of the reference link
// against (include/multi-device-model-compiler/Kernels/GPU/Ops.h:51-74, Utils.h:6-8), as thin
// explicit instantiations that forward to this library's extern "C" entry points.  They exist
// so that reference code calling mgpuMatmulEx<half> / mgpuLayerNorm<half> /
// mgpuAddResidualPreLayerNorm<half> / mgpuAddFusedQKVBiasTranspose<half> / invokeCudaCast
// (as lib/Kernels/GPU/LLM.cu:50-158 does) links unchanged; the encoder-stack entry points of
// this library do not go through them.  Scratch comes from the runtime's device pool and is
// returned in stream order.
#include "mdc_gpu_ops_cxx.h"
#include "ops_common.h"

using namespace mdc;

namespace {
// fp32 copy of n 16-bit values in a pool block (nullptr in -> nullptr out)
float *to_f32(const void *src, int64_t n, void *stream) {
  if (!src) return nullptr;
  float *dst = static_cast<float *>(mgpuMemAllocAsync(static_cast<uint64_t>(n) * 4, stream));
  if (dst) mgpuCast(src, MGPU_DTYPE_F16, dst, MGPU_DTYPE_F32, n, stream);
  return dst;
}
void give_back(void *p, void *stream) {
  if (p) mgpuMemFreeAsync(p, stream);
}

// q / k / v [batch, head, seq, d] <- QKV [token, 3, head * d] + bias [3, head * d]; the biased
// values are also written back into QKV, as the reference kernel does
// (lib/Kernels/GPU/Transpose.cu:6-52).  One thread per 8 consecutive elements of a head row.
__global__ void __launch_bounds__(256)
qkv_bias_transpose_kernel(__half *q, __half *k, __half *v, __half *qkv, const __half *bias, int seq_len,
                          int64_t tokens, int heads, int d) {
  const int64_t n = static_cast<int64_t>(heads) * d;
  const int64_t groups = tokens * 3 * n / 8;
  __half *out[3] = {q, k, v};
  for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t index = g * 8;
    const int64_t in_token = index % (3 * n), token = index / (3 * n);
    const int which = static_cast<int>(in_token / n);
    const int head = static_cast<int>((in_token % n) / d), e = static_cast<int>(in_token % d);
    const int64_t b = token / seq_len, s = token % seq_len;
    uint4 x = *reinterpret_cast<const uint4 *>(qkv + index);
    const uint4 bb = bias ? *reinterpret_cast<const uint4 *>(bias + in_token) : make_uint4(0, 0, 0, 0);
    __half2 *xh = reinterpret_cast<__half2 *>(&x);
    const __half2 *bh = reinterpret_cast<const __half2 *>(&bb);
#pragma unroll
    for (int i = 0; i < 4; ++i) xh[i] = __hadd2(xh[i], bh[i]);
    *reinterpret_cast<uint4 *>(qkv + index) = x;
    *reinterpret_cast<uint4 *>(out[which] + ((b * heads + head) * seq_len + s) * d + e) = x;
  }
}
}  // namespace

// ---- lib/Kernels/GPU/Utils.cu:38-103 ----
template <>
MDC_CXX_API void invokeCudaCast<half, float>(half *dst, float const *const src, const size_t size, cudaStream_t stream) {
  mgpuCast(src, MGPU_DTYPE_F32, dst, MGPU_DTYPE_F16, static_cast<int64_t>(size), stream);
}
template <>
MDC_CXX_API void invokeCudaCast<float, half>(float *dst, half const *const src, const size_t size, cudaStream_t stream) {
  mgpuCast(src, MGPU_DTYPE_F16, dst, MGPU_DTYPE_F32, static_cast<int64_t>(size), stream);
}

// ---- lib/Kernels/GPU/Ops.cu:136-234.  weight is [K, N] row-major like mgpuMatmul's; the
// reference applies the activation to A.W + bias + residual (cuBLASLt adds beta * C before the
// epilogue), the fused epilogue here adds the residual after the activation, so the one
// combination in which the two differ (ReLU together with a residual, which the reference
// layer never uses) is refused.
template <typename T>
static void matmul_ex(T *input, T *weight, T *bias, T *output, T *residual, int64_t M, int64_t N, int64_t K,
                      bool hasBias, bool hasRelu, bool hasResidual, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  if (!device_info().ok) return;
  if (hasRelu && hasResidual) { fail("mgpuMatmulEx: ReLU together with a residual is not supported"); return; }
  constexpr bool is16 = sizeof(T) == 2;
  const int64_t Kp = (K + 7) / 8 * 8;
  if (is16 && Kp != K) { fail("mgpuMatmulEx<half>: K must be a multiple of 8"); return; }
  void *s = stream;
  // operands in the Gemm's form: A 16-bit [M, Kp], W 16-bit [N, Kp], bias fp32, residual 16-bit
  float *w32 = is16 ? to_f32(weight, K * N, s) : reinterpret_cast<float *>(weight);
  bool w_cached = false;
  void *w16 = w32 ? packed_weight(w32, K, N, MGPU_DTYPE_F16, s, &w_cached) : nullptr;
  void *a16 = input;
  if (!is16) {
    a16 = mgpuMemAllocAsync(static_cast<uint64_t>(M) * Kp * 2, s);
    if (a16) cast_rows_padded(reinterpret_cast<const float *>(input), a16, M, K, Kp, MGPU_DTYPE_F16, stream);
  }
  float *b32 = nullptr;
  if (hasBias) b32 = is16 ? to_f32(bias, N, s) : reinterpret_cast<float *>(bias);
  void *r16 = nullptr;
  if (hasResidual) {
    if (is16) r16 = residual;
    else {
      r16 = mgpuMemAllocAsync(static_cast<uint64_t>(M) * N * 2, s);
      if (r16) mgpuCast(residual, MGPU_DTYPE_F32, r16, MGPU_DTYPE_F16, M * N, s);
    }
  }
  if (w16 && a16 && (!hasBias || b32) && (!hasResidual || r16))
    mgpuMatmulEx16(a16, w16, b32, r16, output, M, N, Kp, MGPU_DTYPE_F16, is16 ? MGPU_DTYPE_F16 : MGPU_DTYPE_F32,
                   hasRelu ? MGPU_ACT_RELU : MGPU_ACT_NONE, s);
  else
    fail("mgpuMatmulEx: out of device memory for the converted operands");
  if (is16) give_back(w32, s);
  if (w16 && !w_cached) give_back(w16, s);
  if (!is16) give_back(a16, s);
  if (is16) give_back(b32, s);
  if (!is16) give_back(r16, s);
}
template <>
MDC_CXX_API void mgpuMatmulEx<half>(half *input, half *weight, half *bias, half *output, half *residual, int64_t M,
                                    int64_t N, int64_t K, bool hasBias, bool hasRelu, bool hasResidual,
                                    cudaStream_t stream) {
  matmul_ex<half>(input, weight, bias, output, residual, M, N, K, hasBias, hasRelu, hasResidual, stream);
}
template <>
MDC_CXX_API void mgpuMatmulEx<float>(float *input, float *weight, float *bias, float *output, float *residual,
                                     int64_t M, int64_t N, int64_t K, bool hasBias, bool hasRelu, bool hasResidual,
                                     cudaStream_t stream) {
  matmul_ex<float>(input, weight, bias, output, residual, M, N, K, hasBias, hasRelu, hasResidual, stream);
}

// ---- lib/Kernels/GPU/LayerNorm.cu:410-465.  gamma / beta are 16-bit there and fp32 here;
// `scale` (an int8 hook of the kernel the reference took over) is unused, as in the reference.
template <>
MDC_CXX_API void mgpuLayerNorm<half>(const half *input, const half *gamma, const half *beta, half *output,
                                     const float layernorm_eps, const int m, const int n, float * /*scale*/,
                                     cudaStream_t stream) {
  if (m <= 0 || n <= 0) return;
  float *g = to_f32(gamma, n, stream), *b = to_f32(beta, n, stream);
  mgpuLayerNormEx(input, nullptr, g, b, nullptr, output, layernorm_eps, m, n, MGPU_DTYPE_F16, MGPU_DTYPE_F16, stream);
  give_back(g, stream);
  give_back(b, stream);
}
// output = input + residual (16-bit), normed_output = LayerNorm(output)
template <>
MDC_CXX_API void mgpuAddResidualPreLayerNorm<half>(const half *input, const half *residual, const half *gamma,
                                                   const half *beta, half *output, half *normed_output,
                                                   const float layernorm_eps, int m, int n, float * /*scale*/,
                                                   cudaStream_t stream) {
  if (m <= 0 || n <= 0) return;
  float *g = to_f32(gamma, n, stream), *b = to_f32(beta, n, stream);
  mgpuLayerNormEx(input, residual, g, b, output, normed_output, layernorm_eps, m, n, MGPU_DTYPE_F16, MGPU_DTYPE_F16,
                  stream);
  give_back(g, stream);
  give_back(b, stream);
}

// ---- lib/Kernels/GPU/Transpose.cu:6-85 (not called by the reference layer itself) ----
template <>
MDC_CXX_API void mgpuAddFusedQKVBiasTranspose<half>(half *q_buf, half *k_buf, half *v_buf, half *QKV,
                                                    const half *qkv_bias, const int batch_size, const int seq_len,
                                                    const int token_num, const int head_num, const int size_per_head,
                                                    cudaStream_t stream) {
  (void)batch_size;
  if (token_num <= 0 || head_num <= 0 || size_per_head <= 0 || seq_len <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (size_per_head % 8 || !al(q_buf) || !al(k_buf) || !al(v_buf) || !al(QKV) || (qkv_bias && !al(qkv_bias))) {
    fail("mgpuAddFusedQKVBiasTranspose: size_per_head must be a multiple of 8 and the buffers 16-byte aligned");
    return;
  }
  const int64_t groups = static_cast<int64_t>(token_num) * 3 * head_num * size_per_head / 8;
  const int64_t want = (groups + 255) / 256, cap = static_cast<int64_t>(di.sms) * 8;
  qkv_bias_transpose_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, stream>>>(
      q_buf, k_buf, v_buf, QKV, qkv_bias, seq_len, token_num, head_num, size_per_head);
  launched("qkv_bias_transpose_kernel");
}
