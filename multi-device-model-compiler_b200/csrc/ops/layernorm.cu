// Row LayerNorm (optionally fused with a residual add) for fp32 / fp16 / bf16 tensors.
//
// Replaces generalAddBiasResidualLayerNormOpt2 (lib/Kernels/GPU/LayerNorm.cu:138-260),
// which keeps one block per row, stages the row in shared memory as half2 and derives the
// variance from E[x^2] - mean^2.  Here one WARP owns a row: the row is read from HBM once
// with 128-bit loads straight into registers, the statistics are an exact two-pass
// computation over the registers (the mean by one shuffle butterfly, the centred sum of squares
// by a second one), and the normalised row is written with 128-bit stores.  No shared memory,
// no block barrier, exactly one HBM read and one HBM write per element: fp32 rows are bound by
// HBM bandwidth (8 bytes per element); the shorter 16-bit rows are bound by instruction issue,
// which is why the statistics avoid anything costlier than adds and shuffles.
#include "ops_common.h"
#include "ptx_sm100.cuh"

namespace mdc {

template <typename T>
struct LnTraits;
template <>
struct LnTraits<float> {
  static constexpr int EPC = 4;  // elements per 16-byte chunk
  __device__ static void unpack(const uint4 &r, float *v) {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y);
    v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
  __device__ static float round(float v) { return v; }
};
template <>
struct LnTraits<__half> {
  static constexpr int EPC = 8;
  __device__ static void unpack(const uint4 &r, float *v) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <>
struct LnTraits<__nv_bfloat16> {
  static constexpr int EPC = 8;
  __device__ static void unpack(const uint4 &r, float *v) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// Stores N consecutive floats as T starting at dst (dst aligned to N * sizeof(T) bytes).
template <typename T, int N>
__device__ __forceinline__ void store_vec(T *dst, const float *v);
template <>
__device__ __forceinline__ void store_vec<float, 4>(float *dst, const float *v) {
  __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
}
template <>
__device__ __forceinline__ void store_vec<float, 8>(float *dst, const float *v) {
  __stcs(reinterpret_cast<float4 *>(dst), make_float4(v[0], v[1], v[2], v[3]));
  __stcs(reinterpret_cast<float4 *>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
}
template <>
__device__ __forceinline__ void store_vec<__half, 4>(__half *dst, const float *v) {
  uint2 o;
  *reinterpret_cast<__half2 *>(&o.x) = __floats2half2_rn(v[0], v[1]);
  *reinterpret_cast<__half2 *>(&o.y) = __floats2half2_rn(v[2], v[3]);
  *reinterpret_cast<uint2 *>(dst) = o;
}
template <>
__device__ __forceinline__ void store_vec<__half, 8>(__half *dst, const float *v) {
  uint4 o;
  *reinterpret_cast<__half2 *>(&o.x) = __floats2half2_rn(v[0], v[1]);
  *reinterpret_cast<__half2 *>(&o.y) = __floats2half2_rn(v[2], v[3]);
  *reinterpret_cast<__half2 *>(&o.z) = __floats2half2_rn(v[4], v[5]);
  *reinterpret_cast<__half2 *>(&o.w) = __floats2half2_rn(v[6], v[7]);
  *reinterpret_cast<uint4 *>(dst) = o;
}
template <>
__device__ __forceinline__ void store_vec<__nv_bfloat16, 4>(__nv_bfloat16 *dst, const float *v) {
  uint2 o;
  *reinterpret_cast<__nv_bfloat162 *>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2 *>(dst) = o;
}
template <>
__device__ __forceinline__ void store_vec<__nv_bfloat16, 8>(__nv_bfloat16 *dst, const float *v) {
  uint4 o;
  *reinterpret_cast<__nv_bfloat162 *>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.z) = __floats2bfloat162_rn(v[4], v[5]);
  *reinterpret_cast<__nv_bfloat162 *>(&o.w) = __floats2bfloat162_rn(v[6], v[7]);
  *reinterpret_cast<uint4 *>(dst) = o;
}

constexpr int kLnWarpsPerBlock = 4;

// One warp per row, persistent: a warp walks rows warp_id, warp_id + total_warps, ... and
// has the NEXT row's 128-bit loads in flight while it reduces and writes the current one
// (short 16-bit rows would otherwise leave too few bytes in flight per SM).  n must be a
// multiple of EPC, rows 16-byte aligned, and n <= 32 * MAXI * EPC.  Lane l owns chunks
// l, l+32, ... (coalesced 512-byte warp accesses).
// FULL: the row is exactly 32 * MAXI chunks, so no lane ever skips a chunk and the per-chunk
// tests (and the instructions of chunks that would be predicated off) disappear.
template <typename TIn, typename TOut, int MAXI, bool RES, bool FULL>
__global__ void __launch_bounds__(kLnWarpsPerBlock * 32,
                                  (MAXI >= 8 || sizeof(TIn) == 4) ? 2 : ((RES || (FULL && MAXI >= 4)) ? 4 : 6))
layernorm_warp_kernel(const TIn *__restrict__ x, const TIn *__restrict__ residual,
                      const float *__restrict__ gamma, const float *__restrict__ beta,
                      TIn *__restrict__ sum_out, TOut *__restrict__ y, float eps, int64_t m, int n) {
  constexpr int EPC = LnTraits<TIn>::EPC;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t total_warps = static_cast<int64_t>(gridDim.x) * kLnWarpsPerBlock;
  int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= m) return;
  const int nchunks = n / EPC;
  const float inv_n = 1.f / static_cast<float>(n);
  constexpr bool has_res = RES;
  constexpr bool kPrefetch = sizeof(TIn) == 2;

  uint4 raw[MAXI], raw_res[RES ? MAXI : 1];
  auto fetch = [&](int64_t rw) {
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + rw * n);
#pragma unroll
    for (int i = 0; i < MAXI; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nchunks) raw[i] = __ldcs(xr + c);
    }
    if constexpr (has_res) {
      const uint4 *rr = reinterpret_cast<const uint4 *>(residual + rw * n);
#pragma unroll
      for (int i = 0; i < MAXI; ++i) {
        const int c = lane + 32 * i;
        if (FULL || c < nchunks) raw_res[i] = __ldcs(rr + c);
      }
    }
  };
  fetch(row);

  using ptx::F2;
  using ptx::f2;
  using ptx::f2_add;
  using ptx::f2_fma;
  using ptx::f2_get;
  using ptx::f2_mul;
  for (; row < m;) {
    // the row as pairs of fp32 values: all arithmetic below is two lanes per instruction
    // (add / mul / fma .f32x2), which halves the instruction count of this issue-bound kernel
    F2 v[MAXI][EPC / 2];
#pragma unroll
    for (int i = 0; i < MAXI; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nchunks) {
        float t[EPC];
        LnTraits<TIn>::unpack(raw[i], t);
        if constexpr (has_res) {
          float r[EPC];
          LnTraits<TIn>::unpack(raw_res[i], r);
#pragma unroll
          for (int e = 0; e < EPC; ++e) t[e] = LnTraits<TIn>::round(t[e] + r[e]);
          if (sum_out) store_vec<TIn, EPC>(sum_out + row * n + static_cast<int64_t>(c) * EPC, t);
        }
#pragma unroll
        for (int e = 0; e < EPC / 2; ++e) v[i][e] = f2(t[2 * e], t[2 * e + 1]);
      }
    }
    // 16-bit rows are short: keep the next row's loads in flight during the reduction and
    // the stores below.  fp32 rows carry enough bytes per warp; there one row per warp (and
    // the higher occupancy of the smaller register footprint) is faster.
    const int64_t next = kPrefetch ? row + total_warps : m;
    if (next < m) fetch(next);

    // exact two-pass statistics across the warp: the mean first (one butterfly), then the
    // centred sum of squares (a second one).  Every lane ends with the same bits, because the
    // two partners of a butterfly step add the same two numbers.
    F2 sum2 = f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < MAXI; ++i)
      if (FULL || lane + 32 * i < nchunks) {
#pragma unroll
        for (int e = 0; e < EPC / 2; ++e) sum2 = f2_add(sum2, v[i][e]);
      }
    float sum_a, sum_b;
    f2_get(sum2, sum_a, sum_b);
    float sum = sum_a + sum_b;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float mean = sum * inv_n;
    const F2 neg_mean = f2(-mean, -mean);
    F2 m22 = f2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < MAXI; ++i)
      if (FULL || lane + 32 * i < nchunks) {
#pragma unroll
        for (int e = 0; e < EPC / 2; ++e) {
          v[i][e] = f2_add(v[i][e], neg_mean);  // the centred value is what the output needs too
          m22 = f2_fma(v[i][e], v[i][e], m22);
        }
      }
    float m2_a, m2_b;
    f2_get(m22, m2_a, m2_b);
    float m2 = m2_a + m2_b;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m2 += __shfl_xor_sync(0xffffffffu, m2, off);
    const float rstd = rsqrtf(fmaf(m2, inv_n, eps));
    const F2 rstd2 = f2(rstd, rstd);

#pragma unroll
    for (int i = 0; i < MAXI; ++i) {
      const int c = lane + 32 * i;
      if (FULL || c < nchunks) {
        float o[EPC];
#pragma unroll
        for (int e4 = 0; e4 < EPC / 4; ++e4) {
          F2 y0 = f2_mul(v[i][2 * e4], rstd2), y1 = f2_mul(v[i][2 * e4 + 1], rstd2);
          if (gamma && beta) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gamma) + c * (EPC / 4) + e4);
            const float4 b = __ldg(reinterpret_cast<const float4 *>(beta) + c * (EPC / 4) + e4);
            y0 = f2_fma(y0, f2(g.x, g.y), f2(b.x, b.y));
            y1 = f2_fma(y1, f2(g.z, g.w), f2(b.z, b.w));
          } else if (gamma) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gamma) + c * (EPC / 4) + e4);
            y0 = f2_mul(y0, f2(g.x, g.y));
            y1 = f2_mul(y1, f2(g.z, g.w));
          } else if (beta) {
            const float4 b = __ldg(reinterpret_cast<const float4 *>(beta) + c * (EPC / 4) + e4);
            y0 = f2_add(y0, f2(b.x, b.y));
            y1 = f2_add(y1, f2(b.z, b.w));
          }
          f2_get(y0, o[4 * e4 + 0], o[4 * e4 + 1]);
          f2_get(y1, o[4 * e4 + 2], o[4 * e4 + 3]);
        }
        store_vec<TOut, EPC>(y + row * n + static_cast<int64_t>(c) * EPC, o);
      }
    }
    row = next;
  }
}

// Fallback for any n / alignment: one block per row, the row staged in shared memory as
// fp32, exact two-pass statistics over the staged copy.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
layernorm_block_kernel(const TIn *__restrict__ x, const TIn *__restrict__ residual,
                       const float *__restrict__ gamma, const float *__restrict__ beta,
                       TIn *__restrict__ sum_out, TOut *__restrict__ y, float eps, int64_t m, int n) {
  extern __shared__ float row_s[];
  __shared__ float red[32];
  __shared__ float bcast;
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float s = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float v;
    if constexpr (sizeof(TIn) == 4) v = x[row * n + j];
    else v = static_cast<float>(x[row * n + j]);
    if (residual) {
      float r;
      if constexpr (sizeof(TIn) == 4) r = residual[row * n + j];
      else r = static_cast<float>(residual[row * n + j]);
      v = LnTraits<TIn>::round(v + r);
      if (sum_out) sum_out[row * n + j] = static_cast<TIn>(v);
    }
    row_s[j] = v;
    s += v;
  }
  auto block_sum = [&](float val) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) val += __shfl_xor_sync(0xffffffffu, val, off);
    __syncthreads();
    if (lane == 0) red[warp] = val;
    __syncthreads();
    if (warp == 0) {
      float t = lane < nwarps ? red[lane] : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    return bcast;
  };
  const float mean = block_sum(s) / static_cast<float>(n);
  float q = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float d = row_s[j] - mean;
    q = fmaf(d, d, q);
  }
  const float rstd = rsqrtf(block_sum(q) / static_cast<float>(n) + eps);
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float g = gamma ? gamma[j] : 1.f, b = beta ? beta[j] : 0.f;
    y[row * n + j] = static_cast<TOut>(fmaf((row_s[j] - mean) * rstd, g, b));
  }
}

template <typename TIn, typename TOut>
static void launch_layernorm(const void *x, const void *residual, const float *gamma,
                             const float *beta, void *sum_out, void *y, float eps, int64_t m,
                             int64_t n, cudaStream_t s) {
  constexpr int EPC = LnTraits<TIn>::EPC;
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const bool vec_ok = (n % EPC == 0) && n <= 32 * 16 * EPC && al(x) && al(y) &&
                      (!residual || al(residual)) && (!sum_out || al(sum_out)) &&
                      (!gamma || al(gamma)) && (!beta || al(beta));
  const TIn *xi = static_cast<const TIn *>(x), *ri = static_cast<const TIn *>(residual);
  TIn *so = static_cast<TIn *>(sum_out);
  TOut *yo = static_cast<TOut *>(y);
  if (vec_ok) {
    const int nchunks_host = static_cast<int>(n / EPC);
    const int per_lane = (nchunks_host + 31) / 32;
    // persistent: at most 16 blocks of 4 warps per SM, each warp walking several rows
    const int64_t blocks_needed = (m + kLnWarpsPerBlock - 1) / kLnWarpsPerBlock;
    const int64_t blocks_cap = static_cast<int64_t>(device_info().sms) * 16;
    const unsigned grid = static_cast<unsigned>(
        (sizeof(TIn) == 2 && blocks_needed > blocks_cap) ? blocks_cap : blocks_needed);
    const int threads = kLnWarpsPerBlock * 32;
    const int ni = static_cast<int>(n);
#define MDC_LN_LAUNCH2(MAXI_, FULL_)                                                                  \
  do {                                                                                            \
    if (ri)                                                                                       \
      check_cuda(launch_chain(layernorm_warp_kernel<TIn, TOut, MAXI_, true, FULL_>, dim3(grid), dim3(threads), 0, s, 1, xi, ri, gamma, beta, so, yo, eps, m, ni), "launch layernorm");  \
    else                                                                                          \
      check_cuda(launch_chain(layernorm_warp_kernel<TIn, TOut, MAXI_, false, FULL_>, dim3(grid), dim3(threads), 0, s, 1, xi, ri, gamma, beta, so, yo, eps, m, ni), "launch layernorm"); \
  } while (0)
#define MDC_LN_LAUNCH(MAXI_)                                                                          \
  do {                                                                                            \
    if (nchunks_host == 32 * (MAXI_) && !(sizeof(TIn) == 2 && (MAXI_) == 3)) MDC_LN_LAUNCH2(MAXI_, true); \
    else MDC_LN_LAUNCH2(MAXI_, false);                                                            \
  } while (0)
    if (per_lane <= 2) MDC_LN_LAUNCH(2);
    else if (per_lane <= 3) MDC_LN_LAUNCH(3);
    else if (per_lane <= 4) MDC_LN_LAUNCH(4);
    else if (per_lane <= 6) MDC_LN_LAUNCH(6);
    else if (per_lane <= 8) MDC_LN_LAUNCH(8);
    else MDC_LN_LAUNCH(16);
#undef MDC_LN_LAUNCH
#undef MDC_LN_LAUNCH2
    launched("layernorm_warp_kernel");
  } else {
    const size_t smem = static_cast<size_t>(n) * sizeof(float);
    if (smem > 200 * 1024) {
      fail("mgpuLayerNorm: row too long for the shared-memory kernel (n > 51200)");
      return;
    }
    auto kern = layernorm_block_kernel<TIn, TOut>;
    if (smem > 40 * 1024 &&  // static shared memory counts against the 48 KiB default too
        !check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)),
                    "cudaFuncSetAttribute(layernorm)"))
      return;
    kern<<<static_cast<unsigned>(m), 256, smem, s>>>(xi, ri, gamma, beta, so, yo, eps, m,
                                                     static_cast<int>(n));
    launched("layernorm_block_kernel");
  }
}

}  // namespace mdc

using namespace mdc;

MDC_API void mgpuLayerNormEx(const void *x, const void *residual, const float *gamma,
                             const float *beta, void *sum_out, void *y, float eps, int64_t m,
                             int64_t n, int32_t io_dtype, int32_t out_dtype, void *stream) {
  if (m <= 0 || n <= 0) return;
  if (!device_info().ok) return;
  if (m > 0x7fffffffLL * kLnWarpsPerBlock || n > 0x7fffffffLL) {
    fail("mgpuLayerNorm: shape too large");
    return;
  }
  cudaStream_t s = as_stream(stream);
  ProfileScope prof(kCatLayerNorm, s);
#define MDC_LN_CASE(IN_E, IN_T, OUT_E, OUT_T)                                                   \
  if (io_dtype == IN_E && out_dtype == OUT_E) {                                                 \
    launch_layernorm<IN_T, OUT_T>(x, residual, gamma, beta, sum_out, y, eps, m, n, s);          \
    return;                                                                                     \
  }
  MDC_LN_CASE(MGPU_DTYPE_F32, float, MGPU_DTYPE_F32, float)
  MDC_LN_CASE(MGPU_DTYPE_F16, __half, MGPU_DTYPE_F16, __half)
  MDC_LN_CASE(MGPU_DTYPE_BF16, __nv_bfloat16, MGPU_DTYPE_BF16, __nv_bfloat16)
  MDC_LN_CASE(MGPU_DTYPE_F16, __half, MGPU_DTYPE_F32, float)
  MDC_LN_CASE(MGPU_DTYPE_BF16, __nv_bfloat16, MGPU_DTYPE_F32, float)
  MDC_LN_CASE(MGPU_DTYPE_F32, float, MGPU_DTYPE_F16, __half)
  MDC_LN_CASE(MGPU_DTYPE_F32, float, MGPU_DTYPE_BF16, __nv_bfloat16)
#undef MDC_LN_CASE
  fail("mgpuLayerNormEx: unsupported element type combination");
}

MDC_API void mgpuLayerNormF32(const float *x, const float *gamma, const float *beta, float *y,
                              float eps, int64_t m, int64_t n, void *stream) {
  mgpuLayerNormEx(x, nullptr, gamma, beta, nullptr, y, eps, m, n, MGPU_DTYPE_F32, MGPU_DTYPE_F32,
                  stream);
}
