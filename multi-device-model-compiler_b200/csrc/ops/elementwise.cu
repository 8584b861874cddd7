// Entry points for the HBM-bound elementwise ops: Add / bias / activation (fp32), element
// type casts and the one-time weight packing (cast + transpose) for the tensor-core Gemm.
#include <vector>

#include "elementwise_kernels.cuh"
#include "ops_common.h"

namespace mdc {

std::atomic<uint64_t> g_launch_count{0};

bool pdl_enabled() {
  static const bool on = [] {
    const char *e = getenv("MDC_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

bool g_profiling = false;
namespace {
struct ProfileSpan {
  int cat;
  cudaEvent_t begin, end;
};
std::vector<ProfileSpan> g_spans;
std::vector<cudaEvent_t> g_spare_events;
cudaEvent_t timing_event() {
  if (!g_spare_events.empty()) {
    cudaEvent_t e = g_spare_events.back();
    g_spare_events.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
}  // namespace

void profile_mark(int category, cudaStream_t stream, bool begin) {
  if (begin) {
    ProfileSpan sp{category, timing_event(), timing_event()};
    cudaEventRecord(sp.begin, stream);
    g_spans.push_back(sp);
  } else if (!g_spans.empty()) {
    cudaEventRecord(g_spans.back().end, stream);
  }
}

const DeviceInfo &device_info() {
  static thread_local DeviceInfo info;
  int dev = -1;
  if (!check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) {
    info = DeviceInfo();
    return info;
  }
  // Everything the runtime library hands out (pool blocks, streams, tensor maps) belongs to the
  // device it selected for this thread; an op queued while another device is current would
  // mix the two.  Refuse instead: devices are chosen with mgpuSetDefaultDevice.
  const int rt_dev = mgpuGetDefaultDevice();
  if (rt_dev >= 0 && rt_dev != dev) {
    char msg[160];
    snprintf(msg, sizeof(msg),
             "the thread's current CUDA device (%d) is not the device the runtime selected for it (%d); "
             "choose devices with mgpuSetDefaultDevice", dev, rt_dev);
    fail(msg);
    info = DeviceInfo();
    return info;
  }
  if (info.ok && info.device == dev) return info;  // cached for the thread's current device
  info = DeviceInfo();
  cudaDeviceProp p;
  if (!check_cuda(cudaGetDeviceProperties(&p, dev), "cudaGetDeviceProperties")) return info;
  info.device = dev;
  info.sms = p.multiProcessorCount;
  info.cc_major = p.major;
  info.cc_minor = p.minor;
  if (p.major != 10) {
    fail("this library is built for sm_100a (Blackwell B200) only");
    return info;
  }
  info.ok = true;
  return info;
}

// ---- casts -------------------------------------------------------------------------
template <typename T>
struct Vec8;  // eight 16-bit elements = 16 bytes
template <>
struct Vec8<__half> {
  __half2 v[4];
};
template <>
struct Vec8<__nv_bfloat16> {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ __half2 pack2(float a, float b, __half) { return __floats2half2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 pack2(float a, float b, __nv_bfloat16) {
  return __floats2bfloat162_rn(a, b);
}
__device__ __forceinline__ float2 unpack2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 unpack2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }

// fp32 -> 16-bit: two float4 in, one 16-byte store out per item.
template <typename T16>
__global__ void __launch_bounds__(kEwBlock)
cast_f32_to_16(const float *__restrict__ src, T16 *__restrict__ dst, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (aligned16(src) && aligned16(dst)) {
    const int64_t nvec = n >> 3;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    Vec8<T16> *d8 = reinterpret_cast<Vec8<T16> *>(dst);
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const float4 a = __ldcs(s4 + 2 * i), b = __ldcs(s4 + 2 * i + 1);
      Vec8<T16> o;
      o.v[0] = pack2(a.x, a.y, T16());
      o.v[1] = pack2(a.z, a.w, T16());
      o.v[2] = pack2(b.x, b.y, T16());
      o.v[3] = pack2(b.z, b.w, T16());
      d8[i] = o;
    }
    for (int64_t j = (nvec << 3) + tid; j < n; j += nthreads) dst[j] = from_f32<T16>(src[j]);
  } else {
    for (int64_t j = tid; j < n; j += nthreads) dst[j] = from_f32<T16>(src[j]);
  }
}

template <typename T16>
__global__ void __launch_bounds__(kEwBlock)
cast_16_to_f32(const T16 *__restrict__ src, float *__restrict__ dst, int64_t n) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (aligned16(src) && aligned16(dst)) {
    const int64_t nvec = n >> 3;
    const Vec8<T16> *s8 = reinterpret_cast<const Vec8<T16> *>(src);
    float4 *d4 = reinterpret_cast<float4 *>(dst);
    for (int64_t i = tid; i < nvec; i += nthreads) {
      const Vec8<T16> v = s8[i];
      const float2 a = unpack2(v.v[0]), b = unpack2(v.v[1]), c = unpack2(v.v[2]), d = unpack2(v.v[3]);
      __stcs(d4 + 2 * i, make_float4(a.x, a.y, b.x, b.y));
      __stcs(d4 + 2 * i + 1, make_float4(c.x, c.y, d.x, d.y));
    }
    for (int64_t j = (nvec << 3) + tid; j < n; j += nthreads) dst[j] = to_f32(src[j]);
  } else {
    for (int64_t j = tid; j < n; j += nthreads) dst[j] = to_f32(src[j]);
  }
}

template <typename TS, typename TD>
__global__ void __launch_bounds__(kEwBlock)
cast_generic(const TS *__restrict__ src, TD *__restrict__ dst, int64_t n) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t j = tid; j < n; j += nthreads) dst[j] = from_f32<TD>(to_f32(src[j]));
}

// fp32 [R, C] -> 16-bit [R, Cp], columns C..Cp-1 zero (row padding for the Gemm's A operand
// when C is not a multiple of 8).
template <typename T16>
__global__ void __launch_bounds__(kEwBlock)
cast_pad_rows(const float *__restrict__ src, T16 *__restrict__ dst, int64_t R, int64_t C, int64_t Cp) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t n = R * Cp;
  for (int64_t j = tid; j < n; j += nthreads) {
    const int64_t r = j / Cp, c = j - r * Cp;
    dst[j] = from_f32<T16>(c < C ? src[r * C + c] : 0.f);
  }
}

// weight fp32 [K, N] (N contiguous) -> 16-bit [N, Kp] (K contiguous), zero padded to Kp.
// 64 x 64 tiles through shared memory: reads are 16-byte vectors along n (whole lines of w),
// writes are 16-byte vectors of eight 16-bit values along k (whole lines of out).
template <typename T16>
__global__ void __launch_bounds__(256)
pack_weight_kernel(const float *__restrict__ w, T16 *__restrict__ out, int64_t K, int64_t N, int64_t Kp, int vec_ok) {
  __shared__ float tile[64][65];
  const int64_t k0 = static_cast<int64_t>(blockIdx.y) * 64;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 64;
  {
    const int c4 = (threadIdx.x & 15) * 4, r0 = threadIdx.x >> 4;  // 16 threads per k-row, 16 rows per pass
#pragma unroll
    for (int r = r0; r < 64; r += 16) {
      const int64_t k = k0 + r, n = n0 + c4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < K) {
        if (vec_ok && n + 3 < N) {
          v = __ldg(reinterpret_cast<const float4 *>(w + k * N + n));
        } else {
          if (n < N) v.x = w[k * N + n];
          if (n + 1 < N) v.y = w[k * N + n + 1];
          if (n + 2 < N) v.z = w[k * N + n + 2];
          if (n + 3 < N) v.w = w[k * N + n + 3];
        }
      }
      tile[r][c4] = v.x, tile[r][c4 + 1] = v.y, tile[r][c4 + 2] = v.z, tile[r][c4 + 3] = v.w;
    }
  }
  __syncthreads();
  {
    const int kg = (threadIdx.x & 7) * 8, r0 = threadIdx.x >> 3;  // 8 threads per n-row, 32 rows per pass
#pragma unroll
    for (int r = r0; r < 64; r += 32) {
      const int64_t n = n0 + r, k = k0 + kg;
      if (n < N && k < Kp) {  // Kp is a multiple of 8: a group of eight is inside or outside as a whole
        __align__(16) T16 h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = from_f32<T16>(tile[kg + e][r]);
        *reinterpret_cast<uint4 *>(out + n * Kp + k) = *reinterpret_cast<const uint4 *>(h);
      }
    }
  }
}


}  // namespace mdc

using namespace mdc;

MDC_API uint64_t mgpuOpsLaunchCount(void) { return g_launch_count.load(); }

MDC_API void mgpuOpsProfileBegin(void) {
  g_spans.clear();
  g_profiling = true;
}

// Like mgpuOpsProfileEnd, but returns every launch separately, in launch order: its
// category and its device time.  Returns the number of launches written (at most `capacity`).
MDC_API int64_t mgpuOpsProfileEndSpans(int32_t *category, float *ms, int64_t capacity) {
  g_profiling = false;
  int64_t n = 0;
  for (ProfileSpan &sp : g_spans) {
    float t = 0.f;
    if (cudaEventSynchronize(sp.end) == cudaSuccess && cudaEventElapsedTime(&t, sp.begin, sp.end) == cudaSuccess) {
      if (n < capacity) {
        if (category) category[n] = sp.cat;
        if (ms) ms[n] = t;
        ++n;
      }
    } else {
      (void)cudaGetLastError();
    }
    g_spare_events.push_back(sp.begin);
    g_spare_events.push_back(sp.end);
  }
  g_spans.clear();
  return n;
}

MDC_API void mgpuOpsProfileEnd(double *ms_per_category, uint64_t *launches_per_category) {
  g_profiling = false;
  for (int c = 0; c < kNumCategories; ++c) {
    if (ms_per_category) ms_per_category[c] = 0.0;
    if (launches_per_category) launches_per_category[c] = 0;
  }
  for (ProfileSpan &sp : g_spans) {
    float ms = 0.f;
    if (cudaEventSynchronize(sp.end) == cudaSuccess && cudaEventElapsedTime(&ms, sp.begin, sp.end) == cudaSuccess) {
      if (ms_per_category) ms_per_category[sp.cat] += ms;
      if (launches_per_category) launches_per_category[sp.cat] += 1;
    } else {
      (void)cudaGetLastError();
    }
    g_spare_events.push_back(sp.begin);
    g_spare_events.push_back(sp.end);
  }
  g_spans.clear();
}

MDC_API void mgpuAdd(const float *a, const float *b, float *c, int64_t n, void *stream) {
  if (n <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  ProfileScope prof(kCatElementwise, as_stream(stream));
  mdc_add_f32<<<ew_grid((n + 3) / 4, di.sms), kEwBlock, 0, as_stream(stream)>>>(a, b, c, n);
  launched("mdc_add_f32");
}

MDC_API void mgpuBiasAdd(const float *x, const float *bias, float *y, int64_t rows, int64_t cols,
                         void *stream) {
  if (rows <= 0 || cols <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  mdc_bias_add_f32<<<ew_grid((rows * cols + 3) / 4, di.sms), kEwBlock, 0, as_stream(stream)>>>(
      x, bias, y, rows, cols);
  launched("mdc_bias_add_f32");
}

MDC_API void mgpuActivation(const float *x, float *y, int64_t n, int32_t act, void *stream) {
  if (n <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  const int grid = ew_grid((n + 3) / 4, di.sms);
  cudaStream_t s = as_stream(stream);
  switch (act) {
  case MGPU_ACT_RELU:
    mdc_relu_f32<<<grid, kEwBlock, 0, s>>>(x, y, n);
    break;
  case MGPU_ACT_GELU_ERF:
    mdc_gelu_erf_f32<<<grid, kEwBlock, 0, s>>>(x, y, n);
    break;
  case MGPU_ACT_GELU_TANH:
    mdc_gelu_tanh_f32<<<grid, kEwBlock, 0, s>>>(x, y, n);
    break;
  case MGPU_ACT_NONE:
    if (x != y) check_cuda(cudaMemcpyAsync(y, x, n * sizeof(float), cudaMemcpyDeviceToDevice, s), "copy");
    return;
  default:
    fail("mgpuActivation: unknown activation");
    return;
  }
  launched("mdc_activation");
}

MDC_API void mgpuCast(const void *src, int32_t sd, void *dst, int32_t dd, int64_t n, void *stream) {
  if (n <= 0) return;
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  cudaStream_t s = as_stream(stream);
  const int grid = ew_grid((n + 7) / 8, di.sms);
  ProfileScope prof(kCatElementwise, s);
  if (sd == dd) {
    if (src != dst)
      check_cuda(cudaMemcpyAsync(dst, src, n * dtype_size(sd), cudaMemcpyDeviceToDevice, s), "copy");
    return;
  }
  if (sd == MGPU_DTYPE_F32 && dd == MGPU_DTYPE_F16)
    check_cuda(launch_chain(cast_f32_to_16<__half>, dim3(grid), dim3(kEwBlock), 0, s, 1, (const float *)src, (__half *)dst, n), "launch cast");
  else if (sd == MGPU_DTYPE_F32 && dd == MGPU_DTYPE_BF16)
    check_cuda(launch_chain(cast_f32_to_16<__nv_bfloat16>, dim3(grid), dim3(kEwBlock), 0, s, 1, (const float *)src, (__nv_bfloat16 *)dst, n), "launch cast");
  else if (sd == MGPU_DTYPE_F16 && dd == MGPU_DTYPE_F32)
    cast_16_to_f32<__half><<<grid, kEwBlock, 0, s>>>((const __half *)src, (float *)dst, n);
  else if (sd == MGPU_DTYPE_BF16 && dd == MGPU_DTYPE_F32)
    cast_16_to_f32<__nv_bfloat16><<<grid, kEwBlock, 0, s>>>((const __nv_bfloat16 *)src, (float *)dst, n);
  else if (sd == MGPU_DTYPE_F16 && dd == MGPU_DTYPE_BF16)
    cast_generic<__half, __nv_bfloat16><<<grid, kEwBlock, 0, s>>>((const __half *)src, (__nv_bfloat16 *)dst, n);
  else if (sd == MGPU_DTYPE_BF16 && dd == MGPU_DTYPE_F16)
    cast_generic<__nv_bfloat16, __half><<<grid, kEwBlock, 0, s>>>((const __nv_bfloat16 *)src, (__half *)dst, n);
  else {
    fail("mgpuCast: unknown element type");
    return;
  }
  launched("mdc_cast");
}

namespace mdc {
// fp32 [R,C] -> 16-bit [R,Cp]; plain cast when C == Cp.
void cast_rows_padded(const float *src, void *dst, int64_t R, int64_t C, int64_t Cp, int32_t dtype,
                      cudaStream_t s) {
  if (C == Cp) {
    mgpuCast(src, MGPU_DTYPE_F32, dst, dtype, R * C, s);
    return;
  }
  const DeviceInfo &di = device_info();
  if (!di.ok) return;
  const int grid = ew_grid(R * Cp, di.sms);
  if (dtype == MGPU_DTYPE_F16)
    cast_pad_rows<__half><<<grid, kEwBlock, 0, s>>>(src, (__half *)dst, R, C, Cp);
  else
    cast_pad_rows<__nv_bfloat16><<<grid, kEwBlock, 0, s>>>(src, (__nv_bfloat16 *)dst, R, C, Cp);
  launched("mdc_cast_pad_rows");
}
}  // namespace mdc

MDC_API void mgpuPackWeight(const float *w, void *packed, int64_t K, int64_t N, int32_t dtype,
                            void *stream) {
  if (K <= 0 || N <= 0) return;
  if (!dtype_is16(dtype)) {
    fail("mgpuPackWeight: dtype must be F16 or BF16");
    return;
  }
  if (!device_info().ok) return;
  const int64_t Kp = (K + 7) / 8 * 8;
  if (reinterpret_cast<uintptr_t>(packed) & 15u) { fail("mgpuPackWeight: the packed buffer must be 16-byte aligned"); return; }
  dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((Kp + 63) / 64));
  const int vec_ok = (N % 4 == 0) && !(reinterpret_cast<uintptr_t>(w) & 15u);
  if (dtype == MGPU_DTYPE_F16)
    pack_weight_kernel<__half><<<grid, 256, 0, as_stream(stream)>>>(w, (__half *)packed, K, N, Kp, vec_ok);
  else
    pack_weight_kernel<__nv_bfloat16><<<grid, 256, 0, as_stream(stream)>>>(w, (__nv_bfloat16 *)packed, K, N, Kp, vec_ok);
  launched("mdc_pack_weight");
}
