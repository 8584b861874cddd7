// libMultiDeviceCUDARuntime.so: the mgpu* C ABI that lowered graphs call for streams,
// events, device memory, copies, module loading and kernel launches.  Same symbols and
// argument meaning as the reference's lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:91-384;
// the implementation is new: the CUDA runtime API with the primary context (so the op
// library, which launches with <<<>>>, shares it), a caching stream-ordered device pool,
// a registry of built-in hand-written kernels, and a sticky error status.
//
// The library links the static CUDA runtime only.  The few driver-API calls that have no
// runtime twin (module load, raw launch, tensor-map encode, 16/32-bit memset) are resolved
// through cudaGetDriverEntryPoint, so the library loads on a machine without a driver and
// fails at the first call instead.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <condition_variable>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <iterator>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../ops/elementwise_kernels.cuh"
#include "device_pool.h"
#include "mdc_gpu_runtime.h"

#define MDC_API extern "C" __attribute__((visibility("default")))

namespace {

// Device selection is per host thread.  mgpuSetDefaultDevice(k) is the supported way to choose
// a GPU; a thread that never called it adopts the device that is current on it (the one a
// plain cudaSetDevice chose, ordinal 0 otherwise) at its first runtime call, and the op
// library refuses to run while the thread's current CUDA device differs from this one.
thread_local int32_t g_default_device = 0;
thread_local bool g_device_chosen = false;  // by mgpuSetDefaultDevice on this thread
thread_local bool g_device_bound = false;

// Guards the process-wide tables below (constants, parked streams / events, kernel handle
// caches, overrides).  The calls that touch them are short; one mutex is enough.
std::recursive_mutex g_state_mu;
// Serialises the staged pageable-copy path (one pinned ring and one helper team per process);
// a thread that finds it taken uses the driver's plain copy instead of waiting.
std::mutex g_stage_mu;

std::mutex g_err_mu;
int32_t g_last_error = 0;
std::string g_last_error_msg;

bool debug_enabled() {
  static const bool on = getenv("MULTI_DEVICE_CUDA_DEBUG") != nullptr;
  return on;
}

void record_error(int32_t code, const char *what, const char *detail) {
  fprintf(stderr, "'%s' failed with '%s'\n", what, detail ? detail : "<unknown>");
  std::lock_guard<std::mutex> lock(g_err_mu);
  if (g_last_error == 0) {
    g_last_error = code ? code : -1;
    g_last_error_msg = std::string(what) + ": " + (detail ? detail : "<unknown>");
  }
}

bool rt_ok(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return true;
  record_error(static_cast<int32_t>(e), what, cudaGetErrorName(e));
  (void)cudaGetLastError();
  return false;
}
#define RT_CHECK(expr) rt_ok((expr), #expr)

// Binds the calling thread to the default device's primary context on first use.
bool ensure_device() {
  if (g_device_bound) return true;
  if (!g_device_chosen) {
    int cur = 0;
    if (!RT_CHECK(cudaGetDevice(&cur))) return false;
    g_default_device = cur;
  }
  if (!RT_CHECK(cudaSetDevice(g_default_device))) return false;
  if (!RT_CHECK(cudaFree(nullptr))) return false;  // forces context creation
  g_device_bound = true;
  return true;
}

// ---- driver entry points without a runtime-API twin ----
struct DriverApi {
  CUresult (*ModuleLoad)(CUmodule *, const char *) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           unsigned, CUstream, void **, void **) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*MemsetD32Async)(CUdeviceptr, unsigned, size_t, CUstream) = nullptr;
  CUresult (*MemsetD16Async)(CUdeviceptr, unsigned short, size_t, CUstream) = nullptr;
  CUresult (*GetErrorName)(CUresult, const char **) = nullptr;
  CUresult (*TensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  bool ok = false;
};

template <typename F>
bool resolve(const char *name, F *out) {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    (void)cudaGetLastError();
    record_error(e ? static_cast<int32_t>(e) : -1, name, "driver entry point not found");
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

DriverApi &driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    bool ok = true;
    ok &= resolve("cuModuleLoad", &api.ModuleLoad);
    ok &= resolve("cuModuleUnload", &api.ModuleUnload);
    ok &= resolve("cuModuleGetFunction", &api.ModuleGetFunction);
    ok &= resolve("cuLaunchKernel", &api.LaunchKernel);
    ok &= resolve("cuFuncSetAttribute", &api.FuncSetAttribute);
    ok &= resolve("cuMemsetD32Async", &api.MemsetD32Async);
    ok &= resolve("cuMemsetD16Async", &api.MemsetD16Async);
    ok &= resolve("cuGetErrorName", &api.GetErrorName);
    ok &= resolve("cuTensorMapEncodeTiled", &api.TensorMapEncodeTiled);
    api.ok = ok;
  });
  return api;
}

bool drv_ok(CUresult r, const char *what) {
  if (r == CUDA_SUCCESS) return true;
  const char *name = nullptr;
  if (driver().GetErrorName) driver().GetErrorName(r, &name);
  record_error(static_cast<int32_t>(r), what, name);
  return false;
}
#define DRV_CHECK(expr) drv_ok((expr), #expr)

// ---- module + built-in kernel registry ----
CUmodule g_module = nullptr;
std::unordered_map<std::string, const void *> &builtin_symbols() {
  static std::unordered_map<std::string, const void *> m = {
      {"mdc_add_f32", reinterpret_cast<const void *>(&mdc::mdc_add_f32)},
      {"mdc_bias_add_f32", reinterpret_cast<const void *>(&mdc::mdc_bias_add_f32)},
      {"mdc_relu_f32", reinterpret_cast<const void *>(&mdc::mdc_relu_f32)},
      {"mdc_gelu_erf_f32", reinterpret_cast<const void *>(&mdc::mdc_gelu_erf_f32)},
      {"mdc_gelu_tanh_f32", reinterpret_cast<const void *>(&mdc::mdc_gelu_tanh_f32)},
  };
  return m;
}
std::unordered_map<std::string, CUfunction> g_builtin_cache;
// functions whose dynamic shared memory limit has already been raised to at least this
std::unordered_map<CUfunction, int32_t> g_smem_limit;

// Kernel overrides: a name pattern of a module kernel generated by the reference toolchain,
// routed to a built-in kernel.  The generated kernel takes `operands` contiguous memrefs of
// one rank, each expanded to (allocated, aligned, offset, sizes[rank], strides[rank]).
struct KernelOverride {
  std::string pattern;   // exact name, or a prefix followed by '*'
  std::string builtin;
  int rank = 1, operands = 3;  // rank 0: bare-pointer arguments (one pointer per operand)
  int64_t elements = 0;        // bare form: element count, 0 = grid x block of the launch
  CUfunction target = nullptr;
  int target_device = -1;      // the device `target` was resolved on
};
std::vector<KernelOverride *> g_overrides;          // entries are never freed: they are handed out as handles
std::unordered_set<const void *> g_override_handles;

bool pattern_matches(const std::string &pattern, const char *name) {
  if (!pattern.empty() && pattern.back() == '*') return strncmp(name, pattern.c_str(), pattern.size() - 1) == 0;
  return pattern == name;
}

constexpr int kMaxDevices = 64;
constexpr size_t kMaxParked = 64;
struct ObjectCache {
  std::vector<cudaStream_t> streams;
  std::vector<cudaEvent_t> events;
  std::unordered_set<cudaEvent_t> untimed;  // events created by mgpuEventCreate
};
ObjectCache g_object_caches[kMaxDevices];
ObjectCache &object_cache() {
  int d = g_default_device;
  if (d < 0 || d >= kMaxDevices) d = 0;
  return g_object_caches[d];
}
// Host buffers the caller declared immutable (model weights): a device-resident copy is
// made at the first upload and later uploads become device-to-device copies.
struct Constant {
  uint64_t bytes = 0;
  int device = 0;
  void *dev = nullptr;
  cudaEvent_t uploaded = nullptr;
  cudaEvent_t last_use = nullptr;  // recorded after every copy served from `dev`
  // buffers an op derived from this constant (e.g. a packed 16-bit copy of a weight), by tag
  struct Derived {
    void *dev = nullptr;
    uint64_t bytes = 0;
    cudaEvent_t ready = nullptr;  // recorded once the op has filled it
    bool filled = false;
  };
  std::unordered_map<uint64_t, Derived> derived;
};
std::unordered_map<const void *, Constant> g_constants;
// device buffers whose whole content is a copy of a registered constant: buffer -> host key.
// Entered by mgpuMemcpy when it serves a copy from a constant into the START of a block,
// dropped when the buffer is freed or is the destination of another copy or memset.
std::unordered_map<const void *, const void *> g_copies_of_constants;
mdc::DevicePool g_pools[kMaxDevices];
mdc::DevicePool &pool() {
  int d = g_default_device;
  if (d < 0 || d >= kMaxDevices) d = 0;
  return g_pools[d];
}


// ---- staged copies between pageable host memory and the device ----
// cudaMemcpyAsync on pageable memory goes through the driver's single-threaded bounce
// buffer.  Large copies are instead cut into chunks that a small team of host threads moves
// into / out of a ring of pinned buffers while the copy engine works on the previous chunk.
class CopyTeam {
 public:
  explicit CopyTeam(int helpers) {
    for (int i = 0; i < helpers; ++i) std::thread([this, i] { work(i); }).detach();
    helpers_ = helpers;
  }
  // memcpy(dst, src, n) split over the helpers and the calling thread
  void copy(char *dst, const char *src, size_t n) {
    const int parts = helpers_ + 1;
    if (helpers_ == 0 || n < (size_t(256) << 10)) {
      memcpy(dst, src, n);
      return;
    }
    const size_t per = ((n + parts - 1) / parts + 63) & ~size_t(63);
    {
      std::lock_guard<std::mutex> lock(mu_);
      dst_ = dst, src_ = src, n_ = n, per_ = per;
      pending_ = helpers_;
      ++generation_;
    }
    wake_.notify_all();
    if (per * helpers_ < n) memcpy(dst + per * helpers_, src + per * helpers_, n - per * helpers_);
    std::unique_lock<std::mutex> lock(mu_);
    done_.wait(lock, [this] { return pending_ == 0; });
  }

 private:
  void work(int index) {
    uint64_t seen = 0;
    for (;;) {
      char *dst;
      const char *src;
      size_t n, per;
      {
        std::unique_lock<std::mutex> lock(mu_);
        wake_.wait(lock, [&] { return generation_ != seen; });
        seen = generation_;
        dst = dst_, src = src_, n = n_, per = per_;
      }
      const size_t begin = per * index;
      if (begin < n) memcpy(dst + begin, src + begin, (n - begin < per) ? n - begin : per);
      std::lock_guard<std::mutex> lock(mu_);
      if (--pending_ == 0) done_.notify_one();
    }
  }
  std::mutex mu_;
  std::condition_variable wake_, done_;
  char *dst_ = nullptr;
  const char *src_ = nullptr;
  size_t n_ = 0, per_ = 0;
  int pending_ = 0, helpers_ = 0;
  uint64_t generation_ = 0;
};

CopyTeam &copy_team() {
  // never destroyed: its helper threads may still be parked when the process exits
  static CopyTeam *team = [] {
    // measured on a 16-core host, 256 MiB: upload 11 GB/s through the driver's own path,
    // 12 / 21 / 30 / 43 GB/s with 1 / 2 / 4 / 8 threads; download 18 vs 9 / 16 / 17 / 28
    const int hw = static_cast<int>(std::thread::hardware_concurrency());
    int threads = hw >= 16 ? 8 : (hw >= 2 ? hw / 2 : 1);
    if (const char *e = getenv("MDC_COPY_THREADS")) threads = atoi(e);
    if (hw > 0 && threads > hw) threads = hw;
    if (threads < 1) threads = 1;
    return new CopyTeam(threads - 1);
  }();
  return *team;
}

constexpr size_t kStageChunk = size_t(4) << 20;
constexpr size_t kStageThreshold = size_t(1) << 20;  // smaller copies take the plain path
constexpr int kStageSlots = 4;
struct StagingRing {
  char *slot[kStageSlots] = {};
  cudaEvent_t done[kStageSlots] = {};
  bool busy[kStageSlots] = {};
  bool ready = false, failed = false;
};
StagingRing g_staging[kMaxDevices];

StagingRing *staging_ring() {
  static const bool off = getenv("MDC_STAGED_COPY") && atoi(getenv("MDC_STAGED_COPY")) == 0;
  if (off) return nullptr;
  int d = g_default_device;
  if (d < 0 || d >= kMaxDevices) d = 0;
  StagingRing &r = g_staging[d];
  if (r.failed) return nullptr;
  if (!r.ready) {
    for (int i = 0; i < kStageSlots; ++i) {
      if (cudaHostAlloc(reinterpret_cast<void **>(&r.slot[i]), kStageChunk, cudaHostAllocDefault) != cudaSuccess ||
          cudaEventCreateWithFlags(&r.done[i], cudaEventDisableTiming) != cudaSuccess) {
        (void)cudaGetLastError();
        r.failed = true;  // the plain path still works
        return nullptr;
      }
    }
    r.ready = true;
  }
  return &r;
}

enum class MemKind { PageableHost, PinnedHost, Device, Unknown };
MemKind mem_kind(const void *p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return MemKind::Unknown;
  }
  switch (attr.type) {
    case cudaMemoryTypeUnregistered: return MemKind::PageableHost;
    case cudaMemoryTypeHost: return MemKind::PinnedHost;
    case cudaMemoryTypeDevice: return MemKind::Device;
    default: return MemKind::Unknown;  // managed memory: leave it to the driver
  }
}

// Returns true when the copy was carried out (or failed and was reported) here.
bool staged_copy(void *dst, const void *src, size_t bytes, cudaStream_t s) {
  if (bytes < kStageThreshold) return false;
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return false;
  }
  const MemKind sk = mem_kind(src), dk = mem_kind(dst);
  const bool up = sk == MemKind::PageableHost && dk == MemKind::Device;
  const bool down = sk == MemKind::Device && dk == MemKind::PageableHost;
  if (!up && !down) return false;
  // one staged copy at a time in the process: a second thread takes the plain path
  std::unique_lock<std::mutex> stage_lock(g_stage_mu, std::try_to_lock);
  if (!stage_lock.owns_lock()) return false;
  StagingRing *ring = staging_ring();
  if (!ring) return false;
  CopyTeam &team = copy_team();
  const size_t chunks = (bytes + kStageChunk - 1) / kStageChunk;
  auto span = [&](size_t c) { return (c + 1 == chunks) ? bytes - c * kStageChunk : kStageChunk; };
  if (up) {
    // like the driver's pageable path: returns once the source has been read, not once it
    // has arrived
    for (size_t c = 0; c < chunks; ++c) {
      const int i = static_cast<int>(c % kStageSlots);
      if (ring->busy[i] && !RT_CHECK(cudaEventSynchronize(ring->done[i]))) return true;
      team.copy(ring->slot[i], static_cast<const char *>(src) + c * kStageChunk, span(c));
      if (!RT_CHECK(cudaMemcpyAsync(static_cast<char *>(dst) + c * kStageChunk, ring->slot[i], span(c),
                                    cudaMemcpyHostToDevice, s)) ||
          !RT_CHECK(cudaEventRecord(ring->done[i], s)))
        return true;
      ring->busy[i] = true;
    }
    return true;
  }
  // download: keep the copy engine kStageSlots chunks ahead of the host threads; complete on
  // return, as a copy into pageable memory is
  for (int i = 0; i < kStageSlots; ++i)
    if (ring->busy[i]) {
      if (!RT_CHECK(cudaEventSynchronize(ring->done[i]))) return true;
      ring->busy[i] = false;
    }
  size_t issued = 0;
  for (size_t c = 0; c < chunks; ++c) {
    for (; issued < chunks && issued < c + kStageSlots; ++issued) {
      const int j = static_cast<int>(issued % kStageSlots);
      if (!RT_CHECK(cudaMemcpyAsync(ring->slot[j], static_cast<const char *>(src) + issued * kStageChunk,
                                    span(issued), cudaMemcpyDeviceToHost, s)) ||
          !RT_CHECK(cudaEventRecord(ring->done[j], s)))
        return true;
    }
    const int i = static_cast<int>(c % kStageSlots);
    if (!RT_CHECK(cudaEventSynchronize(ring->done[i]))) return true;
    team.copy(static_cast<char *>(dst) + c * kStageChunk, ring->slot[i], span(c));
  }
  return true;
}

int num_sms() {
  static thread_local int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      sms = 148;
    }
  }
  return sms;
}

// MLIR strided memref descriptor of rank-1 char (rank taken at run time).
struct MemRefDesc {
  char *basePtr;
  char *data;
  int64_t offset;
  int64_t sizes_and_strides[1];  // sizes[rank] then strides[rank]
};

}  // namespace

// ---------------- status ----------------
MDC_API int32_t mgpuGetLastError(void) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  return g_last_error;
}
MDC_API const char *mgpuGetLastErrorString(void) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  static thread_local std::string copy;
  copy = g_last_error_msg;
  return copy.c_str();
}
MDC_API void mgpuClearLastError(void) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  g_last_error = 0;
  g_last_error_msg.clear();
}
MDC_API void mgpuSetLastError(int32_t code, const char *what) {
  record_error(code, what ? what : "op", "reported by the op library");
}

// ---------------- module / launch ----------------
MDC_API void mgpuModuleFileLoad(const char *fname) {
  if (!ensure_device() || !driver().ok) return;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  if (g_module) {
    DRV_CHECK(driver().ModuleUnload(g_module));
    g_module = nullptr;
  }
  if (!fname || !*fname) return;
  FILE *f = fopen(fname, "rb");
  if (!f) {
    // Graphs made only of built-in kernels need no module file.
    if (debug_enabled()) fprintf(stderr, "mgpuModuleFileLoad: '%s' not found, built-ins only\n", fname);
    return;
  }
  fclose(f);
  DRV_CHECK(driver().ModuleLoad(&g_module, fname));
}

MDC_API void mgpuModuleUnload(void) {
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  if (g_module && driver().ok) {
    DRV_CHECK(driver().ModuleUnload(g_module));
    g_module = nullptr;
  }
}

MDC_API mgpu_function_t mgpuModuleGetFunction(const char *name) {
  if (!name || !ensure_device() || !driver().ok) return nullptr;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  // a function handle belongs to the context it was resolved in: the cache is per device
  const std::string key = std::to_string(g_default_device) + ":" + name;
  auto cached = g_builtin_cache.find(key);
  if (cached != g_builtin_cache.end()) return cached->second;
  auto sym = builtin_symbols().find(name);
  if (sym != builtin_symbols().end()) {
    cudaFunction_t fn = nullptr;
    if (!RT_CHECK(cudaGetFuncBySymbol(&fn, sym->second))) return nullptr;
    g_builtin_cache[key] = reinterpret_cast<CUfunction>(fn);
    return fn;
  }
  // a module kernel that the caller routed to a built-in one
  for (KernelOverride *o : g_overrides)
    if (!o->pattern.empty() && pattern_matches(o->pattern, name)) {
      if (!o->target || o->target_device != g_default_device) {
        o->target = reinterpret_cast<CUfunction>(mgpuModuleGetFunction(o->builtin.c_str()));
        o->target_device = g_default_device;
      }
      return o->target ? o : nullptr;
    }
  CUfunction function = nullptr;
  if (!g_module) {
    record_error(-1, name, "no such built-in kernel and no module loaded");
    return nullptr;
  }
  DRV_CHECK(driver().ModuleGetFunction(&function, g_module, name));
  return function;
}

MDC_API void mgpuLaunchKernel(mgpu_function_t function, intptr_t gridX, intptr_t gridY,
                              intptr_t gridZ, intptr_t blockX, intptr_t blockY, intptr_t blockZ,
                              int32_t smem, mgpu_stream_t stream, void **params, void **extra) {
  if (!function) {
    record_error(-1, "mgpuLaunchKernel", "null function");
    return;
  }
  if (!ensure_device() || !driver().ok) return;
  bool is_override;
  {
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    is_override = g_override_handles.count(function) != 0;
  }
  if (is_override) {
    // The caller passes the generated kernel's own arguments.  The built-in takes the data
    // pointers and the element count and chooses its own launch shape.
    //  * bare-pointer form (what the reference's GPU pipeline emits, lib/Pipelines/
    //    MLIRToGPU.cpp:162-165,180-183: one pointer per operand, shapes static and known only
    //    to the generated code): the element count comes from the registration, or from the
    //    caller's grid x block when registered as 0;
    //  * memref form: per operand (allocated, aligned, offset, sizes[rank], strides[rank]).
    const KernelOverride *o = static_cast<const KernelOverride *>(function);
    const int per = 3 + 2 * o->rank;
    void *ptrs[3] = {nullptr, nullptr, nullptr};
    int64_t n = 1;
    if (o->rank == 0) {
      for (int op = 0; op < o->operands; ++op) ptrs[op] = *static_cast<void **>(params[op]);
      n = o->elements > 0 ? o->elements
                          : static_cast<int64_t>(gridX) * gridY * gridZ * blockX * blockY * blockZ;
    }
    for (int op = 0; o->rank > 0 && op < o->operands; ++op) {
      void **g = params + op * per;
      char *aligned = *static_cast<char **>(g[1]);
      const int64_t offset = *static_cast<int64_t *>(g[2]);
      ptrs[op] = aligned + offset * 4;
      int64_t count = 1, expect = 1;
      for (int d = o->rank - 1; d >= 0; --d) {
        const int64_t size = *static_cast<int64_t *>(g[3 + d]), stride = *static_cast<int64_t *>(g[3 + o->rank + d]);
        if (size != 1 && stride != expect) {
          record_error(-1, "mgpuLaunchKernel", "an overridden kernel needs contiguous operands");
          return;
        }
        expect *= size;
        count *= size;
      }
      if (op == 0) n = count;
      else if (count != n) {
        record_error(-1, "mgpuLaunchKernel", "an overridden kernel needs operands of one size");
        return;
      }
    }
    intptr_t grid = 1, block = 1;
    mgpuBuiltinLaunchShape(n, &grid, &block);
    void *args3[] = {&ptrs[0], &ptrs[1], &ptrs[2], &n};
    void *args2[] = {&ptrs[0], &ptrs[1], &n};
    if (n > 0)
      DRV_CHECK(driver().LaunchKernel(o->target, (unsigned)grid, 1, 1, (unsigned)block, 1, 1, 0,
                                      reinterpret_cast<CUstream>(stream), o->operands == 3 ? args3 : args2, nullptr));
    return;
  }
  CUfunction fn = reinterpret_cast<CUfunction>(function);
  // Raise the dynamic shared-memory limit only when a launch needs more than the default
  // 48 KiB and more than was already granted (the reference queries the device and sets
  // the attribute on every launch, CudaRuntimeWrappers.cpp:118-131).
  if (smem > 48 * 1024) {
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    auto it = g_smem_limit.find(fn);
    if (it == g_smem_limit.end() || it->second < smem) {
      if (!DRV_CHECK(driver().FuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                               smem)))
        return;
      g_smem_limit[fn] = smem;
    }
  }
  if (debug_enabled())
    fprintf(stderr, "Launching kernel, grid=%ld,%ld,%ld, threads: %ld, %ld, %ld, smem: %d B\n",
            (long)gridX, (long)gridY, (long)gridZ, (long)blockX, (long)blockY, (long)blockZ, smem);
  DRV_CHECK(driver().LaunchKernel(fn, (unsigned)gridX, (unsigned)gridY, (unsigned)gridZ,
                                  (unsigned)blockX, (unsigned)blockY, (unsigned)blockZ,
                                  (unsigned)smem, reinterpret_cast<CUstream>(stream), params,
                                  extra));
}

MDC_API void mgpuBuiltinLaunchShape(int64_t n, intptr_t *gridX, intptr_t *blockX) {
  if (blockX) *blockX = mdc::kEwBlock;
  if (gridX) *gridX = mdc::ew_grid((n + 3) / 4, ensure_device() ? num_sms() : 148);
}

// ---------------- streams / events ----------------
// A lowered graph creates and destroys two streams and two events on every call
// (lib/Dialect/Device/Transform/AsyncDependencyConvert.cpp:49-56,135-139).  Destroyed
// objects are parked per device and handed out again: a parked stream may still have work
// queued, which is harmless because whatever is submitted next is ordered behind it.
MDC_API mgpu_stream_t mgpuStreamCreate(void) {
  if (!ensure_device()) return nullptr;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  ObjectCache &c = object_cache();
  if (!c.streams.empty()) {
    cudaStream_t s = c.streams.back();
    c.streams.pop_back();
    return s;
  }
  cudaStream_t s = nullptr;
  RT_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  return s;
}
MDC_API void mgpuStreamDestroy(mgpu_stream_t stream) {
  if (!stream) return;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  ObjectCache &c = object_cache();
  if (c.streams.size() < kMaxParked) {
    c.streams.push_back(static_cast<cudaStream_t>(stream));
    return;
  }
  RT_CHECK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
}
MDC_API void mgpuStreamSynchronize(mgpu_stream_t stream) {
  RT_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}
MDC_API void mgpuStreamWaitEvent(mgpu_stream_t stream, mgpu_event_t event) {
  RT_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
}
MDC_API mgpu_event_t mgpuEventCreate(void) {
  if (!ensure_device()) return nullptr;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  ObjectCache &c = object_cache();
  if (!c.events.empty()) {
    cudaEvent_t e = c.events.back();
    c.events.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  RT_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  c.untimed.insert(e);
  return e;
}
MDC_API mgpu_event_t mgpuEventCreateWithStream(mgpu_stream_t /*stream*/) { return mgpuEventCreate(); }
MDC_API mgpu_event_t mgpuEventEnableTimeCreate(void) {
  if (!ensure_device()) return nullptr;
  cudaEvent_t e = nullptr;
  RT_CHECK(cudaEventCreateWithFlags(&e, cudaEventDefault));
  return e;
}
MDC_API void mgpuEventDestroy(mgpu_event_t event) {
  if (!event) return;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  ObjectCache &c = object_cache();
  cudaEvent_t e = static_cast<cudaEvent_t>(event);
  // only the plain (timing-disabled) events are parked; timing events are rare
  if (c.untimed.count(e) && c.events.size() < kMaxParked) {
    c.events.push_back(e);
    return;
  }
  c.untimed.erase(e);
  RT_CHECK(cudaEventDestroy(e));
}
MDC_API void mgpuEventSynchronize(mgpu_event_t event) {
  RT_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
}
MDC_API void mgpuEventRecord(mgpu_event_t event, mgpu_stream_t stream) {
  RT_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}
MDC_API float mgpuEventElapsedTime(mgpu_event_t begin, mgpu_event_t end) {
  float ms = 0.f;
  RT_CHECK(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(begin), static_cast<cudaEvent_t>(end)));
  return ms;
}

// ---------------- memory ----------------
// Guard bands (MDC_POOL_GUARD=1, a debugging aid that stands in for a memory checker): every
// block handed out is preceded and followed by kGuardBytes of a fixed pattern inside the same
// pool block; mgpuMemFree reads both bands back (which synchronises the stream) and reports
// an overwritten band through the sticky status, naming the block.  Out-of-range writes by a
// kernel thus land in memory this library owns and are detected instead of corrupting a
// neighbour silently.
namespace {
constexpr size_t kGuardBytes = 256;
constexpr unsigned char kGuardPattern = 0xA5;
bool guard_enabled() {
  static const bool on = getenv("MDC_POOL_GUARD") && atoi(getenv("MDC_POOL_GUARD")) != 0;
  return on;
}
std::unordered_map<const void *, uint64_t> g_guarded;  // user pointer -> user size
}  // namespace

MDC_API void *mgpuMemAlloc(uint64_t sizeBytes, mgpu_stream_t stream) {
  if (!ensure_device()) return nullptr;
  cudaError_t e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (guard_enabled()) {
    const uint64_t user = (sizeBytes + 15) & ~uint64_t(15);
    char *raw = static_cast<char *>(pool().alloc(user + 2 * kGuardBytes, s, &e));
    rt_ok(e, "mgpuMemAlloc");
    if (!raw) return nullptr;
    RT_CHECK(cudaMemsetAsync(raw, kGuardPattern, kGuardBytes, s));
    RT_CHECK(cudaMemsetAsync(raw + kGuardBytes + user, kGuardPattern, kGuardBytes, s));
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    g_guarded[raw + kGuardBytes] = user;
    return raw + kGuardBytes;
  }
  void *p = pool().alloc(sizeBytes, s, &e);
  rt_ok(e, "mgpuMemAlloc");
  return p;
}
MDC_API void mgpuMemFree(void *ptr, mgpu_stream_t stream) {
  if (!ptr) return;
  {
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    if (!g_copies_of_constants.empty()) g_copies_of_constants.erase(ptr);
  }
  cudaError_t e;
  if (guard_enabled()) {
    uint64_t user = 0;
    bool known = false;
    {
      std::lock_guard<std::recursive_mutex> lock(g_state_mu);
      auto it = g_guarded.find(ptr);
      if (it != g_guarded.end()) {
        user = it->second;
        known = true;
        g_guarded.erase(it);
      }
    }
    if (known) {
      cudaStream_t s = static_cast<cudaStream_t>(stream);
      char *raw = static_cast<char *>(ptr) - kGuardBytes;
      unsigned char bands[2 * kGuardBytes];
      if (RT_CHECK(cudaMemcpyAsync(bands, raw, kGuardBytes, cudaMemcpyDeviceToHost, s)) &&
          RT_CHECK(cudaMemcpyAsync(bands + kGuardBytes, raw + kGuardBytes + user, kGuardBytes, cudaMemcpyDeviceToHost, s)) &&
          RT_CHECK(cudaStreamSynchronize(s))) {
        for (size_t i = 0; i < 2 * kGuardBytes; ++i)
          if (bands[i] != kGuardPattern) {
            char msg[160];
            snprintf(msg, sizeof(msg), "guard band %s block %p (%llu bytes) was overwritten at offset %zu",
                     i < kGuardBytes ? "before" : "after", ptr, (unsigned long long)user, i % kGuardBytes);
            record_error(-1, "mgpuMemFree", msg);
            break;
          }
      }
      pool().free(raw, s, &e);
      rt_ok(e, "mgpuMemFree");
      return;
    }
  }
  if (!pool().free(ptr, static_cast<cudaStream_t>(stream), &e)) {
    // not from the pool (e.g. a tensor map made by mgpuTensorMapEncodeTiledMemref)
    RT_CHECK(cudaFree(ptr));
    return;
  }
  rt_ok(e, "mgpuMemFree");
}
MDC_API void *mgpuMemAllocAsync(uint64_t sizeBytes, mgpu_stream_t stream) {
  return mgpuMemAlloc(sizeBytes, stream);
}
MDC_API void mgpuMemFreeAsync(void *ptr, mgpu_stream_t stream) { mgpuMemFree(ptr, stream); }

MDC_API void mgpuMemcpy(void *dst, void *src, size_t sizeBytes, mgpu_stream_t stream) {
  if (!ensure_device()) return;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // a registered host constant (model weights): served from its device-resident copy
  std::unique_lock<std::recursive_mutex> state_lock(g_state_mu);
  if (!g_constants.empty()) {
    auto it = g_constants.find(src);
    if (it != g_constants.end() && sizeBytes <= it->second.bytes && it->second.device == g_default_device) {
      Constant &c = it->second;
      if (!c.dev) {
        cudaError_t e;
        c.dev = pool().alloc(c.bytes, s, &e);
        if (c.dev && RT_CHECK(cudaMemcpyAsync(c.dev, src, c.bytes, cudaMemcpyHostToDevice, s)))
          RT_CHECK(cudaEventRecord(c.uploaded, s));
      } else {
        RT_CHECK(cudaStreamWaitEvent(s, c.uploaded, 0));
      }
      if (c.dev) {
        RT_CHECK(cudaMemcpyAsync(dst, c.dev, sizeBytes, cudaMemcpyDeviceToDevice, s));
        // remembered so that the copy can be waited for before the block is given back
        if (c.last_use) RT_CHECK(cudaEventRecord(c.last_use, s));
        if (sizeBytes == c.bytes) g_copies_of_constants[dst] = src;
        else g_copies_of_constants.erase(dst);
        return;
      }
    }
  }
  if (!g_copies_of_constants.empty()) g_copies_of_constants.erase(dst);
  state_lock.unlock();
  if (staged_copy(dst, src, sizeBytes, s)) return;
  RT_CHECK(cudaMemcpyAsync(dst, src, sizeBytes, cudaMemcpyDefault, s));
}

MDC_API void mgpuRegisterConstant(void *hostPtr, uint64_t sizeBytes) {
  if (!hostPtr || !sizeBytes || !ensure_device()) return;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  mgpuUnregisterConstant(hostPtr);
  Constant c;
  c.bytes = sizeBytes;
  c.device = g_default_device;
  if (!RT_CHECK(cudaEventCreateWithFlags(&c.uploaded, cudaEventDisableTiming)) ||
      !RT_CHECK(cudaEventCreateWithFlags(&c.last_use, cudaEventDisableTiming)))
    return;
  g_constants[hostPtr] = c;
}

MDC_API void mgpuUnregisterConstant(void *hostPtr) {
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  auto it = g_constants.find(hostPtr);
  if (it == g_constants.end()) return;
  Constant &c = it->second;
  if (c.dev) {
    // the device copy may still be the source of copies queued on any stream: wait for the
    // upload and for the last copy served from it, then give the block back to the pool of
    // the device it came from
    int cur = -1;
    const bool switched = cudaGetDevice(&cur) == cudaSuccess && cur != c.device && cudaSetDevice(c.device) == cudaSuccess;
    if (c.uploaded) cudaEventSynchronize(c.uploaded);
    if (c.last_use) cudaEventSynchronize(c.last_use);
    cudaError_t e;
    const int d = (c.device >= 0 && c.device < kMaxDevices) ? c.device : 0;
    g_pools[d].free(c.dev, nullptr, &e);
    if (switched) cudaSetDevice(cur);
    (void)cudaGetLastError();
  }
  for (auto &kv : c.derived) {
    Constant::Derived &dv = kv.second;
    if (dv.ready) {
      cudaEventSynchronize(dv.ready);
      cudaEventDestroy(dv.ready);
    }
    if (dv.dev) {
      // its users were queued on streams this library cannot enumerate: drain the device
      cudaDeviceSynchronize();
      cudaError_t e;
      const int d = (c.device >= 0 && c.device < kMaxDevices) ? c.device : 0;
      g_pools[d].free(dv.dev, nullptr, &e);
    }
  }
  for (auto t = g_copies_of_constants.begin(); t != g_copies_of_constants.end();)
    t = (t->second == hostPtr) ? g_copies_of_constants.erase(t) : std::next(t);
  if (c.uploaded) cudaEventDestroy(c.uploaded);
  if (c.last_use) cudaEventDestroy(c.last_use);
  g_constants.erase(it);
}
MDC_API const void *mgpuConstantSourceOf(const void *devPtr) {
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  if (g_copies_of_constants.empty()) return nullptr;
  auto it = g_copies_of_constants.find(devPtr);
  return it == g_copies_of_constants.end() ? nullptr : it->second;
}

MDC_API void *mgpuConstantDerived(const void *hostKey, uint64_t tag, uint64_t bytes, mgpu_stream_t stream,
                                  int32_t *needsFill) {
  if (needsFill) *needsFill = 0;
  if (!hostKey || !bytes || !ensure_device()) return nullptr;
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  auto it = g_constants.find(hostKey);
  if (it == g_constants.end() || it->second.device != g_default_device) return nullptr;
  Constant::Derived &dv = it->second.derived[tag];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dv.dev && dv.bytes != bytes) return nullptr;  // a tag names one size
  if (!dv.dev) {
    cudaError_t e;
    dv.dev = pool().alloc(bytes, s, &e);
    if (!dv.dev) {
      rt_ok(e, "mgpuConstantDerived");
      it->second.derived.erase(tag);
      return nullptr;
    }
    dv.bytes = bytes;
    if (!RT_CHECK(cudaEventCreateWithFlags(&dv.ready, cudaEventDisableTiming))) dv.ready = nullptr;
  }
  if (!dv.filled) {
    if (needsFill) *needsFill = 1;
  } else if (dv.ready) {
    RT_CHECK(cudaStreamWaitEvent(s, dv.ready, 0));
  }
  return dv.dev;
}

MDC_API void mgpuConstantDerivedReady(const void *hostKey, uint64_t tag, mgpu_stream_t stream) {
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  auto it = g_constants.find(hostKey);
  if (it == g_constants.end()) return;
  auto dv = it->second.derived.find(tag);
  if (dv == it->second.derived.end() || !dv->second.dev) return;
  if (dv->second.ready) RT_CHECK(cudaEventRecord(dv->second.ready, static_cast<cudaStream_t>(stream)));
  dv->second.filled = true;
}

MDC_API void mgpuMemset32(void *dst, unsigned int value, size_t count, mgpu_stream_t stream) {
  if (!ensure_device() || !driver().ok) return;
  {
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    if (!g_copies_of_constants.empty()) g_copies_of_constants.erase(dst);
  }
  DRV_CHECK(driver().MemsetD32Async(reinterpret_cast<CUdeviceptr>(dst), value, count,
                                    reinterpret_cast<CUstream>(stream)));
}
MDC_API void mgpuMemset16(void *dst, unsigned short value, size_t count, mgpu_stream_t stream) {
  if (!ensure_device() || !driver().ok) return;
  {
    std::lock_guard<std::recursive_mutex> lock(g_state_mu);
    if (!g_copies_of_constants.empty()) g_copies_of_constants.erase(dst);
  }
  DRV_CHECK(driver().MemsetD16Async(reinterpret_cast<CUdeviceptr>(dst), value, count,
                                    reinterpret_cast<CUstream>(stream)));
}

MDC_API void mgpuMemHostRegister(void *ptr, uint64_t sizeBytes) {
  if (!ensure_device()) return;
  RT_CHECK(cudaHostRegister(ptr, sizeBytes, cudaHostRegisterDefault));
}
MDC_API void mgpuMemHostUnregister(void *ptr) { RT_CHECK(cudaHostUnregister(ptr)); }

MDC_API void mgpuMemHostRegisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes) {
  auto *d = static_cast<MemRefDesc *>(descriptor);
  const int64_t *sizes = d->sizes_and_strides;
  const int64_t *strides = sizes + rank;
  int64_t running = 1;
  for (int64_t i = rank - 1; i >= 0; --i) {  // only densely packed tensors are supported
    if (strides[i] != running) {
      record_error(-1, "mgpuMemHostRegisterMemRef", "memref is not densely packed");
      return;
    }
    running *= sizes[i];
  }
  mgpuMemHostRegister(d->data + d->offset * elementSizeBytes,
                      static_cast<uint64_t>(running * elementSizeBytes));
}
MDC_API void mgpuMemHostUnregisterMemRef(int64_t /*rank*/, void *descriptor,
                                         int64_t elementSizeBytes) {
  auto *d = static_cast<MemRefDesc *>(descriptor);
  mgpuMemHostUnregister(d->data + d->offset * elementSizeBytes);
}

MDC_API void mgpuSetDefaultDevice(int32_t device) {
  if (device != g_default_device) g_device_bound = false;
  g_default_device = device;
  g_device_chosen = true;
}

MDC_API int32_t mgpuGetDefaultDevice(void) { return ensure_device() ? g_default_device : -1; }

MDC_API void mgpuMemGetInfo(uint64_t *freeBytes, uint64_t *totalBytes) {
  size_t f = 0, t = 0;
  if (ensure_device()) RT_CHECK(cudaMemGetInfo(&f, &t));
  if (freeBytes) *freeBytes = f;
  if (totalBytes) *totalBytes = t;
}

MDC_API uint64_t mgpuPoolReservedBytes(void) { return pool().reserved_bytes(); }
MDC_API uint64_t mgpuPoolInUseBytes(void) { return pool().in_use_bytes(); }
MDC_API void mgpuPoolTrim(void) { pool().trim(); }

// ---------------- tensor maps ----------------
MDC_API void mgpuTensorMapEncodeTiled(void *tensorMap, int tensorDataType, uint32_t tensorRank,
                                      void *globalAddress, const uint64_t *globalDim,
                                      const uint64_t *globalStrides, const uint32_t *boxDim,
                                      const uint32_t *elementStrides, int interleave, int swizzle,
                                      int l2Promotion, int oobFill) {
  if (!ensure_device() || !driver().ok) return;
  DRV_CHECK(driver().TensorMapEncodeTiled(
      static_cast<CUtensorMap *>(tensorMap), static_cast<CUtensorMapDataType>(tensorDataType),
      tensorRank, globalAddress, reinterpret_cast<const cuuint64_t *>(globalDim),
      reinterpret_cast<const cuuint64_t *>(globalStrides), boxDim, elementStrides,
      static_cast<CUtensorMapInterleave>(interleave), static_cast<CUtensorMapSwizzle>(swizzle),
      static_cast<CUtensorMapL2promotion>(l2Promotion),
      static_cast<CUtensorMapFloatOOBfill>(oobFill)));
}

MDC_API void *mgpuTensorMapEncodeTiledMemref(int64_t tensorRank, void *descriptor,
                                             int tensorDataType, int interleave, int swizzle,
                                             int l2Promotion, int oobFill, int64_t *inputBoxDims) {
  if (tensorRank < 1 || tensorRank > 5) {
    record_error(-1, "mgpuTensorMapEncodeTiledMemref", "rank must be 1..5");
    return nullptr;
  }
  auto *d = static_cast<MemRefDesc *>(descriptor);
  const int64_t *sizes = d->sizes_and_strides;
  // element sizes of CUtensorMapDataType 0..12
  static const int elem_bytes[] = {1, 2, 4, 4, 8, 8, 2, 4, 8, 2, 4, 4, 4};
  if (tensorDataType < 0 || tensorDataType > 12) {
    record_error(-1, "mgpuTensorMapEncodeTiledMemref", "unknown element type");
    return nullptr;
  }
  uint32_t box[5] = {1, 1, 1, 1, 1}, estr[5] = {1, 1, 1, 1, 1};
  uint64_t gdim[5] = {1, 1, 1, 1, 1}, gstr[5] = {0, 0, 0, 0, 0};
  for (int64_t r = 0; r < tensorRank; ++r) {  // innermost dimension first
    box[r] = static_cast<uint32_t>(inputBoxDims[tensorRank - r - 1]);
    gdim[r] = static_cast<uint64_t>(sizes[tensorRank - r - 1]);
  }
  // byte strides of dimensions 1..rank-1 of a densely packed tensor
  uint64_t running = gdim[0] * elem_bytes[tensorDataType];
  for (int64_t r = 0; r + 1 < tensorRank; ++r) {
    gstr[r] = running;
    running *= gdim[r + 1];
  }
  CUtensorMap map;
  mgpuTensorMapEncodeTiled(&map, tensorDataType, static_cast<uint32_t>(tensorRank), d->data, gdim,
                           gstr, box, estr, interleave, swizzle, l2Promotion, oobFill);
  void *dmap = nullptr;
  if (!RT_CHECK(cudaMalloc(&dmap, sizeof(CUtensorMap)))) return nullptr;
  RT_CHECK(cudaMemcpy(dmap, &map, sizeof(CUtensorMap), cudaMemcpyHostToDevice));
  return dmap;
}

namespace {
int builtin_operands(const std::string &b) {
  if (b == "mdc_add_f32") return 3;
  if (b == "mdc_relu_f32" || b == "mdc_gelu_erf_f32" || b == "mdc_gelu_tanh_f32") return 2;
  return 0;
}
void register_override(const char *pattern, const std::string &b, int rank, int operands, int64_t elements) {
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  for (KernelOverride *o : g_overrides)
    if (o->pattern == pattern) {  // redefinition
      o->builtin = b, o->rank = rank, o->operands = operands, o->elements = elements, o->target = nullptr;
      return;
    }
  KernelOverride *o = new KernelOverride;
  o->pattern = pattern, o->builtin = b, o->rank = rank, o->operands = operands, o->elements = elements;
  g_overrides.push_back(o);
  g_override_handles.insert(o);
}
}  // namespace

MDC_API void mgpuModuleOverrideKernel(const char *pattern, const char *builtin, int32_t rank) {
  if (!pattern || !builtin || rank < 1 || rank > 8) {
    record_error(-1, "mgpuModuleOverrideKernel", "needs a pattern, a built-in kernel name and a rank of 1-8");
    return;
  }
  const std::string b = builtin;
  const int operands = builtin_operands(b);
  if (!operands) {
    record_error(-1, "mgpuModuleOverrideKernel", "the built-in must be mdc_add_f32, mdc_relu_f32, mdc_gelu_erf_f32 or mdc_gelu_tanh_f32");
    return;
  }
  register_override(pattern, b, rank, operands, 0);
}

MDC_API void mgpuModuleOverrideKernelBare(const char *pattern, const char *builtin, int64_t elements) {
  if (!pattern || !builtin || elements < 0) {
    record_error(-1, "mgpuModuleOverrideKernelBare", "needs a pattern, a built-in kernel name and an element count >= 0");
    return;
  }
  const int operands = builtin_operands(builtin);
  if (!operands) {
    record_error(-1, "mgpuModuleOverrideKernelBare", "the built-in must be mdc_add_f32, mdc_relu_f32, mdc_gelu_erf_f32 or mdc_gelu_tanh_f32");
    return;
  }
  register_override(pattern, builtin, 0, operands, elements);
}

MDC_API void mgpuModuleClearOverrides(void) {
  // handles already given out stay valid objects; they only stop being matched
  std::lock_guard<std::recursive_mutex> lock(g_state_mu);
  for (KernelOverride *o : g_overrides) o->pattern.clear();
}
