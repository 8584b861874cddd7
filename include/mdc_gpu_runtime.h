/*
 * C ABI of libMultiDeviceCUDARuntime.so: the stream / event / memory / module / launch
 * wrappers that graphs lowered by Multi-device-model-compiler's Device dialect call.
 *
 * Every entry point keeps the name, argument order and argument meaning of the reference
 * symbol cited beside it (paths are relative to the reference project), so a lowered
 * model .so resolves against this library unchanged.  CUstream / CUevent / CUfunction are
 * the CUDA driver's handle types; they are spelled as opaque pointers here so the header
 * needs no CUDA include.
 *
 * Differences from the reference that a caller can observe:
 *  - mgpuMemAlloc / mgpuMemFree are served by a caching, stream-ordered device pool
 *    instead of a synchronous cuMemAlloc / cuMemFree per call.
 *  - mgpuMemcpy between pageable host memory and the device, 1 MiB and larger, is cut into
 *    4 MiB chunks that a small team of host threads moves through a ring of pinned buffers
 *    while the copy engine transfers the previous chunk (MDC_COPY_THREADS sets the team
 *    size, MDC_STAGED_COPY=0 restores the plain cuMemcpyAsync).  Completion semantics are
 *    those of a pageable copy: an upload returns once the source has been read, a download
 *    is complete on return.
 *  - mgpuModuleGetFunction first looks the name up in a registry of built-in hand-written
 *    kernels (mdc_add_f32, ...) and only then in the module loaded from a file.
 *  - Errors never abort or throw: they are printed to stderr like the reference does and
 *    are also kept as a sticky status readable with mgpuGetLastError().
 * Threading contract (as in the reference): one host thread per process drives the
 * library; all work is ordered on the streams the caller passes.
 */
#ifndef MDC_GPU_RUNTIME_H_
#define MDC_GPU_RUNTIME_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mgpu_stream_t;   /* CUstream  */
typedef void *mgpu_event_t;    /* CUevent   */
typedef void *mgpu_function_t; /* CUfunction */

/* include/multi-device-model-compiler/Runtime/CUDA/CudaRuntimeWrappers.h:26-28,
 * lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:91-107.  The file may be a cubin, a fatbin or
 * a PTX text file; a missing file is reported but leaves the built-in kernels usable. */
void mgpuModuleFileLoad(const char *fname);
void mgpuModuleUnload(void);
mgpu_function_t mgpuModuleGetFunction(const char *name);

/* CudaRuntimeWrappers.h:29-33, .cpp:112-139.  params is the array of pointers to the
 * kernel arguments (cuLaunchKernel convention). */
void mgpuLaunchKernel(mgpu_function_t function, intptr_t gridX, intptr_t gridY, intptr_t gridZ,
                      intptr_t blockX, intptr_t blockY, intptr_t blockZ, int32_t smem,
                      mgpu_stream_t stream, void **params, void **extra);

/* CudaRuntimeWrappers.h:34-36, .cpp:141-160 (mgpuStreamSynchronize: .cpp:152-155). */
mgpu_stream_t mgpuStreamCreate(void);
void mgpuStreamDestroy(mgpu_stream_t stream);
void mgpuStreamSynchronize(mgpu_stream_t stream);
void mgpuStreamWaitEvent(mgpu_stream_t stream, mgpu_event_t event);

/* CudaRuntimeWrappers.h:37-44, .cpp:162-202. */
mgpu_event_t mgpuEventCreate(void);
mgpu_event_t mgpuEventEnableTimeCreate(void);
mgpu_event_t mgpuEventCreateWithStream(mgpu_stream_t stream);
void mgpuEventDestroy(mgpu_event_t event);
void mgpuEventSynchronize(mgpu_event_t event);
void mgpuEventRecord(mgpu_event_t event, mgpu_stream_t stream);
float mgpuEventElapsedTime(mgpu_event_t begin, mgpu_event_t end); /* milliseconds */

/* CudaRuntimeWrappers.h:45-52, .cpp:204-243.  Alloc/Free and AllocAsync/FreeAsync share
 * one pool; a block freed on a stream is reused on another stream only after an event
 * wait, so the stream ordering a lowered graph sets up stays valid. */
void *mgpuMemAlloc(uint64_t sizeBytes, mgpu_stream_t stream);
void mgpuMemFree(void *ptr, mgpu_stream_t stream);
void *mgpuMemAllocAsync(uint64_t sizeBytes, mgpu_stream_t stream);
void mgpuMemFreeAsync(void *ptr, mgpu_stream_t stream);
void mgpuMemcpy(void *dst, void *src, size_t sizeBytes, mgpu_stream_t stream);
void mgpuMemset32(void *dst, unsigned int value, size_t count, mgpu_stream_t stream);
void mgpuMemset16(void *dst, unsigned short value, size_t count, mgpu_stream_t stream);

/* lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:251-295.  The MemRef forms take an MLIR
 * strided memref descriptor {data, aligned, offset, sizes[rank], strides[rank]} of char. */
void mgpuMemHostRegister(void *ptr, uint64_t sizeBytes);
void mgpuMemHostRegisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes);
void mgpuMemHostUnregister(void *ptr);
void mgpuMemHostUnregisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes);

/* lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:297-299: device ordinal used by this thread.
 * This is THE way to choose a GPU: every later runtime and op call of the thread works on that
 * device (pool, streams, tensor maps, kernels).  A thread that never calls it adopts, at its
 * first runtime call, the device that is current on it (the one cudaSetDevice chose, else
 * ordinal 0).  Op entry points refuse to run (status set, nothing queued) while the thread's
 * current CUDA device differs from the selected one, e.g. after a later cudaSetDevice.
 * mgpuGetDefaultDevice (an addition) returns the selected ordinal, or -1 without a device. */
void mgpuSetDefaultDevice(int32_t device);
int32_t mgpuGetDefaultDevice(void);

/* lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:303-384.  tensorMap points at a 128-byte
 * CUtensorMap; the enum arguments are the driver's CUtensorMap* enums passed as ints. */
void mgpuTensorMapEncodeTiled(void *tensorMap, int tensorDataType, uint32_t tensorRank,
                              void *globalAddress, const uint64_t *globalDim,
                              const uint64_t *globalStrides, const uint32_t *boxDim,
                              const uint32_t *elementStrides, int interleave, int swizzle,
                              int l2Promotion, int oobFill);
void *mgpuTensorMapEncodeTiledMemref(int64_t tensorRank, void *descriptor, int tensorDataType,
                                     int interleave, int swizzle, int l2Promotion, int oobFill,
                                     int64_t *inputBoxDims);

/* ---- additions (no counterpart in the reference) ---- */

/* Sticky status: 0 when no wrapper has failed since the last clear, otherwise the CUDA
 * error code of the first failure.  The reference only prints (CudaRuntimeWrappers.cpp:3-12). */
int32_t mgpuGetLastError(void);
const char *mgpuGetLastErrorString(void);
void mgpuClearLastError(void);
/* Lets the op library report its own failures through the same status. */
void mgpuSetLastError(int32_t code, const char *what);

/* Constant-weight cache.  A lowered graph re-uploads its weights with mgpuMemcpy on every
 * call (lib/Dialect/Device/Transform/DeviceDataCopyGeneration.cpp:26-70).  After
 * mgpuRegisterConstant(p, n) the caller promises not to change host bytes [p, p+n); the first
 * mgpuMemcpy whose source is exactly p uploads them once into a device-resident copy and this
 * and every later such copy is served device-to-device.  Unregister before freeing or
 * changing the buffer. */
void mgpuRegisterConstant(void *hostPtr, uint64_t sizeBytes);
void mgpuUnregisterConstant(void *hostPtr);
/* What the op library builds on the constant cache (lowered graphs do not call these).
 * mgpuConstantSourceOf(p): when the device block starting at p was last filled, whole, by an
 * mgpuMemcpy from a registered constant (and has not since been freed or been the target of
 * another mgpuMemcpy / mgpuMemset), the constant's host pointer; else NULL.  A kernel that
 * writes into such a block is not seen: graphs do not modify their weight buffers.
 * mgpuConstantDerived(key, tag, bytes, stream, &needsFill): a device buffer of `bytes` that
 * lives as long as the registration of `key` (one per tag; e.g. the packed 16-bit form of a
 * weight).  needsFill = 1: the caller must write it on `stream` and then call
 * mgpuConstantDerivedReady(key, tag, stream); needsFill = 0: it is filled, and `stream` has
 * been made to wait for that.  NULL when `key` is not a registered constant of this device. */
const void *mgpuConstantSourceOf(const void *devPtr);
void *mgpuConstantDerived(const void *hostKey, uint64_t tag, uint64_t bytes, mgpu_stream_t stream,
                          int32_t *needsFill);
void mgpuConstantDerivedReady(const void *hostKey, uint64_t tag, mgpu_stream_t stream);

/* Kernel overrides.  The reference generates a scalar one-element-per-thread kernel for every
 * elementwise graph (lib/Dialect/Device/IR/GPUOffloadingAttr.cpp:255-313) and the lowered graph
 * fetches it by name.  After mgpuModuleOverrideKernel(pattern, builtin, rank),
 * mgpuModuleGetFunction of a matching name (exact, or a prefix ending in '*') returns a handle
 * that mgpuLaunchKernel routes to the built-in kernel (mdc_add_f32: three operands;
 * mdc_relu_f32 / mdc_gelu_erf_f32 / mdc_gelu_tanh_f32: two).  The caller keeps passing the
 * generated kernel's arguments - per operand the expanded memref (allocated, aligned, offset,
 * sizes[rank], strides[rank]) - and its own grid, which is ignored.  Operands must be
 * contiguous and of one size, otherwise the launch is refused with a status. */
void mgpuModuleOverrideKernel(const char *pattern, const char *builtin, int32_t rank);
/* The same for kernels in the argument form the reference's GPU pipeline really emits: it lowers
 * generated kernels and their launches with bare pointers (lib/Pipelines/MLIRToGPU.cpp:162-165
 * useBarePtrCallConv, :180-183 kernelBarePtrCallConv; the argument array is built from the launch
 * operands at lib/Dialect/Device/IR/GPUOffloadingAttr.cpp:222-247), so the kernel receives one
 * pointer per operand and nothing else; shapes are static and known only to the generated code.
 * `elements` is the element count of every operand; 0 means "the launch's grid x block", for
 * graphs whose one-thread-per-element launch covers the tensor exactly. */
void mgpuModuleOverrideKernelBare(const char *pattern, const char *builtin, int64_t elements);
void mgpuModuleClearOverrides(void);

/* Pool introspection / control: bytes held from the driver, bytes handed out, and a call
 * that returns every cached block to the driver. */
uint64_t mgpuPoolReservedBytes(void);
uint64_t mgpuPoolInUseBytes(void);
void mgpuPoolTrim(void);
/* Free and total device memory of the selected device as the driver reports them
 * (cudaMemGetInfo); sees every allocation of the process, the pool's included. */
void mgpuMemGetInfo(uint64_t *freeBytes, uint64_t *totalBytes);

/* Grid / block a caller should pass to mgpuLaunchKernel for a built-in elementwise kernel
 * over n elements (the kernels are grid-stride, so any launch shape is still correct). */
void mgpuBuiltinLaunchShape(int64_t n, intptr_t *gridX, intptr_t *blockX);

#ifdef __cplusplus
}
#endif
#endif /* MDC_GPU_RUNTIME_H_ */
