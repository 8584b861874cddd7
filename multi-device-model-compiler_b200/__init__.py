"""ctypes binding of the two C-ABI libraries (libMultiDeviceCUDARuntime.so,
libMultiDeviceGPUOps.so) plus small numpy conveniences used by the tests, the benchmark
and the smoke run.

There is no CPU implementation behind these calls: if the libraries are not built, or no
CUDA device is present, the compute entry points raise `MdcError`.  Device memory, streams
and copies all go through the library's own mgpu* runtime (no torch tensors involved).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "lib")
BIN_DIR = os.path.join(_HERE, "bin")
RUNTIME_LIB = os.path.join(LIB_DIR, "libMultiDeviceCUDARuntime.so")
OPS_LIB = os.path.join(LIB_DIR, "libMultiDeviceGPUOps.so")

F32, F16, BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH = 0, 1, 2, 3


class MdcError(RuntimeError):
    pass


def build(verbose: bool = False, ptxas_v: bool = False) -> None:
    """Compile every library / tool for sm_100a with the Makefile beside this file."""
    cmd = ["make", "-C", _HERE, "-j", str(min(8, os.cpu_count() or 1))]
    if ptxas_v:
        cmd.append("PTXAS_V=1")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout[-4000:])
        print(res.stderr[-4000:])
    if res.returncode != 0:
        raise MdcError("building the CUDA libraries failed")


_vp, _i64, _i32, _u32, _u64, _f = C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_uint64, C.c_float
_b = C.c_bool

# name -> (restype, argtypes); the single source the symbol-export test checks against
RUNTIME_SIGNATURES = {
    "mgpuModuleFileLoad": (None, [C.c_char_p]),
    "mgpuModuleUnload": (None, []),
    "mgpuModuleGetFunction": (_vp, [C.c_char_p]),
    "mgpuLaunchKernel": (None, [_vp] + [C.c_ssize_t] * 6 + [_i32, _vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "mgpuStreamCreate": (_vp, []),
    "mgpuStreamDestroy": (None, [_vp]),
    "mgpuStreamSynchronize": (None, [_vp]),
    "mgpuStreamWaitEvent": (None, [_vp, _vp]),
    "mgpuEventCreate": (_vp, []),
    "mgpuEventEnableTimeCreate": (_vp, []),
    "mgpuEventCreateWithStream": (_vp, [_vp]),
    "mgpuEventDestroy": (None, [_vp]),
    "mgpuEventSynchronize": (None, [_vp]),
    "mgpuEventRecord": (None, [_vp, _vp]),
    "mgpuEventElapsedTime": (_f, [_vp, _vp]),
    "mgpuMemAlloc": (_vp, [_u64, _vp]),
    "mgpuMemFree": (None, [_vp, _vp]),
    "mgpuMemAllocAsync": (_vp, [_u64, _vp]),
    "mgpuMemFreeAsync": (None, [_vp, _vp]),
    "mgpuMemcpy": (None, [_vp, _vp, C.c_size_t, _vp]),
    "mgpuMemset32": (None, [_vp, C.c_uint, C.c_size_t, _vp]),
    "mgpuMemset16": (None, [_vp, C.c_ushort, C.c_size_t, _vp]),
    "mgpuMemHostRegister": (None, [_vp, _u64]),
    "mgpuMemHostRegisterMemRef": (None, [_i64, _vp, _i64]),
    "mgpuMemHostUnregister": (None, [_vp]),
    "mgpuMemHostUnregisterMemRef": (None, [_i64, _vp, _i64]),
    "mgpuSetDefaultDevice": (None, [_i32]),
    "mgpuTensorMapEncodeTiled": (None, [_vp, C.c_int, _u32, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int]),
    "mgpuTensorMapEncodeTiledMemref": (_vp, [_i64, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "mgpuModuleOverrideKernel": (None, [C.c_char_p, C.c_char_p, _i32]),
    "mgpuModuleOverrideKernelBare": (None, [C.c_char_p, C.c_char_p, _i64]),
    "mgpuModuleClearOverrides": (None, []),
    "mgpuGetDefaultDevice": (_i32, []),
    "mgpuMemGetInfo": (None, [C.POINTER(_u64), C.POINTER(_u64)]),
    "mgpuGetLastError": (_i32, []),
    "mgpuGetLastErrorString": (C.c_char_p, []),
    "mgpuClearLastError": (None, []),
    "mgpuSetLastError": (None, [_i32, C.c_char_p]),
    "mgpuRegisterConstant": (None, [_vp, _u64]),
    "mgpuUnregisterConstant": (None, [_vp]),
    "mgpuConstantSourceOf": (_vp, [_vp]),
    "mgpuConstantDerived": (_vp, [_vp, _u64, _u64, _vp, C.POINTER(_i32)]),
    "mgpuConstantDerivedReady": (None, [_vp, _u64, _vp]),
    "mgpuPoolReservedBytes": (_u64, []),
    "mgpuPoolInUseBytes": (_u64, []),
    "mgpuPoolTrim": (None, []),
    "mgpuBuiltinLaunchShape": (None, [_i64, C.POINTER(C.c_ssize_t), C.POINTER(C.c_ssize_t)]),
}

OPS_SIGNATURES = {
    "mgpuMatmul": (None, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mgpuMatmulNoAlloc": (None, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "mgpuConv2d": (None, [_vp] * 5 + [_i64] * 17 + [_b, _b, _vp]),
    "mgpuPool2d": (None, [_vp, _vp] + [_i64] * 15 + [_vp]),
    "mgpuLLMDecodingContextLayer": (None, [_vp] * 9 + [_i64] * 5 + [_b, _b, _b, _vp]),
    "mgpuOpsInit": (_i32, []),
    "mgpuOpsDeinit": (None, []),
    "mgpuAdd": (None, [_vp, _vp, _vp, _i64, _vp]),
    "mgpuBiasAdd": (None, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "mgpuActivation": (None, [_vp, _vp, _i64, _i32, _vp]),
    "mgpuCast": (None, [_vp, _i32, _vp, _i32, _i64, _vp]),
    "mgpuLayerNormF32": (None, [_vp, _vp, _vp, _vp, _f, _i64, _i64, _vp]),
    "mgpuLayerNormEx": (None, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i64, _i64, _i32, _i32, _vp]),
    "mgpuPackWeight": (None, [_vp, _vp, _i64, _i64, _i32, _vp]),
    "mgpuMatmulEx16": (None, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "mgpuAttention": (None, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _b, _i32, _vp]),
    "mgpuEncoderStackCreate": (_vp, [_i64, _i64, _i64, _i64, _b, _b, _i32, _i32, _f]),
    "mgpuEncoderStackSetLayer": (None, [_vp, _i64] + [_vp] * 12 + [_vp]),
    "mgpuEncoderStackRun": (None, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "mgpuEncoderStackDestroy": (None, [_vp]),
    "mgpuEncoderStackRunHost": (None, [_vp, _vp, _vp, _vp, _i64, _i64, _i32]),
    "mgpuEncoderStackSubmitHost": (_i64, [_vp, _vp, _vp, _vp, _i64, _i64]),
    "mgpuEncoderStackWaitHost": (None, [_vp, _i64]),
    "mgpuTransformerEncoderLayer": (None, [_vp] * 15 + [_i64] * 5 + [_b, _b, _i32, _i32, _f, _vp]),
    "mgpuOpsLaunchCount": (_u64, []),
    "mgpuOpsCheckDeviceStatus": (_u32, [_vp]),
    "mgpuOpsProfileBegin": (None, []),
    "mgpuOpsProfileEnd": (None, [C.POINTER(C.c_double), C.POINTER(_u64)]),
    "mgpuOpsProfileEndSpans": (_i64, [C.POINTER(_i32), C.POINTER(_f), _i64]),
}

_rt = None
_ops = None


def _bind(lib, table):
    for name, (res, args) in table.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def runtime():
    """The runtime library (loads without a GPU; calls then fail with a status)."""
    global _rt
    if _rt is None:
        if not os.path.exists(RUNTIME_LIB):
            raise MdcError(f"{RUNTIME_LIB} is missing: run build() (make -C {_HERE})")
        _rt = C.CDLL(RUNTIME_LIB, mode=C.RTLD_GLOBAL)
        _bind(_rt, RUNTIME_SIGNATURES)
    return _rt


def ops():
    global _ops
    if _ops is None:
        runtime()
        if not os.path.exists(OPS_LIB):
            raise MdcError(f"{OPS_LIB} is missing: run build() (make -C {_HERE})")
        _ops = C.CDLL(OPS_LIB, mode=C.RTLD_GLOBAL)
        _bind(_ops, OPS_SIGNATURES)
    return _ops


def check(where: str = "") -> None:
    """Raise if any library call has failed since the last clear."""
    rt = runtime()
    code = rt.mgpuGetLastError()
    if code != 0:
        msg = rt.mgpuGetLastErrorString().decode(errors="replace")
        rt.mgpuClearLastError()
        raise MdcError(f"{where}: error {code}: {msg}")


def init(device: int = 0) -> None:
    rt = runtime()
    rt.mgpuSetDefaultDevice(device)
    if ops().mgpuOpsInit() != 0:
        check("mgpuOpsInit")
        raise MdcError("mgpuOpsInit failed (no sm_100 CUDA device?)")
    check("init")


# ---------------------------------------------------------------- numpy helpers
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


class DeviceBuffer:
    """A block from the runtime's device pool; freed when released or collected."""

    def __init__(self, nbytes: int, stream=None):
        self.nbytes = int(nbytes)
        self.ptr = runtime().mgpuMemAlloc(max(self.nbytes, 1), stream)
        if not self.ptr:
            check("mgpuMemAlloc")
            raise MdcError("mgpuMemAlloc returned NULL")

    def release(self, stream=None):
        if self.ptr:
            runtime().mgpuMemFree(self.ptr, stream)
            self.ptr = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def to_device(arr: np.ndarray, stream=None) -> DeviceBuffer:
    arr = np.ascontiguousarray(arr)
    buf = DeviceBuffer(arr.nbytes, stream)
    if arr.nbytes:
        runtime().mgpuMemcpy(buf.ptr, arr.ctypes.data, arr.nbytes, stream)
        runtime().mgpuStreamSynchronize(stream)
    buf._keep = arr
    return buf


def to_host(buf: DeviceBuffer, shape, dtype, stream=None, offset_bytes: int = 0) -> np.ndarray:
    out = np.empty(shape, dtype=dtype)
    if out.nbytes:
        runtime().mgpuMemcpy(out.ctypes.data, buf.ptr + offset_bytes, out.nbytes, stream)
    runtime().mgpuStreamSynchronize(stream)
    return out


def _np16(dtype):
    return np.float16 if dtype == F16 else np.uint16


def encode16(x: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 array -> the 16-bit storage array for F16 / BF16."""
    if dtype == F16:
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)
    return f32_to_bf16_bits(x)


def decode16(x: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F16:
        return x.astype(np.float32)
    return bf16_bits_to_f32(x)


# ---------------------------------------------------------------- op conveniences
def add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    da, db = to_device(a), to_device(b)
    dc = DeviceBuffer(a.nbytes)
    ops().mgpuAdd(da.ptr, db.ptr, dc.ptr, a.size, None)
    out = to_host(dc, a.shape, np.float32)
    check("mgpuAdd")
    return out


def bias_add(x: np.ndarray, bias: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    dx, db = to_device(x), to_device(bias)
    dy = DeviceBuffer(x.nbytes)
    ops().mgpuBiasAdd(dx.ptr, db.ptr, dy.ptr, x.size // bias.size, bias.size, None)
    out = to_host(dy, x.shape, np.float32)
    check("mgpuBiasAdd")
    return out


def activation(x: np.ndarray, act: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    dx = to_device(x)
    dy = DeviceBuffer(x.nbytes)
    ops().mgpuActivation(dx.ptr, dy.ptr, x.size, act, None)
    out = to_host(dy, x.shape, np.float32)
    check("mgpuActivation")
    return out


def cast(x: np.ndarray, src: int, dst: int) -> np.ndarray:
    """x is the storage array of `src` (float32, float16 or uint16 bf16 bits)."""
    x = np.ascontiguousarray(x)
    dx = to_device(x)
    item = 4 if dst == F32 else 2
    dy = DeviceBuffer(x.size * item)
    ops().mgpuCast(dx.ptr, src, dy.ptr, dst, x.size, None)
    out = to_host(dy, x.shape, np.float32 if dst == F32 else _np16(dst))
    check("mgpuCast")
    return out


def conv2d(x, w, bias, post_add=None, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1), relu=False):
    """mgpuConv2d on numpy arrays: x [N,IC,H,W], w [OC,IC,KH,KW], pad = (top, left, bottom, right)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    N, IC, H, W = x.shape
    OC, _, KH, KW = w.shape
    OH = (H + pad[0] + pad[2] - (KH - 1) * dilation[0] - 1) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - (KW - 1) * dilation[1] - 1) // stride[1] + 1
    dx, dw, db = to_device(x), to_device(w), to_device(bias)
    dp = to_device(np.ascontiguousarray(post_add, dtype=np.float32)) if post_add is not None else None
    dy = DeviceBuffer(N * OC * OH * OW * 4)
    ops().mgpuConv2d(dx.ptr, dw.ptr, db.ptr, dy.ptr, dp.ptr if dp else None, N, IC, H, W, OC, KH, KW, OH, OW,
                     pad[0], pad[1], pad[2], pad[3], stride[0], stride[1], dilation[0], dilation[1],
                     post_add is not None, bool(relu), None)
    out = to_host(dy, (N, OC, OH, OW), np.float32)
    status = ops().mgpuOpsCheckDeviceStatus(None)
    check("mgpuConv2d")
    if status:
        raise MdcError(f"device status 0x{status:08x}")
    return out


def pool2d(x, kernel, stride, pad=(0, 0, 0, 0), method=0):
    """mgpuPool2d on a numpy array [N,C,H,W]; method 0 = max, 1 = average with the padding counted."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    N, Cc, H, W = x.shape
    OH = (H + pad[0] + pad[2] - kernel[0]) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - kernel[1]) // stride[1] + 1
    dx = to_device(x)
    dy = DeviceBuffer(N * Cc * OH * OW * 4)
    ops().mgpuPool2d(dx.ptr, dy.ptr, N, Cc, H, W, OH, OW, kernel[0], kernel[1], pad[0], pad[1], pad[2], pad[3],
                     stride[0], stride[1], method, None)
    out = to_host(dy, (N, Cc, OH, OW), np.float32)
    check("mgpuPool2d")
    return out


def layernorm(x, gamma=None, beta=None, eps=1e-5, residual=None, io_dtype=F32, out_dtype=F32,
              return_sum=False):
    """x / residual are storage arrays of io_dtype; returns the storage array of out_dtype."""
    x = np.ascontiguousarray(x)
    n = x.shape[-1]
    m = x.size // n
    dx = to_device(x)
    dr = to_device(np.ascontiguousarray(residual)) if residual is not None else None
    dg = to_device(np.ascontiguousarray(gamma, dtype=np.float32)) if gamma is not None else None
    db = to_device(np.ascontiguousarray(beta, dtype=np.float32)) if beta is not None else None
    item_out = 4 if out_dtype == F32 else 2
    dy = DeviceBuffer(x.size * item_out)
    ds = DeviceBuffer(x.nbytes) if return_sum else None
    ops().mgpuLayerNormEx(dx.ptr, dr.ptr if dr else None, dg.ptr if dg else None,
                          db.ptr if db else None, ds.ptr if ds else None, dy.ptr, eps, m, n,
                          io_dtype, out_dtype, None)
    y = to_host(dy, x.shape, np.float32 if out_dtype == F32 else _np16(out_dtype))
    check("mgpuLayerNormEx")
    if return_sum:
        return y, to_host(ds, x.shape, x.dtype)
    return y


def matmul(inp: np.ndarray, w_kn: np.ndarray, bias=None) -> np.ndarray:
    """The reference entry point mgpuMatmul: fp32 in / out, weight [K, N]."""
    inp = np.ascontiguousarray(inp, dtype=np.float32)
    w_kn = np.ascontiguousarray(w_kn, dtype=np.float32)
    K, N = w_kn.shape
    M = inp.size // K
    if bias is None:
        bias = np.zeros(N, dtype=np.float32)
    di, dw, db = to_device(inp), to_device(w_kn), to_device(np.ascontiguousarray(bias, dtype=np.float32))
    do = DeviceBuffer(M * N * 4)
    ops().mgpuMatmul(di.ptr, dw.ptr, db.ptr, do.ptr, M, N, K, None)
    out = to_host(do, inp.shape[:-1] + (N,), np.float32)
    status = ops().mgpuOpsCheckDeviceStatus(None)
    check("mgpuMatmul")
    if status:
        raise MdcError(f"device status 0x{status:08x}")
    return out


def matmul16(a: np.ndarray, w_kn: np.ndarray, bias=None, residual=None, act=ACT_NONE, dtype=F16,
             out_dtype=None) -> np.ndarray:
    """mgpuPackWeight + mgpuMatmulEx16 on fp32 numpy inputs (rounded to `dtype` first).
    Returns fp32 values (decoded from out_dtype)."""
    out_dtype = dtype if out_dtype is None else out_dtype
    a = np.ascontiguousarray(a, dtype=np.float32)
    w_kn = np.ascontiguousarray(w_kn, dtype=np.float32)
    K, N = w_kn.shape
    M = a.size // K
    Kp = (K + 7) // 8 * 8
    a16 = np.zeros((M, Kp), dtype=_np16(dtype))
    a16[:, :K] = encode16(a.reshape(M, K), dtype)
    da, dw = to_device(a16), to_device(w_kn)
    dwp = DeviceBuffer(N * Kp * 2)
    ops().mgpuPackWeight(dw.ptr, dwp.ptr, K, N, dtype, None)
    db = to_device(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
    dr = to_device(encode16(np.asarray(residual, dtype=np.float32).reshape(M, N), dtype)) if residual is not None else None
    item = 4 if out_dtype == F32 else 2
    do = DeviceBuffer(M * N * item)
    ops().mgpuMatmulEx16(da.ptr, dwp.ptr, db.ptr if db else None, dr.ptr if dr else None, do.ptr,
                         M, N, Kp, dtype, out_dtype, act, None)
    raw = to_host(do, (M, N), np.float32 if out_dtype == F32 else _np16(out_dtype))
    status = ops().mgpuOpsCheckDeviceStatus(None)
    check("mgpuMatmulEx16")
    if status:
        raise MdcError(f"device status 0x{status:08x}")
    return raw if out_dtype == F32 else decode16(raw, out_dtype)


def attention(qkv: np.ndarray, seq_lens, B, S, H, D, causal=False, dtype=F16) -> np.ndarray:
    """qkv fp32 [B*S, 3, H, D] (rounded to dtype); returns fp32 [B*S, H*D]."""
    q16 = encode16(np.ascontiguousarray(qkv, dtype=np.float32).reshape(B * S, 3 * H * D), dtype)
    dq = to_device(q16)
    dl = to_device(np.ascontiguousarray(seq_lens, dtype=np.int32)) if seq_lens is not None else None
    do = DeviceBuffer(B * S * H * D * 2)
    runtime().mgpuMemset16(do.ptr, 0, B * S * H * D, None)
    ops().mgpuAttention(dq.ptr, dl.ptr if dl else None, do.ptr, B, S, H, D, causal, dtype, None)
    raw = to_host(do, (B * S, H * D), _np16(dtype))
    status = ops().mgpuOpsCheckDeviceStatus(None)
    check("mgpuAttention")
    if status:
        raise MdcError(f"device status 0x{status:08x}")
    return decode16(raw, dtype)


_W_KEYS = ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2", "ln1_g", "ln1_b", "ln2_g", "ln2_b")


class EncoderStack:
    """Handle over mgpuEncoderStack*: weights are uploaded and packed once."""

    def __init__(self, layers, heads, norm_first=False, causal=False, act=ACT_GELU_ERF, dtype=F16,
                 eps=1e-5):
        self.d = int(layers[0]["wqkv"].shape[0])
        self.F = int(layers[0]["w1"].shape[1])
        self.h = ops().mgpuEncoderStackCreate(len(layers), self.d, self.F, heads, norm_first, causal,
                                              act, dtype, eps)
        if not self.h:
            check("mgpuEncoderStackCreate")
            raise MdcError("mgpuEncoderStackCreate failed")
        for i, lw in enumerate(layers):
            bufs = [to_device(np.ascontiguousarray(lw[k], dtype=np.float32)) if lw.get(k) is not None else None
                    for k in _W_KEYS]
            ops().mgpuEncoderStackSetLayer(self.h, i, *[b.ptr if b else None for b in bufs], None)
            runtime().mgpuStreamSynchronize(None)
            for b in bufs:
                if b:
                    b.release()
        check("mgpuEncoderStackSetLayer")

    def run(self, x: np.ndarray, seq_lens=None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        B, S, d = x.shape
        dx = to_device(x)
        dl = to_device(np.ascontiguousarray(seq_lens, dtype=np.int32)) if seq_lens is not None else None
        dy = DeviceBuffer(x.nbytes)
        ops().mgpuEncoderStackRun(self.h, dx.ptr, dl.ptr if dl else None, dy.ptr, B, S, None)
        y = to_host(dy, x.shape, np.float32)
        status = ops().mgpuOpsCheckDeviceStatus(None)
        check("mgpuEncoderStackRun")
        if status:
            raise MdcError(f"device status 0x{status:08x}")
        return y

    def run_device(self, x_ptr, lens_ptr, y_ptr, B, S, stream=None):
        ops().mgpuEncoderStackRun(self.h, x_ptr, lens_ptr, y_ptr, B, S, stream)

    def run_host(self, x: np.ndarray, y: np.ndarray, seq_lens=None, chunks=4):
        """x, y: C-contiguous fp32 host arrays (pin them with mgpuMemHostRegister for speed)."""
        B, S, _ = x.shape
        lens = np.ascontiguousarray(seq_lens, dtype=np.int32) if seq_lens is not None else None
        ops().mgpuEncoderStackRunHost(self.h, x.ctypes.data, lens.ctypes.data if lens is not None else None,
                                      y.ctypes.data, B, S, chunks)

    def submit_host(self, x: np.ndarray, y: np.ndarray, seq_lens=None) -> int:
        """Queue one batch (upload, stack, download) and return its ticket without waiting.  x, y
        (and seq_lens, int32) must stay alive and untouched until wait_host(ticket)."""
        B, S, _ = x.shape
        if seq_lens is not None and (seq_lens.dtype != np.int32 or not seq_lens.flags.c_contiguous):
            raise ValueError("seq_lens must be a C-contiguous int32 array that outlives the call")
        t = ops().mgpuEncoderStackSubmitHost(self.h, x.ctypes.data, seq_lens.ctypes.data if seq_lens is not None else None,
                                             y.ctypes.data, B, S)
        if t < 0:
            check("mgpuEncoderStackSubmitHost")
            raise MdcError("mgpuEncoderStackSubmitHost failed")
        return t

    def wait_host(self, ticket: int) -> None:
        ops().mgpuEncoderStackWaitHost(self.h, ticket)
        check("mgpuEncoderStackWaitHost")

    def close(self):
        if self.h:
            ops().mgpuEncoderStackDestroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
