"""numpy-facing wrapper over the C oracle (TEST INFRASTRUCTURE, not product).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import this module.
The arithmetic lives in mdc_oracle.c (each function there cites the reference lines it
restates); this file only marshals numpy arrays through ctypes.  PARITY UNPINNED against
oneDNN itself (the reference holds no golden vectors); pinned against fixtures made from
the reference's PyTorch model definitions (tests/golden/).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmdc_oracle.so")

ROUND_NONE, ROUND_F16, ROUND_BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH = 0, 1, 2, 3

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int32)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "mdc_oracle.c")
    graphs = os.path.join(_HERE, "libcpu_graph_add.so")
    if (force or not os.path.exists(_LIB_PATH) or not os.path.exists(graphs)
            or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
            or os.path.getmtime(graphs) < os.path.getmtime(os.path.join(_HERE, "cpu_graphs.c"))):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


class _LayerWeights(C.Structure):
    _fields_ = [(n, _fp) for n in ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2",
                                   "ln1_g", "ln1_b", "ln2_g", "ln2_b")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_blas(on: bool = True) -> bool:
    """Timed CPU baseline only: route the oracle's Gemm through cblas_sgemm of the OpenBLAS
    bundled with numpy (when the wheel carries one).  Returns whether it is in use."""
    import glob
    if not on:
        lib().oracle_use_blas(None, None)
        return False
    libs = glob.glob(os.path.join(os.path.dirname(np.__file__), "..", "numpy.libs", "libscipy_openblas64_*.so"))
    for path in libs:
        if lib().oracle_use_blas(os.path.abspath(path).encode(), b"scipy_cblas_sgemm64_"):
            return True
    return False


def gemm_kernel_name() -> str:
    if lib().oracle_blas_in_use():
        return "cblas_sgemm of the OpenBLAS bundled with numpy"
    return "own AVX2/FMA 4x32 register-panel loop (OpenMP)"


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_fp)


def _fo(a):
    if a is None:
        return None, None
    return _f(a)


def round_array(x, mode):
    x = np.array(x, dtype=np.float32, copy=True, order="C")
    lib().oracle_round_array(x.ctypes.data_as(_fp), C.c_int64(x.size), C.c_int(mode))
    return x


def add(a, b):
    a, pa = _f(a)
    b, pb = _f(b)
    assert a.shape == b.shape
    c = np.empty_like(a)
    lib().oracle_add_f32(pa, pb, c.ctypes.data_as(_fp), C.c_int64(a.size))
    return c


def bias_add(x, bias):
    x, px = _f(x)
    bias, pb = _f(bias)
    n = bias.size
    y = np.empty_like(x)
    lib().oracle_bias_add_f32(px, pb, y.ctypes.data_as(_fp), C.c_int64(x.size // n), C.c_int64(n))
    return y


def activation(x, act):
    x, px = _f(x)
    y = np.empty_like(x)
    lib().oracle_activation_f32(px, y.ctypes.data_as(_fp), C.c_int64(x.size), C.c_int(act))
    return y


def matmul(inp, w, bias=None, residual=None, round_mode=ROUND_NONE, accum64=False,
           act=ACT_NONE, out_round=ROUND_NONE):
    """out[M,N] = act(in[M,K] . w[K,N] + bias[N]) + residual[M,N]."""
    inp, pi = _f(inp)
    w, pw = _f(w)
    K, N = w.shape
    M = inp.size // K
    bias, pb = _fo(bias)
    residual, pr = _fo(residual)
    out = np.empty(inp.shape[:-1] + (N,), dtype=np.float32)
    lib().oracle_matmul_ex(pi, pw, pb, pr, out.ctypes.data_as(_fp), C.c_int64(M), C.c_int64(N),
                           C.c_int64(K), C.c_int(round_mode), C.c_int(int(accum64)), C.c_int(act),
                           C.c_int(out_round))
    return out


def layernorm(x, gamma=None, beta=None, eps=1e-5, residual=None, sum_round=ROUND_NONE,
              out_round=ROUND_NONE, return_sum=False):
    x, px = _f(x)
    n = x.shape[-1]
    m = x.size // n
    gamma, pg = _fo(gamma)
    beta, pbeta = _fo(beta)
    residual, pr = _fo(residual)
    y = np.empty_like(x)
    s = np.empty_like(x) if return_sum else None
    lib().oracle_layernorm_ex(px, pr, pg, pbeta, s.ctypes.data_as(_fp) if return_sum else None,
                              y.ctypes.data_as(_fp), C.c_float(eps), C.c_int64(m), C.c_int64(n),
                              C.c_int(sum_round), C.c_int(out_round))
    return (y, s) if return_sum else y


def conv2d(x, w, bias=None, post_add=None, stride=(1, 1), pad=(0, 0, 0, 0), dilation=(1, 1),
           relu=False, round_mode=ROUND_NONE, accum64=False):
    """x [N,IC,H,W], w [OC,IC,KH,KW]; pad = (top, left, bottom, right)."""
    x, px = _f(x)
    w, pw = _f(w)
    bias, pb = _fo(bias)
    post_add, pp = _fo(post_add)
    N, IC, H, W = x.shape
    OC, _, KH, KW = w.shape
    OH = (H + pad[0] + pad[2] - (KH - 1) * dilation[0] - 1) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - (KW - 1) * dilation[1] - 1) // stride[1] + 1
    out = np.empty((N, OC, OH, OW), dtype=np.float32)
    i64 = C.c_int64
    lib().oracle_conv2d(px, pw, pb, pp, out.ctypes.data_as(_fp), i64(N), i64(IC), i64(H), i64(W),
                        i64(OC), i64(KH), i64(KW), i64(OH), i64(OW), i64(pad[0]), i64(pad[1]),
                        i64(stride[0]), i64(stride[1]), i64(dilation[0]), i64(dilation[1]),
                        C.c_int(int(post_add is not None)), C.c_int(int(relu)), C.c_int(round_mode),
                        C.c_int(int(accum64)))
    return out


def pool2d(x, kernel, stride, pad=(0, 0, 0, 0), method=0):
    """x [N,C,H,W]; pad = (top, left, bottom, right); method 0 = max, 1 = average (padding counted)."""
    x, px = _f(x)
    N, Cc, H, W = x.shape
    OH = (H + pad[0] + pad[2] - kernel[0]) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - kernel[1]) // stride[1] + 1
    out = np.empty((N, Cc, OH, OW), dtype=np.float32)
    i64 = C.c_int64
    lib().oracle_pool2d(px, out.ctypes.data_as(_fp), i64(N), i64(Cc), i64(H), i64(W), i64(OH), i64(OW),
                        i64(kernel[0]), i64(kernel[1]), i64(pad[0]), i64(pad[1]), i64(pad[2]), i64(pad[3]),
                        i64(stride[0]), i64(stride[1]), C.c_int(method))
    return out


def attention(qkv, seq_lens, B, S, H, D, causal=False, round_mode=ROUND_NONE):
    """qkv: [B*S, 3, H, D] packed per token; returns [B*S, H*D]."""
    qkv, pq = _f(qkv)
    assert qkv.size == B * S * 3 * H * D
    lens = None
    pl = None
    if seq_lens is not None:
        lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        pl = lens.ctypes.data_as(_ip)
    out = np.empty((B * S, H * D), dtype=np.float32)
    lib().oracle_attention(pq, pl, out.ctypes.data_as(_fp), C.c_int64(B), C.c_int64(S),
                           C.c_int64(H), C.c_int64(D), C.c_int(int(causal)), C.c_int(round_mode))
    return out


_W_KEYS = ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2", "ln1_g", "ln1_b", "ln2_g", "ln2_b")


def _pack_weights(layers):
    """layers: list of dicts keyed like _W_KEYS (missing / None = absent)."""
    arr = (_LayerWeights * len(layers))()
    keep = []
    for i, lw in enumerate(layers):
        for k in _W_KEYS:
            v = lw.get(k)
            if v is None:
                setattr(arr[i], k, None)
            else:
                a, p = _f(v)
                keep.append(a)
                setattr(arr[i], k, p)
    return arr, keep


def encoder_stack(x, layers, seq_lens, heads, norm_first=False, causal=False, act=ACT_GELU_ERF,
                  eps=1e-5, round_mode=ROUND_F16):
    """x: [B,S,d] fp32; layers: list of weight dicts; returns [B,S,d] fp32."""
    x, px = _f(x)
    B, S, d = x.shape
    F = layers[0]["w1"].shape[1]
    arr, keep = _pack_weights(layers)
    lens = None
    pl = None
    if seq_lens is not None:
        lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        pl = lens.ctypes.data_as(_ip)
    y = np.empty_like(x)
    lib().oracle_encoder_stack(px, arr, C.c_int64(len(layers)), pl, y.ctypes.data_as(_fp),
                               C.c_int64(B), C.c_int64(S), C.c_int64(d), C.c_int64(F),
                               C.c_int64(heads), C.c_int(int(norm_first)), C.c_int(int(causal)),
                               C.c_int(act), C.c_float(eps), C.c_int(round_mode))
    del keep
    return y


def encoder_layer(x, weights, seq_lens, heads, **kw):
    return encoder_stack(x, [weights], seq_lens, heads, **kw)


def diff_table(standard, compare):
    """The comparison the reference's examples/data_diff.py:8-25 prints, as a dict."""
    a = np.asarray(standard, dtype=np.float32).ravel()
    b = np.asarray(compare, dtype=np.float32).ravel()
    ad = np.abs(a - b)
    rd = ad / (np.abs(a) + 1e-10)
    out = {"abs_min": float(ad.min()), "abs_max": float(ad.max()), "abs_mean": float(ad.mean()),
           "rel_min": float(rd.min()), "rel_max": float(rd.max()), "rel_mean": float(rd.mean())}
    for bound in (1, 1e-1, 1e-2, 1e-3, 1e-4, 1e-5, 1e-6, 1e-7):
        out[f"gt_{bound:g}"] = int(np.count_nonzero(ad > bound))
    return out


def max_rel_err(ref, got, floor_frac=1e-2):
    """max |got-ref| / max(|ref|, floor_frac * rms(ref)): relative error with a floor so
    that near-zero outputs of a 16-bit GEMM do not dominate."""
    ref = np.asarray(ref, dtype=np.float64).ravel()
    got = np.asarray(got, dtype=np.float64).ravel()
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    den = np.maximum(np.abs(ref), floor_frac * rms + 1e-30)
    return float(np.max(np.abs(got - ref) / den)) if ref.size else 0.0
