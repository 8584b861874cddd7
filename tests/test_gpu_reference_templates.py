"""GPU parity of the C++-linkage template instantiations the reference's other translation
units call (Kernels/GPU/Ops.h:51-74, Utils.h:6-8), reached here through their mangled names."""
import ctypes as C
import subprocess

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


@pytest.fixture(scope="module")
def cxx(m):
    """demangled name -> ctypes function of the operator library"""
    lib = m.ops()
    mangled = subprocess.run(["nm", "-D", "--defined-only", m.OPS_LIB], capture_output=True, text=True, check=True).stdout
    plain = subprocess.run(["nm", "-DC", "--defined-only", m.OPS_LIB], capture_output=True, text=True, check=True).stdout
    table = {}
    for a, b in zip(mangled.splitlines(), plain.splitlines()):
        sym, dem = a.split()[-1], b.split(" ", 2)[-1]
        if sym.startswith("_Z"):
            fn = getattr(lib, sym)
            fn.restype = None
            table[dem.split("(")[0].replace("void ", "")] = fn
    return table


def _h(m, x):
    return m.to_device(np.ascontiguousarray(x, dtype=np.float32).astype(np.float16))


def test_casts(m, cxx):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(1000).astype(np.float32)
    dx, dh, dy = m.to_device(x), m.DeviceBuffer(2000), m.DeviceBuffer(4000)
    cxx["invokeCudaCast<__half, float>"](C.c_void_p(dh.ptr), C.c_void_p(dx.ptr), C.c_size_t(1000), None)
    cxx["invokeCudaCast<float, __half>"](C.c_void_p(dy.ptr), C.c_void_p(dh.ptr), C.c_size_t(1000), None)
    assert np.array_equal(m.to_host(dy, (1000,), np.float32), x.astype(np.float16).astype(np.float32))
    m.check("invokeCudaCast")


@pytest.mark.parametrize("kind", ["half", "float"])
def test_matmul_ex(m, cxx, kind):
    rng = np.random.default_rng(1)
    M, N, K = 200, 136, 128
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.05 * rng.standard_normal(N)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    i64, cb, vp = C.c_int64, C.c_bool, C.c_void_p
    if kind == "half":
        da, dw, db, dr = _h(m, a), _h(m, w), _h(m, b), _h(m, r)
        do = m.DeviceBuffer(M * N * 2)
        cxx["mgpuMatmulEx<__half>"](vp(da.ptr), vp(dw.ptr), vp(db.ptr), vp(do.ptr), vp(dr.ptr), i64(M), i64(N), i64(K),
                                    cb(True), cb(False), cb(True), None)
        got = m.to_host(do, (M, N), np.float16).astype(np.float32)
        h = lambda x: x.astype(np.float16).astype(np.float32)
        ref = oracle.matmul(h(a), h(w), h(b), residual=h(r), round_mode=oracle.ROUND_F16, out_round=oracle.ROUND_F16)
    else:
        da, dw, db = m.to_device(a), m.to_device(w), m.to_device(b)
        do = m.DeviceBuffer(M * N * 4)
        cxx["mgpuMatmulEx<float>"](vp(da.ptr), vp(dw.ptr), vp(db.ptr), vp(do.ptr), None, i64(M), i64(N), i64(K),
                                   cb(True), cb(True), cb(False), None)
        got = m.to_host(do, (M, N), np.float32)
        ref = oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16, act=oracle.ACT_RELU)
    assert m.ops().mgpuOpsCheckDeviceStatus(None) == 0
    m.check("mgpuMatmulEx")
    assert oracle.max_rel_err(ref, got) <= TOL
    # the one combination whose epilogue order differs from the reference's is refused
    rt = m.runtime()
    cxx["mgpuMatmulEx<float>"](vp(da.ptr), vp(dw.ptr), vp(db.ptr), vp(do.ptr), vp(do.ptr), i64(M), i64(N), i64(K),
                               cb(True), cb(True), cb(True), None)
    assert rt.mgpuGetLastError() != 0
    rt.mgpuClearLastError()


def test_layernorm_and_add_residual_pre_layernorm(m, cxx):
    rng = np.random.default_rng(2)
    rows, n = 300, 768
    h = lambda x: np.asarray(x, np.float32).astype(np.float16).astype(np.float32)
    x, res = h(rng.standard_normal((rows, n))), h(rng.standard_normal((rows, n)))
    g, b = h(1 + 0.1 * rng.standard_normal(n)), h(0.1 * rng.standard_normal(n))
    dx, dr, dg, db = _h(m, x), _h(m, res), _h(m, g), _h(m, b)
    dy, ds = m.DeviceBuffer(rows * n * 2), m.DeviceBuffer(rows * n * 2)
    vp = C.c_void_p
    cxx["mgpuLayerNorm<__half>"](vp(dx.ptr), vp(dg.ptr), vp(db.ptr), vp(dy.ptr), C.c_float(1e-5), C.c_int(rows), C.c_int(n),
                                 None, None)
    got = m.to_host(dy, (rows, n), np.float16).astype(np.float32)
    assert np.max(np.abs(got - oracle.layernorm(x, g, b, 1e-5))) <= 4e-3     # one fp16 ulp of values up to 4
    cxx["mgpuAddResidualPreLayerNorm<__half>"](vp(dx.ptr), vp(dr.ptr), vp(dg.ptr), vp(db.ptr), vp(ds.ptr), vp(dy.ptr),
                                               C.c_float(1e-5), C.c_int(rows), C.c_int(n), None, None)
    s = m.to_host(ds, (rows, n), np.float16).astype(np.float32)
    got = m.to_host(dy, (rows, n), np.float16).astype(np.float32)
    assert np.array_equal(s, h(x + res))
    assert np.max(np.abs(got - oracle.layernorm(s, g, b, 1e-5))) <= 4e-3
    m.check("layernorm templates")


def test_qkv_bias_transpose(m, cxx):
    rng = np.random.default_rng(3)
    B, S, H, D = 2, 5, 3, 16
    n = H * D
    h = lambda x: np.asarray(x, np.float32).astype(np.float16)
    qkv, bias = h(rng.standard_normal((B * S, 3, n))), h(rng.standard_normal((3, n)))
    dq, dbias = m.to_device(qkv), m.to_device(bias)
    outs = [m.DeviceBuffer(B * H * S * D * 2) for _ in range(3)]
    vp, ci = C.c_void_p, C.c_int
    cxx["mgpuAddFusedQKVBiasTranspose<__half>"](vp(outs[0].ptr), vp(outs[1].ptr), vp(outs[2].ptr), vp(dq.ptr), vp(dbias.ptr),
                                                ci(B), ci(S), ci(B * S), ci(H), ci(D), None)
    want = (qkv + bias[None]).astype(np.float16)                               # one fp16 add per element
    assert np.array_equal(m.to_host(dq, qkv.shape, np.float16), want)          # written back in place
    for which in range(3):
        got = m.to_host(outs[which], (B, H, S, D), np.float16)
        ref = want[:, which].reshape(B, S, H, D).transpose(0, 2, 1, 3)
        assert np.array_equal(got, ref)
    m.check("qkv transpose")
