"""mgpuMatmulNoAlloc: the matmul entry point for callers that cannot allocate device memory
(latency-critical loops that cannot take cudaMalloc's device-wide synchronisation, or
processes whose device memory another component has already reserved in full).

It must give what mgpuMatmul gives, from a fixed scratch array inside the library, without
asking the device pool (or the driver) for memory, on repeated calls that reuse the array,
and it must refuse problems larger than the array.  Collected last on purpose: a failure
here cannot hide another test's result when a run stops at the first failure."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-2  # 16-bit tensor-core Gemm: max-rel, error divided by max(|ref|, 1e-2 * rms(ref))


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _both(m, a, w, b):
    """Runs mgpuMatmul and mgpuMatmulNoAlloc on the same device buffers; returns both results
    and the growth of the pool's reserved bytes across the no-alloc call."""
    K, N = w.shape
    M = a.size // K
    da, dw, db = m.to_device(a), m.to_device(w), m.to_device(b)
    d1, d2 = m.DeviceBuffer(M * N * 4), m.DeviceBuffer(M * N * 4)
    rt, ops = m.runtime(), m.ops()
    ops.mgpuMatmul(da.ptr, dw.ptr, db.ptr, d1.ptr, M, N, K, None)
    y1 = m.to_host(d1, (M, N), np.float32)
    rt.mgpuMemset32(d2.ptr, 0x7FC00000, M * N, None)  # NaN fill: every element must be written
    reserved = rt.mgpuPoolReservedBytes()
    in_use = rt.mgpuPoolInUseBytes()
    ops.mgpuMatmulNoAlloc(da.ptr, dw.ptr, db.ptr, d2.ptr, M, N, K, None)
    y2 = m.to_host(d2, (M, N), np.float32)
    grew = (rt.mgpuPoolReservedBytes() - reserved, rt.mgpuPoolInUseBytes() - in_use)
    assert ops.mgpuOpsCheckDeviceStatus(None) == 0
    m.check("mgpuMatmulNoAlloc")
    return y1, y2, grew


def test_two_calls_in_a_row_match_mgpu_matmul(m):
    rng = np.random.default_rng(0)
    # first call: K not a multiple of 8 (padded operand rows), ragged M and N
    a = rng.standard_normal((300, 515)).astype(np.float32)
    w = (0.05 * rng.standard_normal((515, 264))).astype(np.float32)
    b = (0.05 * rng.standard_normal(264)).astype(np.float32)
    y1, y2, grew = _both(m, a, w, b)
    assert grew == (0, 0)  # nothing was taken from the pool
    assert np.array_equal(y1, y2)
    assert oracle.max_rel_err(oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16), y2) <= TOL
    # second call, smaller and differently shaped: the array still holds the first call's
    # operands, none of which may leak into this result
    a = rng.standard_normal((64, 72)).astype(np.float32)
    w = (0.05 * rng.standard_normal((72, 40))).astype(np.float32)
    b = (0.05 * rng.standard_normal(40)).astype(np.float32)
    y1, y2, grew = _both(m, a, w, b)
    assert grew == (0, 0)
    assert np.array_equal(y1, y2)
    assert oracle.max_rel_err(oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16), y2) <= TOL
    # third call near the limit of the array (1024 x 768 x 4096 needs 14 MiB of its 16)
    a = rng.standard_normal((1024, 4096)).astype(np.float32)
    w = (0.02 * rng.standard_normal((4096, 768))).astype(np.float32)
    b = np.zeros(768, np.float32)
    y1, y2, grew = _both(m, a, w, b)
    assert grew == (0, 0)
    assert np.array_equal(y1, y2)


def test_sizes_beyond_the_fixed_array_are_rejected(m):
    rt, ops = m.runtime(), m.ops()
    rt.mgpuClearLastError()
    M, N, K = 2048, 4096, 4096  # needs 48 MiB of scratch
    out = m.DeviceBuffer(16)
    launches = ops.mgpuOpsLaunchCount()
    ops.mgpuMatmulNoAlloc(out.ptr, out.ptr, out.ptr, out.ptr, M, N, K, None)  # must not touch the pointers
    assert ops.mgpuOpsLaunchCount() == launches
    assert rt.mgpuGetLastError() != 0
    msg = rt.mgpuGetLastErrorString().decode()
    assert "mgpuMatmulNoAlloc" in msg and "scratch" in msg
    rt.mgpuClearLastError()


def test_first_library_call_in_a_fresh_process_and_no_driver_allocation():
    """A process whose FIRST operator-library call is mgpuMatmulNoAlloc (no mgpuOpsInit, no
    other op before it): the result must be right, the device status word must be readable
    (and zero) although nothing ever allocated it, and a warmed call must leave the driver's
    free-memory figure untouched, which also sees a direct cudaMalloc that the pool counters
    cannot."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = textwrap.dedent(f"""
        import ctypes as C, sys
        import numpy as np
        sys.path.insert(0, {root!r}); sys.path.insert(0, {os.path.join(root, "oracle")!r})
        import __graft_entry__ as entry
        import oracle
        m = entry.load_package()
        rt, ops = m.runtime(), m.ops()          # libraries loaded; mgpuOpsInit is NOT called
        rng = np.random.default_rng(3)
        M, N, K = 200, 136, 100
        a = rng.standard_normal((M, K)).astype(np.float32)
        w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
        b = (0.05 * rng.standard_normal(N)).astype(np.float32)
        da, dw, db, do = m.to_device(a), m.to_device(w), m.to_device(b), m.DeviceBuffer(M * N * 4)
        assert ops.mgpuOpsLaunchCount() == 0
        ops.mgpuMatmulNoAlloc(da.ptr, dw.ptr, db.ptr, do.ptr, M, N, K, None)   # the first op call
        y = m.to_host(do, (M, N), np.float32)
        assert ops.mgpuOpsCheckDeviceStatus(None) == 0
        m.check("first call")
        err = oracle.max_rel_err(oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16), y)
        assert err <= {TOL}, err
        free0, free1, total = C.c_uint64(), C.c_uint64(), C.c_uint64()
        rt.mgpuStreamSynchronize(None)
        rt.mgpuMemGetInfo(C.byref(free0), C.byref(total))
        for _ in range(3):
            ops.mgpuMatmulNoAlloc(da.ptr, dw.ptr, db.ptr, do.ptr, M, N, K, None)
        rt.mgpuStreamSynchronize(None)
        assert ops.mgpuOpsCheckDeviceStatus(None) == 0
        rt.mgpuMemGetInfo(C.byref(free1), C.byref(total))
        assert free0.value == free1.value, (free0.value, free1.value)
        assert np.array_equal(m.to_host(do, (M, N), np.float32), y)
        m.check("warmed calls")
        print("NOALLOC_FRESH_OK")
    """)
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, cwd=root)
    assert res.returncode == 0 and "NOALLOC_FRESH_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
