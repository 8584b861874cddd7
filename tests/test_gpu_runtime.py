"""GPU tests of the runtime wrappers' copy path (reference: mgpuMemcpy,
lib/Runtime/CUDA/CudaRuntimeWrappers.cpp:226-231).  Copies between pageable host memory and
the device of 1 MiB and more are cut into chunks staged through pinned buffers by a team of
host threads; these tests check that the bytes arrive unchanged at every chunk boundary."""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MIB = 1 << 20


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _roundtrip(m, nbytes, stream=None, seed=0):
    rt = m.runtime()
    rng = np.random.default_rng(seed)
    src = rng.integers(0, 256, size=nbytes, dtype=np.uint8)
    keep = src.copy()
    buf = m.DeviceBuffer(nbytes, stream)
    rt.mgpuMemcpy(buf.ptr, src.ctypes.data, nbytes, stream)
    # the call returns once the source has been read: the caller may overwrite it now
    src[:] = 0
    out = np.full(nbytes, 0xA5, dtype=np.uint8)
    rt.mgpuMemcpy(out.ctypes.data, buf.ptr, nbytes, stream)
    # a copy into pageable memory is complete on return for staged sizes; smaller ones need the sync
    rt.mgpuStreamSynchronize(stream)
    buf.release(stream)
    m.check("mgpuMemcpy round trip")
    assert np.array_equal(out, keep)


@pytest.mark.parametrize("nbytes", [MIB - 1, MIB, MIB + 1, 4 * MIB - 64, 4 * MIB, 4 * MIB + 3,
                                    16 * MIB, 16 * MIB + 4097, 37 * MIB + 12345])
def test_pageable_roundtrip_sizes(m, nbytes):
    _roundtrip(m, nbytes)


def test_pageable_roundtrip_on_created_stream(m):
    rt = m.runtime()
    s = rt.mgpuStreamCreate()
    try:
        _roundtrip(m, 9 * MIB + 5, stream=s, seed=1)
        _roundtrip(m, 21 * MIB, stream=s, seed=2)
    finally:
        rt.mgpuStreamDestroy(s)


def test_unaligned_host_addresses(m):
    rt = m.runtime()
    n = 6 * MIB + 17
    backing = np.random.default_rng(3).integers(0, 256, size=n + 64, dtype=np.uint8)
    src = backing[13:13 + n]
    out_backing = np.zeros(n + 64, dtype=np.uint8)
    out = out_backing[7:7 + n]
    buf = m.DeviceBuffer(n)
    rt.mgpuMemcpy(buf.ptr, src.ctypes.data, n, None)
    rt.mgpuMemcpy(out.ctypes.data, buf.ptr, n, None)
    rt.mgpuStreamSynchronize(None)
    buf.release()
    assert np.array_equal(out, src)
    assert not out_backing[:7].any() and not out_backing[7 + n:].any()


def test_upload_then_kernel_sees_all_chunks(m):
    """Add over arrays spanning many staging chunks: every chunk must have landed before the
    kernel that follows on the same stream reads it."""
    n = 5 * MIB + 3  # 20 MiB + 12 B per array
    rng = np.random.default_rng(4)
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    assert np.array_equal(m.add(a, b), a + b)


def test_pageable_copy_rate_report(m, capsys):
    """Not a pass/fail threshold: prints the achieved rates so a log shows them."""
    rt = m.runtime()
    n = 256 * MIB
    src = np.ones(n, dtype=np.uint8)
    out = np.empty(n, dtype=np.uint8)
    buf = m.DeviceBuffer(n)
    rates = {}
    for name, dst, s in (("h2d", buf.ptr, src.ctypes.data), ("d2h", out.ctypes.data, buf.ptr)):
        best = 0.0
        for _ in range(3):
            t0 = time.perf_counter()
            rt.mgpuMemcpy(dst, s, n, None)
            rt.mgpuStreamSynchronize(None)
            best = max(best, n / (time.perf_counter() - t0) / 1e9)
        rates[name] = best
    buf.release()
    assert out[0] == 1 and out[-1] == 1
    with capsys.disabled():
        print(f"\n[pageable mgpuMemcpy, 256 MiB] h2d {rates['h2d']:.1f} GB/s, d2h {rates['d2h']:.1f} GB/s")
