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


# A kernel in the form the reference's toolchain emits for an elementwise graph: PTX for sm_70
# (lib/Utils/CompileOptions.cpp:107-123) whose arguments are the expanded memref descriptors
# (allocated pointer, aligned pointer, offset, size, stride per operand).  The driver JIT-compiles
# it for sm_100 when mgpuModuleFileLoad hands the file to cuModuleLoad.
_ADD_PTX = """
.version 7.0
.target sm_70
.address_size 64

.visible .entry main_graph_kernel(
    .param .u64 a_alloc, .param .u64 a_aligned, .param .u64 a_off, .param .u64 a_size, .param .u64 a_stride,
    .param .u64 b_alloc, .param .u64 b_aligned, .param .u64 b_off, .param .u64 b_size, .param .u64 b_stride,
    .param .u64 c_alloc, .param .u64 c_aligned, .param .u64 c_off, .param .u64 c_size, .param .u64 c_stride)
{
    .reg .pred p;
    .reg .b32 r<5>;
    .reg .b64 rd<12>;
    .reg .f32 f<4>;
    ld.param.u64 rd1, [a_aligned];
    ld.param.u64 rd2, [b_aligned];
    ld.param.u64 rd3, [c_aligned];
    ld.param.u64 rd4, [a_size];
    mov.u32 r1, %ctaid.x;
    mov.u32 r2, %ntid.x;
    mov.u32 r3, %tid.x;
    mad.lo.s32 r4, r1, r2, r3;
    cvt.u64.u32 rd5, r4;
    setp.ge.u64 p, rd5, rd4;
    @p bra DONE;
    cvta.to.global.u64 rd1, rd1;
    cvta.to.global.u64 rd2, rd2;
    cvta.to.global.u64 rd3, rd3;
    shl.b64 rd6, rd5, 2;
    add.s64 rd7, rd1, rd6;
    add.s64 rd8, rd2, rd6;
    add.s64 rd9, rd3, rd6;
    ld.global.f32 f1, [rd7];
    ld.global.f32 f2, [rd8];
    add.f32 f3, f1, f2;
    st.global.f32 [rd9], f3;
DONE:
    ret;
}
"""


def test_ptx_module_from_the_reference_toolchain_loads_and_runs(m, tmp_path):
    rt = m.runtime()
    path = tmp_path / "ops.ptx"
    path.write_text(_ADD_PTX)
    n = 100_003
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    da, db, dc = m.to_device(a), m.to_device(b), m.DeviceBuffer(n * 4)
    rt.mgpuModuleFileLoad(str(path).encode())
    m.check("mgpuModuleFileLoad")
    fn = rt.mgpuModuleGetFunction(b"main_graph_kernel")
    assert fn
    vals = []
    for ptr in (da.ptr, db.ptr, dc.ptr):
        vals += [ptr, ptr, 0, n, 1]  # allocated, aligned, offset, size, stride
    cells = [C.c_uint64(v) for v in vals]
    params = (C.c_void_p * len(cells))(*[C.cast(C.pointer(c), C.c_void_p) for c in cells])
    block = 256
    rt.mgpuLaunchKernel(fn, (n + block - 1) // block, 1, 1, block, 1, 1, 0, None, params, None)
    rt.mgpuStreamSynchronize(None)
    m.check("launch of the loaded kernel")
    assert np.array_equal(m.to_host(dc, (n,), np.float32), a + b)
    # the built-in registry still answers while a module is loaded, and after it is unloaded
    assert rt.mgpuModuleGetFunction(b"mdc_add_f32")
    rt.mgpuModuleUnload()
    assert rt.mgpuModuleGetFunction(b"mdc_add_f32")
    m.check("module unload")


def test_kernel_override_routes_a_generated_kernel_to_the_builtin(m, tmp_path):
    """The module's kernel here SUBTRACTS, so the result tells which kernel ran: with the
    override in place the built-in Add runs on the generated kernel's own argument list."""
    rt = m.runtime()
    path = tmp_path / "ops.ptx"
    path.write_text(_ADD_PTX.replace("add.f32 f3, f1, f2;", "sub.f32 f3, f1, f2;"))
    n = 70_001
    rng = np.random.default_rng(6)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    da, db, dc = m.to_device(a), m.to_device(b), m.DeviceBuffer(n * 4)
    rt.mgpuModuleFileLoad(str(path).encode())
    vals = []
    for ptr in (da.ptr, db.ptr, dc.ptr):
        vals += [ptr, ptr, 0, n, 1]
    cells = [C.c_uint64(v) for v in vals]
    params = (C.c_void_p * len(cells))(*[C.cast(C.pointer(c), C.c_void_p) for c in cells])

    def launch():
        fn = rt.mgpuModuleGetFunction(b"main_graph_kernel")
        assert fn
        rt.mgpuLaunchKernel(fn, (n + 255) // 256, 1, 1, 256, 1, 1, 0, None, params, None)
        rt.mgpuStreamSynchronize(None)
        m.check("launch")
        return m.to_host(dc, (n,), np.float32)

    assert np.array_equal(launch(), a - b)
    rt.mgpuModuleOverrideKernel(b"main_graph_ker*", b"mdc_add_f32", 1)
    assert np.array_equal(launch(), a + b)
    # a non-contiguous operand is refused, not silently mishandled
    cells[4].value = 2
    fn = rt.mgpuModuleGetFunction(b"main_graph_kernel")
    rt.mgpuLaunchKernel(fn, 1, 1, 1, 256, 1, 1, 0, None, params, None)
    assert rt.mgpuGetLastError() != 0
    rt.mgpuClearLastError()
    cells[4].value = 1
    rt.mgpuModuleClearOverrides()
    assert np.array_equal(launch(), a - b)
    rt.mgpuModuleOverrideKernel(b"x", b"no_such_builtin", 1)
    assert rt.mgpuGetLastError() != 0
    rt.mgpuClearLastError()
    rt.mgpuModuleUnload()


# The same graph kernel in the argument form the reference's GPU pipeline really emits
# (lib/Pipelines/MLIRToGPU.cpp:162-165,180-183: bare pointers): one pointer per operand and
# nothing else, the static element count compiled into the code.
def _bare_ptx(n, op="add.f32"):
    return f"""
.version 7.0
.target sm_70
.address_size 64

.visible .entry main_graph_kernel(.param .u64 a, .param .u64 b, .param .u64 c)
{{
    .reg .pred p;
    .reg .b32 r<5>;
    .reg .b64 rd<12>;
    .reg .f32 f<4>;
    ld.param.u64 rd1, [a];
    ld.param.u64 rd2, [b];
    ld.param.u64 rd3, [c];
    mov.u32 r1, %ctaid.x;
    mov.u32 r2, %ntid.x;
    mov.u32 r3, %tid.x;
    mad.lo.s32 r4, r1, r2, r3;
    cvt.u64.u32 rd5, r4;
    setp.ge.u64 p, rd5, {n};
    @p bra DONE;
    cvta.to.global.u64 rd1, rd1;
    cvta.to.global.u64 rd2, rd2;
    cvta.to.global.u64 rd3, rd3;
    shl.b64 rd6, rd5, 2;
    add.s64 rd7, rd1, rd6;
    add.s64 rd8, rd2, rd6;
    add.s64 rd9, rd3, rd6;
    ld.global.f32 f1, [rd7];
    ld.global.f32 f2, [rd8];
    {op} f3, f1, f2;
    st.global.f32 [rd9], f3;
DONE:
    ret;
}}
"""


def test_kernel_override_with_bare_pointer_arguments(m, tmp_path):
    """A module kernel that SUBTRACTS, launched with the reference's bare-pointer argument
    array; once overridden, the built-in Add must run on those three pointers, with the element
    count taken from the registration or, when registered as 0, from the launch's grid x block."""
    rt = m.runtime()
    n = 3 * 640 * 64  # a multiple of the block, so grid x block covers it exactly
    path = tmp_path / "ops.ptx"
    path.write_text(_bare_ptx(n, "sub.f32"))
    rng = np.random.default_rng(8)
    a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    da, db, dc = m.to_device(a), m.to_device(b), m.DeviceBuffer(n * 4)
    rt.mgpuModuleFileLoad(str(path).encode())
    m.check("mgpuModuleFileLoad")
    cells = [C.c_uint64(p) for p in (da.ptr, db.ptr, dc.ptr)]
    params = (C.c_void_p * 3)(*[C.cast(C.pointer(c), C.c_void_p) for c in cells])

    def launch(grid):
        fn = rt.mgpuModuleGetFunction(b"main_graph_kernel")
        assert fn
        rt.mgpuMemset32(dc.ptr, 0x7FC00000, n, None)
        rt.mgpuLaunchKernel(fn, grid, 1, 1, 256, 1, 1, 0, None, params, None)
        rt.mgpuStreamSynchronize(None)
        m.check("launch")
        return m.to_host(dc, (n,), np.float32)

    assert np.array_equal(launch(n // 256), a - b)               # the module's own kernel
    rt.mgpuModuleOverrideKernelBare(b"main_graph_kernel", b"mdc_add_f32", n)
    assert np.array_equal(launch(n // 256 + 7), a + b)           # count from the registration
    rt.mgpuModuleOverrideKernelBare(b"main_graph_kernel", b"mdc_add_f32", 0)
    assert np.array_equal(launch(n // 256), a + b)               # count from grid x block
    rt.mgpuModuleClearOverrides()
    assert np.array_equal(launch(n // 256), a - b)
    rt.mgpuModuleOverrideKernelBare(b"x", b"no_such_builtin", 4)
    assert rt.mgpuGetLastError() != 0
    rt.mgpuClearLastError()
    rt.mgpuModuleUnload()


def test_pageable_copies_from_two_threads_at_once(m):
    """Two host threads upload and download different 8 MiB pageable buffers on their own
    streams at the same time: the staged-copy ring is one per process, so a second thread must
    neither corrupt the first one's chunks nor hang."""
    import threading
    rt = m.runtime()
    nbytes = 8 << 20
    results, errors = {}, []

    def worker(idx):
        try:
            rt.mgpuSetDefaultDevice(0)
            rng = np.random.default_rng(100 + idx)
            stream = rt.mgpuStreamCreate()
            buf = rt.mgpuMemAlloc(nbytes, stream)
            ok = True
            for rep in range(6):
                src = rng.integers(0, 256, nbytes, dtype=np.uint8)
                dst = np.zeros(nbytes, np.uint8)
                rt.mgpuMemcpy(buf, src.ctypes.data, nbytes, stream)
                rt.mgpuMemcpy(dst.ctypes.data, buf, nbytes, stream)
                rt.mgpuStreamSynchronize(stream)
                ok = ok and np.array_equal(src, dst)
            rt.mgpuMemFree(buf, stream)
            rt.mgpuStreamDestroy(stream)
            results[idx] = ok
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a copy thread is stuck"
    assert not errors, errors
    assert results == {0: True, 1: True}
    m.check("threaded copies")


def test_packed_weight_is_cached_for_copies_of_registered_constants(m):
    """A lowered graph uploads its weights with mgpuMemcpy on every call.  Once the host buffer is
    registered as a constant, mgpuMatmul packs the weight (cast + transpose) only the first time;
    a buffer that has since been overwritten from elsewhere is packed afresh."""
    import oracle
    rt, ops = m.runtime(), m.ops()
    rng = np.random.default_rng(12)
    M, K, N = 96, 200, 136
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    w2 = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.05 * rng.standard_normal(N)).astype(np.float32)
    da, db = m.to_device(a), m.to_device(b)
    dw, do = m.DeviceBuffer(w.nbytes), m.DeviceBuffer(M * N * 4)
    rt.mgpuRegisterConstant(w.ctypes.data, w.nbytes)

    def call():
        n0 = ops.mgpuOpsLaunchCount()
        ops.mgpuMatmul(da.ptr, dw.ptr, db.ptr, do.ptr, M, N, K, None)
        y = m.to_host(do, (M, N), np.float32)
        m.check("mgpuMatmul")
        return y, ops.mgpuOpsLaunchCount() - n0

    rt.mgpuMemcpy(dw.ptr, w.ctypes.data, w.nbytes, None)       # upload (served from the constant cache)
    assert rt.mgpuConstantSourceOf(dw.ptr) == w.ctypes.data
    y1, launches1 = call()
    rt.mgpuMemcpy(dw.ptr, w.ctypes.data, w.nbytes, None)       # the graph's next call uploads again
    y2, launches2 = call()
    assert launches2 == launches1 - 1                           # no pack kernel the second time
    assert np.array_equal(y1, y2)
    assert oracle.max_rel_err(oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16), y2) <= 2e-2
    # the same device buffer refilled from an ordinary host array: not a constant any more
    rt.mgpuMemcpy(dw.ptr, w2.ctypes.data, w2.nbytes, None)
    assert not rt.mgpuConstantSourceOf(dw.ptr)
    y3, launches3 = call()
    assert launches3 == launches1
    assert oracle.max_rel_err(oracle.matmul(a, w2, b, round_mode=oracle.ROUND_F16), y3) <= 2e-2
    rt.mgpuStreamSynchronize(None)
    rt.mgpuUnregisterConstant(w.ctypes.data)
    m.check("unregister")


def test_pool_guard_bands_catch_a_write_past_the_end():
    """MDC_POOL_GUARD=1 (read once per process, hence the child process): a write that runs past
    the end of a block lands in the guard band the pool keeps behind it, and freeing the block
    reports it; well-behaved use stays silent and the encoder layer still gives the same result."""
    import os
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = textwrap.dedent(f"""
        import sys
        import numpy as np
        sys.path.insert(0, {root!r})
        import __graft_entry__ as entry
        m = entry.load_package(); m.init(0)
        rt = m.runtime()
        a = np.arange(1000, dtype=np.float32)
        good = m.to_device(a)
        assert np.array_equal(m.add(a, a), a + a)            # ordinary use: no report
        good.release()
        assert rt.mgpuGetLastError() == 0
        buf = rt.mgpuMemAlloc(4000, None)
        rt.mgpuMemset32(buf, 0, 1001, None)                   # one element too many: into the band
        rt.mgpuMemFree(buf, None)
        assert rt.mgpuGetLastError() != 0
        assert b"guard band after" in rt.mgpuGetLastErrorString()
        rt.mgpuClearLastError()
        print("GUARD_OK")
    """)
    env = dict(os.environ, MDC_POOL_GUARD="1")
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert res.returncode == 0 and "GUARD_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-1500:]
