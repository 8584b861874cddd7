"""GPU parity: elementwise ops, casts and LayerNorm against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _uniform(shape, seed):
    return np.random.default_rng(seed).uniform(-1, 1, shape).astype(np.float32)


@pytest.mark.parametrize("shape", [(3, 640, 640), (2, 10, 10), (3, 32, 32), (1,), (1000003,), (9830400,)])
def test_add_bit_exact(m, shape):
    # (3,640,640): test/End2End/GPU/add.mlir:4-5; (2,10,10): add.mlir:14-28
    a, b = _uniform(shape, 0), _uniform(shape, 1)
    got = m.add(a, b)
    assert np.array_equal(got.view(np.uint32), oracle.add(a, b).view(np.uint32))


def test_add_empty_and_unaligned(m):
    assert m.add(np.zeros(0, np.float32), np.zeros(0, np.float32)).size == 0
    # pointers offset by one float: the kernel must take its scalar path
    n = 4099
    a, b = _uniform(n + 1, 2), _uniform(n + 1, 3)
    da, db = m.to_device(a), m.to_device(b)
    dc = m.DeviceBuffer((n + 1) * 4)
    m.runtime().mgpuMemset32(dc.ptr, 0, n + 1, None)
    m.ops().mgpuAdd(da.ptr + 4, db.ptr + 4, dc.ptr + 4, n, None)
    out = m.to_host(dc, (n + 1,), np.float32)
    m.check("mgpuAdd")
    assert out[0] == 0.0
    assert np.array_equal(out[1:], a[1:] + b[1:])


def test_add_special_values(m):
    a = np.array([np.inf, -np.inf, np.nan, 0.0, -0.0, 1e-45, 3.4e38, 3.4e38], np.float32)
    b = np.array([1.0, np.inf, 1.0, -0.0, -0.0, 1e-45, 3.4e38, -3.4e38], np.float32)
    got, ref = m.add(a, b), oracle.add(a, b)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok].view(np.uint32), ref[ok].view(np.uint32))


@pytest.mark.parametrize("rows,cols", [(96, 64), (7, 13), (2048, 4096)])
def test_bias_add(m, rows, cols):
    x, b = _uniform((rows, cols), 4), _uniform(cols, 5)
    assert np.array_equal(m.bias_add(x, b), oracle.bias_add(x, b))


@pytest.mark.parametrize("act,tol", [(1, 0.0), (2, 1e-5), (3, 1e-5)])
def test_activation(m, act, tol):
    x = (4 * np.random.default_rng(6).standard_normal(100001)).astype(np.float32)
    got, ref = m.activation(x, act), oracle.activation(x, act)
    assert np.max(np.abs(got - ref)) <= tol  # fp32 elementwise: max-abs <= 1e-5


@pytest.mark.parametrize("n", [1, 7, 8, 4096, 100003])
def test_casts(m, n):
    x = (100 * np.random.default_rng(7).standard_normal(n)).astype(np.float32)
    h = m.cast(x, m.F32, m.F16)
    assert np.array_equal(h.view(np.uint16), x.astype(np.float16).view(np.uint16))
    b = m.cast(x, m.F32, m.BF16)
    assert np.array_equal(b, m.f32_to_bf16_bits(x))
    assert np.array_equal(m.cast(h, m.F16, m.F32), h.astype(np.float32))
    assert np.array_equal(m.cast(b, m.BF16, m.F32), m.bf16_bits_to_f32(b))


# fp32 LayerNorm: max-abs error <= 1e-5 against the oracle (double-precision statistics)
@pytest.mark.parametrize("shape", [(32, 512, 768), (32, 512, 1024), (5, 7, 48), (3, 2048), (4, 4096),
                                   (9, 770), (6, 1000), (11, 7), (2, 1), (1, 12288)])
def test_layernorm_f32(m, shape):
    rng = np.random.default_rng(8)
    x = rng.standard_normal(shape).astype(np.float32)
    n = shape[-1]
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    got = m.layernorm(x, g, b, 1e-5)
    ref = oracle.layernorm(x, g, b, 1e-5)
    assert np.max(np.abs(got - ref)) <= 1e-5


def test_layernorm_f32_golden_and_no_affine(m, golden):
    got = m.layernorm(golden["ln_x"], golden["ln_g"], golden["ln_b"], 1e-5)
    assert np.max(np.abs(got - golden["ln_y"])) <= 1e-5
    x = golden["ln_x"]
    assert np.max(np.abs(m.layernorm(x, None, None, 1e-5) - oracle.layernorm(x, None, None, 1e-5))) <= 1e-5


def test_layernorm_f32_large_offset_rows(m):
    # mean far from zero: a sum-of-squares formulation would lose the variance here
    rng = np.random.default_rng(9)
    x = (1000.0 + rng.standard_normal((64, 768))).astype(np.float32)
    got, ref = m.layernorm(x, None, None, 1e-5), oracle.layernorm(x, None, None, 1e-5)
    assert np.max(np.abs(got - ref)) <= 2e-4  # input quantum at 1000 is 6e-5; the oracle sees the same inputs


@pytest.mark.parametrize("dtype_name", ["f16", "bf16"])
@pytest.mark.parametrize("n", [768, 1024, 72])
def test_layernorm_16bit_with_residual(m, dtype_name, n):
    dt = m.F16 if dtype_name == "f16" else m.BF16
    rm = oracle.ROUND_F16 if dt == m.F16 else oracle.ROUND_BF16
    rng = np.random.default_rng(10)
    x = oracle.round_array(rng.standard_normal((130, n)).astype(np.float32), rm)
    r = oracle.round_array(rng.standard_normal((130, n)).astype(np.float32), rm)
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    y, s = m.layernorm(m.encode16(x, dt), g, b, 1e-5, residual=m.encode16(r, dt), io_dtype=dt,
                       out_dtype=dt, return_sum=True)
    ref_y, ref_s = oracle.layernorm(x, g, b, 1e-5, residual=r, sum_round=rm, out_round=rm, return_sum=True)
    assert np.array_equal(m.decode16(s, dt), ref_s)  # the sum is a single rounded add
    tol = 2 ** -9 if dt == m.F16 else 2 ** -6  # one output ulp at |y| < 8
    assert np.max(np.abs(m.decode16(y, dt) - ref_y)) <= tol
    # 16-bit in, fp32 out (the last LayerNorm of a post-LN stack)
    y32 = m.layernorm(m.encode16(x, dt), g, b, 1e-5, io_dtype=dt, out_dtype=m.F32)
    assert np.max(np.abs(y32 - oracle.layernorm(x, g, b, 1e-5))) <= 1e-5


@pytest.mark.parametrize("rows,n", [(4096, 768), (3001, 1024), (2051, 1536), (40000, 72)])
@pytest.mark.parametrize("dtype_name", ["f16", "bf16"])
def test_layernorm_16bit_large(m, rows, n, dtype_name):
    # sizes that take the shared-memory ring kernel (rows staged by bulk copies), including
    # a last group that is only partly filled
    dt = m.F16 if dtype_name == "f16" else m.BF16
    rm = oracle.ROUND_F16 if dt == m.F16 else oracle.ROUND_BF16
    rng = np.random.default_rng(11)
    x = oracle.round_array((2.0 * rng.standard_normal((rows, n)) + 0.5).astype(np.float32), rm)
    g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    b = (0.1 * rng.standard_normal(n)).astype(np.float32)
    ref = oracle.layernorm(x, g, b, 1e-5)
    y32 = m.layernorm(m.encode16(x, dt), g, b, 1e-5, io_dtype=dt, out_dtype=m.F32)
    assert np.max(np.abs(y32 - ref)) <= 1e-5
    y16 = m.decode16(m.layernorm(m.encode16(x, dt), g, b, 1e-5, io_dtype=dt, out_dtype=dt), dt)
    tol = 2 ** -9 if dt == m.F16 else 2 ** -6  # one output ulp at |y| < 8
    assert np.max(np.abs(y16 - ref)) <= tol
    assert m.ops().mgpuOpsCheckDeviceStatus(None) == 0
