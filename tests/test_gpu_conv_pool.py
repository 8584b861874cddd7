"""GPU parity of mgpuConv2d / mgpuPool2d (reference: lib/Kernels/GPU/Ops.cu:238-374) against
the CPU oracle and the fixtures made from the reference's PyTorch models.

Tolerances: pooling is comparison / fp32 addition work -> max pooling bit-exact, average
pooling max-abs <= 1e-6 (summation order).  Convolution feeds 16-bit operands to the tensor
cores with fp32 accumulation, like the Gemm: max-rel <= 2e-2 against the oracle run on the
same 16-bit-rounded operands, an element's error divided by max(|ref|, 1e-2 * rms(ref))
(in fact the two agree to 2e-4 of the rms: only the fp32 summation order differs).  Against
the fp32 PyTorch fixtures the operand rounding itself is part of the difference (about
2^-12 of the rms per element whatever the element's size), so there the floor is
1e-1 * rms(ref)."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _check_conv(m, x, w, b, post_add=None, tol16=2e-4, floor32=1e-1, **kw):
    got = m.conv2d(x, w, b, post_add=post_add, **kw)
    ref32 = oracle.conv2d(x, w, b, post_add=post_add, accum64=True, **kw)
    ref16 = oracle.conv2d(x, w, b, post_add=post_add, round_mode=oracle.ROUND_F16, accum64=True, **kw)
    assert got.shape == ref32.shape
    assert oracle.max_rel_err(ref16, got, floor_frac=1e-2) <= 2e-2
    assert oracle.max_rel_err(ref32, got, floor_frac=floor32) <= 2e-2
    # same rounded operands, exact accumulation: only fp32 summation order is left
    scale = max(float(np.sqrt(np.mean(ref16.astype(np.float64) ** 2))), 1e-6)
    assert np.max(np.abs(got - ref16)) <= tol16 * scale
    return got


def test_reference_conv_fixture(m, golden_cnn):
    g = golden_cnn
    got = _check_conv(m, g["conv_x"], g["conv_w"], g["conv_b"], pad=(1, 1, 1, 1))
    assert oracle.max_rel_err(g["conv_y"], got, floor_frac=1e-1) <= 2e-2


def test_crosscheck_conv_fixtures(m, golden_cnn):
    g = golden_cnn
    got = _check_conv(m, g["res_x"], g["res_w"], g["res_b"], post_add=g["res_add"], stride=(2, 2),
                      pad=(1, 1, 1, 1), relu=True)
    assert oracle.max_rel_err(g["res_y"], got, floor_frac=1e-1) <= 2e-2
    got = _check_conv(m, g["dil_x"], g["dil_w"], g["dil_b"], stride=(1, 2), dilation=(2, 3))
    assert oracle.max_rel_err(g["dil_y"], got, floor_frac=1e-1) <= 2e-2


@pytest.mark.parametrize("shape", [
    # N, IC, H, W, OC, KH, KW, stride, pad(t,l,b,r), dilation, post_add, relu
    (1, 1, 5, 5, 1, 1, 1, (1, 1), (0, 0, 0, 0), (1, 1), False, False),
    (2, 3, 9, 11, 5, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1), False, True),
    (3, 16, 14, 14, 32, 1, 1, (1, 1), (0, 0, 0, 0), (1, 1), True, True),      # pointwise + residual
    (2, 7, 12, 10, 9, 5, 3, (2, 1), (2, 1, 2, 1), (1, 1), True, False),
    (1, 4, 17, 13, 6, 3, 3, (2, 2), (0, 1, 1, 0), (1, 1), False, False),     # asymmetric padding
    (2, 64, 28, 28, 128, 3, 3, (2, 2), (1, 1, 1, 1), (1, 1), False, True),   # a ResNet down-sampling layer
    (1, 3, 32, 32, 64, 7, 7, (2, 2), (3, 3, 3, 3), (1, 1), False, True),     # a ResNet stem
    (2, 6, 16, 16, 10, 3, 3, (1, 1), (2, 2, 2, 2), (2, 2), False, False),    # dilated, "same"
])
def test_conv_against_oracle(m, shape):
    N, IC, H, W, OC, KH, KW, stride, pad, dil, has_add, relu = shape
    rng = np.random.default_rng(hash(shape[:7]) % (1 << 31))
    x = rng.standard_normal((N, IC, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, IC, KH, KW)) / np.sqrt(IC * KH * KW)).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    OH = (H + pad[0] + pad[2] - (KH - 1) * dil[0] - 1) // stride[0] + 1
    OW = (W + pad[1] + pad[3] - (KW - 1) * dil[1] - 1) // stride[1] + 1
    add = rng.standard_normal((N, OC, OH, OW)).astype(np.float32) if has_add else None
    _check_conv(m, x, w, b, post_add=add, stride=stride, pad=pad, dilation=dil, relu=relu)


@pytest.mark.parametrize("OC", [128, 320])
def test_conv_wide_channel_tiles(m, OC):
    """Enough pixels that the 128- and 256-channel tiles are chosen (the second 256-channel
    tile of OC = 320 is three quarters empty)."""
    rng = np.random.default_rng(OC)
    x = rng.standard_normal((8, 32, 56, 56)).astype(np.float32)
    w = (rng.standard_normal((OC, 32, 3, 3)) / np.sqrt(32 * 9)).astype(np.float32)
    b = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    # 8 million outputs, half of them zeroed by the ReLU (which halves the rms): the largest
    # operand-rounding error among so many lies further out, hence the wider floor
    _check_conv(m, x, w, b, pad=(1, 1, 1, 1), relu=True, floor32=2e-1)


def test_conv_gather_modes_agree(m):
    """Channel counts that are multiples of 32 are served either by the direct gather or by the
    shared-memory staged one; both feed the tensor core the same operands in the same order, so
    the results are bit-identical."""
    import os
    rng = np.random.default_rng(21)
    cases = [((4, 64, 14, 14), (96, 64, 3, 3), dict(pad=(1, 1, 1, 1))),
             ((2, 32, 17, 13), (40, 32, 3, 2), dict(stride=(2, 1), pad=(1, 0, 2, 1), dilation=(1, 2))),
             ((3, 96, 9, 9), (64, 96, 1, 1), dict())]
    for xs, ws, kw in cases:
        x = rng.standard_normal(xs).astype(np.float32)
        w = (rng.standard_normal(ws) / np.sqrt(np.prod(ws[1:]))).astype(np.float32)
        b = (0.1 * rng.standard_normal(ws[0])).astype(np.float32)
        staged = _check_conv(m, x, w, b, **kw)
        os.environ["MDC_CONV_DIRECT"] = "1"
        try:
            direct = m.conv2d(x, w, b, **kw)
        finally:
            del os.environ["MDC_CONV_DIRECT"]
        assert np.array_equal(staged, direct)


def test_conv_exact_on_small_integers(m):
    """Integer-valued operands are exact in fp16 and every partial sum is exact in fp32, so the
    result must equal the oracle bit for bit: this isolates the gather / scatter indexing."""
    rng = np.random.default_rng(7)
    x = rng.integers(-4, 5, size=(2, 5, 13, 11)).astype(np.float32)
    w = rng.integers(-3, 4, size=(12, 5, 3, 3)).astype(np.float32)
    b = rng.integers(-8, 9, size=12).astype(np.float32)
    add = rng.integers(-8, 9, size=(2, 12, 7, 6)).astype(np.float32)
    got = m.conv2d(x, w, b, post_add=add, stride=(2, 2), pad=(1, 1, 1, 1), relu=True)
    ref = oracle.conv2d(x, w, b, post_add=add, stride=(2, 2), pad=(1, 1, 1, 1), relu=True)
    assert np.array_equal(got, ref)


def test_conv_reference_test_layer_full_size(m):
    """test/End2End/GPU/conv.mlir: 16x3x256x256 -> 16x64x256x256, 3x3, padding 1."""
    rng = np.random.default_rng(11)
    # multiples of 1/64: exact in fp16 and far from its subnormal range, so doubling commutes
    # with the rounding
    x = (np.round(rng.standard_normal((16, 3, 256, 256)) * 64) / 64).astype(np.float32)
    w = (rng.standard_normal((64, 3, 3, 3)) * 0.1).astype(np.float32)
    b = (0.1 * rng.standard_normal(64)).astype(np.float32)
    got = m.conv2d(x, w, b, pad=(1, 1, 1, 1))
    ref = oracle.conv2d(x, w, b, pad=(1, 1, 1, 1), round_mode=oracle.ROUND_F16)
    assert got.shape == (16, 64, 256, 256)
    assert np.max(np.abs(got - ref)) <= 1e-4
    # linearity in the input at full size: conv(2x) - bias = 2 (conv(x) - bias), exactly
    got2 = m.conv2d(2 * x, w, np.zeros_like(b), pad=(1, 1, 1, 1))
    got1 = m.conv2d(x, w, np.zeros_like(b), pad=(1, 1, 1, 1))
    assert np.array_equal(got2, 2 * got1)


def test_reference_pool_fixtures(m, golden_cnn):
    g = golden_cnn
    assert np.array_equal(m.pool2d(g["maxpool_x"], (4, 4), (4, 4)), g["maxpool_y"])
    assert np.array_equal(m.pool2d(g["pool_x"], (3, 3), (2, 2), pad=(1, 1, 1, 1), method=0), g["pool_max_y"])
    avg = m.pool2d(g["pool_x"], (3, 3), (2, 2), pad=(1, 1, 1, 1), method=1)
    assert np.max(np.abs(avg - g["pool_avg_y"])) <= 1e-6


@pytest.mark.parametrize("case", [
    # N, C, H, W, kernel, stride, pad
    (1, 1, 4, 4, (2, 2), (2, 2), (0, 0, 0, 0)),
    (2, 3, 17, 19, (3, 3), (2, 2), (1, 1, 1, 1)),
    (3, 5, 16, 12, (2, 3), (1, 2), (0, 1, 1, 2)),
    (2, 64, 56, 56, (3, 3), (2, 2), (1, 1, 1, 1)),
    (1, 2, 9, 9, (9, 9), (1, 1), (0, 0, 0, 0)),     # global pooling
    (16, 3, 256, 256, (4, 4), (4, 4), (0, 0, 0, 0)),  # test/End2End/GPU/pool.mlir
])
@pytest.mark.parametrize("method", [0, 1])
def test_pool_against_oracle(m, case, method):
    N, C, H, W, kernel, stride, pad = case
    rng = np.random.default_rng(hash(case[:4]) % (1 << 31))
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    got = m.pool2d(x, kernel, stride, pad=pad, method=method)
    ref = oracle.pool2d(x, kernel, stride, pad=pad, method=method)
    assert got.shape == ref.shape
    if method == 0:
        assert np.array_equal(got, ref)
    else:
        assert np.max(np.abs(got - ref)) <= 1e-6 * max(1.0, kernel[0] * kernel[1] / 9)


def test_pool_special_values(m):
    x = np.zeros((1, 1, 4, 4), np.float32)
    x[0, 0, 0, 0] = -np.inf
    x[0, 0, 2, 2] = np.inf
    x[0, 0, 1, 3] = -0.0
    got = m.pool2d(x, (2, 2), (2, 2), method=0)
    ref = oracle.pool2d(x, (2, 2), (2, 2), method=0)
    assert np.array_equal(got, ref)


def test_bad_geometry_is_reported(m):
    x = np.zeros((1, 1, 4, 4), np.float32)
    rt, ops = m.runtime(), m.ops()
    buf = m.to_device(x)
    out = m.DeviceBuffer(64)
    rt.mgpuClearLastError()
    ops.mgpuPool2d(buf.ptr, out.ptr, 1, 1, 4, 4, 3, 3, 2, 2, 0, 0, 0, 0, 2, 2, 0, None)  # OH too large
    assert rt.mgpuGetLastError() != 0
    rt.mgpuClearLastError()
