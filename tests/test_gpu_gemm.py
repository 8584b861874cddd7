"""GPU parity: the tcgen05 Gemm (mgpuMatmulEx16) and the reference entry point mgpuMatmul
against the CPU oracle.  Tolerance for 16-bit tensor-core math: max-rel <= 2e-2, where the
error of an element is divided by max(|ref|, 1e-2 * rms(ref))."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _rm(m, dt):
    return oracle.ROUND_F16 if dt == m.F16 else oracle.ROUND_BF16


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 64)])
def test_small_integers_are_exact(m, M, N, K):
    # products and sums of small integers are exact in fp16 x fp16 -> fp32, so any layout,
    # swizzle or descriptor mistake shows up as a hard mismatch
    rng = np.random.default_rng(0)
    a = rng.integers(-3, 4, (M, K)).astype(np.float32)
    w = rng.integers(-2, 3, (K, N)).astype(np.float32)
    got = m.matmul16(a, w, out_dtype=m.F32)
    assert np.array_equal(got, a @ w)


@pytest.mark.parametrize("M,N,K", [(37, 70, 129), (1, 8, 8), (130, 264, 72), (300, 40, 520), (129, 257, 65)])
@pytest.mark.parametrize("dtype_name", ["f16", "bf16"])
def test_ragged_shapes(m, M, N, K, dtype_name):
    dt = m.F16 if dtype_name == "f16" else m.BF16
    rng = np.random.default_rng(1)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.05 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.05 * rng.standard_normal(N)).astype(np.float32)
    got = m.matmul16(a, w, bias=b, dtype=dt, out_dtype=m.F32)
    ref = oracle.matmul(a, w, b, round_mode=_rm(m, dt))
    assert oracle.max_rel_err(ref, got) <= TOL


@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_epilogues(m, act):
    rng = np.random.default_rng(2)
    M, N, K = 200, 328, 192
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.1 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    r = rng.standard_normal((M, N)).astype(np.float32)
    got = m.matmul16(a, w, bias=b, residual=r, act=act)
    ref = oracle.matmul(a, w, b, residual=oracle.round_array(r, oracle.ROUND_F16), round_mode=oracle.ROUND_F16,
                        act=act, out_round=oracle.ROUND_F16)
    assert oracle.max_rel_err(ref, got) <= TOL


def test_layer_shapes(m):
    # the four Gemm shapes of one encoder layer at d=768, F=3072 (tokens reduced to 1024)
    rng = np.random.default_rng(3)
    T = 1024
    for K, N in ((768, 2304), (768, 768), (768, 3072), (3072, 768)):
        a = rng.standard_normal((T, K)).astype(np.float32)
        w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
        got = m.matmul16(a, w)
        ref = oracle.matmul(a, w, round_mode=oracle.ROUND_F16, out_round=oracle.ROUND_F16)
        assert oracle.max_rel_err(ref, got) <= TOL, (K, N)


def test_mgpu_matmul_config(m):
    # BASELINE config: A fp32 [2048,4096] N(0,1), W [4096,4096] N(0,0.02) passed as [K,N], bias N(0,0.02)
    rng = np.random.default_rng(4)
    a = rng.standard_normal((2048, 4096)).astype(np.float32)
    w = (0.02 * rng.standard_normal((4096, 4096))).astype(np.float32)
    b = (0.02 * rng.standard_normal(4096)).astype(np.float32)
    got = m.matmul(a, w, b)
    ref = oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16)
    assert oracle.max_rel_err(ref, got) <= TOL
    t = oracle.diff_table(ref, got)
    assert t["gt_0.1"] == 0


def test_mgpu_matmul_reference_fixtures(m, golden):
    # benchmark/PyTorch/Models/Linear.py in the shape of test/End2End/GPU/linear.mlir
    y = m.activation(m.matmul(golden["lin_x"], golden["lin_w"], golden["lin_b"]), m.ACT_RELU)
    assert y.shape == golden["lin_y"].shape
    ref16 = oracle.matmul(golden["lin_x"], golden["lin_w"], golden["lin_b"], round_mode=oracle.ROUND_F16,
                          act=oracle.ACT_RELU)
    assert oracle.max_rel_err(ref16, y) <= TOL
    # against the fp32 model output the fp16 operand rounding shows: elements near zero are
    # judged against 5 % of the rms (as in tests/test_oracle_golden.py)
    assert oracle.max_rel_err(golden["lin_y"], y, floor_frac=5e-2) <= TOL
    # examples/genonnx.py:52-64: Gemm 20x10 . 10x20 (K not a multiple of 8)
    rng = np.random.default_rng(5)
    a, w = rng.standard_normal((20, 10)).astype(np.float32), rng.standard_normal((10, 20)).astype(np.float32)
    got = m.matmul(a, w, None)
    assert oracle.max_rel_err(oracle.matmul(a, w, round_mode=oracle.ROUND_F16), got) <= TOL


def test_linearity_at_full_size(m):
    # size-independent property: Gemm(a1 + a2) == Gemm(a1) + Gemm(a2) when a1, a2 have
    # disjoint supports (exact in fp16), checked at the full config size without the oracle
    rng = np.random.default_rng(6)
    M, K, N = 2048, 4096, 4096
    a = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
    a1, a2 = a.copy(), a.copy()
    a1[:, K // 2:] = 0
    a2[:, :K // 2] = 0
    y = m.matmul16(a, w, out_dtype=m.F32)
    y12 = m.matmul16(a1, w, out_dtype=m.F32) + m.matmul16(a2, w, out_dtype=m.F32)
    # equal up to the order of the fp32 accumulation
    assert oracle.max_rel_err(y12, y) <= 5e-3
    assert np.max(np.abs(y12 - y)) <= 1e-4


@pytest.mark.parametrize("M,N,K", [(32768, 768, 64), (1024, 128, 64), (8192, 768, 192)])
def test_narrow_tiles_are_exact(m, M, N, K):
    # shapes for which the library picks 192- or 128-column tiles (fewer wasted tiles in the
    # last wave); small integers again, so the result must match exactly, with every epilogue
    # input in play (bias and residual are integers too)
    rng = np.random.default_rng(7)
    a = rng.integers(-3, 4, (M, K)).astype(np.float32)
    w = rng.integers(-2, 3, (K, N)).astype(np.float32)
    b = rng.integers(-4, 5, N).astype(np.float32)
    r = rng.integers(-8, 9, (M, N)).astype(np.float32)
    ref = a @ w + b + r
    assert np.array_equal(m.matmul16(a, w, bias=b, residual=r), ref)              # 16-bit output
    assert np.array_equal(m.matmul16(a, w, bias=b, residual=r, out_dtype=m.F32), ref)


@pytest.mark.parametrize("bn", ["192", "128"])
def test_forced_tile_width(bn):
    # every shape of this file again with the tile width forced (read once per process)
    import os
    import subprocess
    import sys
    env = dict(os.environ, MDC_GEMM_BN=bn)
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-m", "gpu", "-x",
                        "-k", "small_integers or ragged or epilogues or narrow"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
