"""GPU parity: the tcgen05 fused attention kernel against the CPU oracle.

Tolerance: max-rel <= 2e-2 where an element's error is divided by max(|ref|, rms(ref)).
The floor is the rms (not a small fraction of it as for the Gemm) because the softmax
weights are stored in 16 bits before the second matrix product: every output carries an
absolute error of about 2^-11 (fp16) or 2^-8 (bf16) of the typical output magnitude however
small the output itself is; the oracle's own 16-bit path differs from its fp32 path by the
same amount, which `_case` checks as well."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _case(m, B, S, H, lens, causal, dt, seed=0):
    D = 64
    rm = oracle.ROUND_F16 if dt == m.F16 else oracle.ROUND_BF16
    rng = np.random.default_rng(seed)
    qkv = oracle.round_array(rng.standard_normal((B * S, 3, H, D)).astype(np.float32), rm)
    got = m.attention(qkv, lens, B, S, H, D, causal=causal, dtype=dt).reshape(B, S, H * D)
    ref = oracle.attention(qkv, lens, B, S, H, D, causal=causal, round_mode=rm).reshape(B, S, H * D)
    ref32 = oracle.attention(qkv, lens, B, S, H, D, causal=causal).reshape(B, S, H * D)
    assert np.all(np.isfinite(got))
    for b in range(B):  # padded query rows carry no meaning
        n = S if lens is None else int(lens[b])
        if n:
            assert oracle.max_rel_err(ref[b, :n], got[b, :n], floor_frac=1.0) <= TOL, (b, n)
            # no noisier than the oracle's own 16-bit path is against exact arithmetic
            noise = np.max(np.abs(ref[b, :n] - ref32[b, :n]))
            assert np.max(np.abs(got[b, :n] - ref32[b, :n])) <= 2.0 * noise + 1e-6, (b, n)
    return got, ref


@pytest.mark.parametrize("S", [128, 384, 12, 200, 256])
def test_full_length(m, S):
    _case(m, 2, S, 3, None, False, m.F16)


def test_padding_masks(m):
    lens = np.array([384, 192, 200, 383, 129, 256, 1, 300], np.int32)
    _case(m, 8, 384, 2, lens, False, m.F16, seed=1)


def test_zero_length_sequence_gives_zeros(m):
    lens = np.array([5, 0], np.int32)
    got, _ = _case(m, 2, 128, 1, lens, False, m.F16, seed=2)
    assert np.all(got[1] == 0)


@pytest.mark.parametrize("S", [128, 384, 77])
def test_causal(m, S):
    _case(m, 2, S, 2, None, True, m.F16, seed=3)
    _case(m, 2, S, 2, np.array([S, max(1, S // 2)], np.int32), True, m.F16, seed=4)


def test_bf16(m):
    _case(m, 2, 256, 2, np.array([256, 130], np.int32), False, m.BF16, seed=5)


def test_config_shapes(m):
    # encoder-layer config: 12 heads x 64, S = 384, lengths uniform in [192, 384]
    rng = np.random.default_rng(6)
    lens = rng.integers(192, 385, 4).astype(np.int32)
    _case(m, 4, 384, 12, lens, False, m.F16, seed=6)
    _case(m, 4, 128, 12, None, False, m.F16, seed=7)


def test_large_scores_do_not_overflow(m):
    D, B, S, H = 64, 1, 128, 1
    rng = np.random.default_rng(8)
    qkv = rng.standard_normal((B * S, 3, H, D)).astype(np.float32)
    qkv[:, 0] *= 30.0  # scores of several hundred: exp() must be taken relative to the row max
    qkv = oracle.round_array(qkv, oracle.ROUND_F16)
    got = m.attention(qkv, None, B, S, H, D)
    ref = oracle.attention(qkv, None, B, S, H, D, round_mode=oracle.ROUND_F16)
    assert np.all(np.isfinite(got))
    assert oracle.max_rel_err(ref, got, floor_frac=1.0) <= TOL
