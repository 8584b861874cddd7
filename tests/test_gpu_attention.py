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
from parity_report import report

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def m(mdc):
    mdc.init()
    return mdc


def _case(m, B, S, H, lens, causal, dt, seed=0, D=64, name=None, capsys=None):
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
    if name:
        rows = np.concatenate([np.arange(b * S, b * S + (S if lens is None else int(lens[b]))) for b in range(B)])
        report(name, ref.reshape(B * S, -1)[rows], got.reshape(B * S, -1)[rows], capsys)
    return got, ref


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [128, 384, 12, 200, 256, 640])
def test_full_length(m, S, D):
    _case(m, 2, S, 3, None, False, m.F16, D=D)


@pytest.mark.parametrize("D", [64, 128])
def test_padding_masks(m, D):
    lens = np.array([384, 192, 200, 383, 129, 256, 1, 300], np.int32)
    _case(m, 8, 384, 2, lens, False, m.F16, seed=1, D=D)


def test_many_items_per_cta(m):
    # more work items than persistent CTAs: every CTA walks several items, of unequal length
    rng = np.random.default_rng(11)
    B, S, H = 40, 256, 12
    lens = rng.integers(0, S + 1, B).astype(np.int32)
    _case(m, B, S, H, lens, False, m.F16, seed=12)
    _case(m, 24, 384, 16, rng.integers(1, 385, 24).astype(np.int32), True, m.F16, seed=13, D=128)


def test_rows_of_the_next_sequence_are_never_read(m):
    # sequence length not a multiple of the tile: the tile rows past a sequence's end belong to
    # the next sequence in memory; poison them (NaN) and check that nothing leaks
    B, S, H, D = 3, 200, 2, 64
    rng = np.random.default_rng(14)
    qkv = oracle.round_array(rng.standard_normal((B * S, 3, H, D)).astype(np.float32), oracle.ROUND_F16)
    ref = oracle.attention(qkv, None, B, S, H, D, round_mode=oracle.ROUND_F16).reshape(B, S, H * D)
    poisoned = qkv.reshape(B, S, 3, H, D).copy()
    poisoned[1] = np.nan
    got = m.attention(poisoned.reshape(B * S, 3, H, D), None, B, S, H, D).reshape(B, S, H * D)
    for b in (0, 2):
        assert np.all(np.isfinite(got[b]))
        assert oracle.max_rel_err(ref[b], got[b], floor_frac=1.0) <= TOL


def test_zero_length_sequence_gives_zeros(m):
    lens = np.array([5, 0], np.int32)
    got, _ = _case(m, 2, 128, 1, lens, False, m.F16, seed=2)
    assert np.all(got[1] == 0)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S", [128, 384, 77])
def test_causal(m, S, D):
    _case(m, 2, S, 2, None, True, m.F16, seed=3, D=D)
    _case(m, 2, S, 2, np.array([S, max(1, S // 2)], np.int32), True, m.F16, seed=4, D=D)


@pytest.mark.parametrize("D", [64, 128])
def test_bf16(m, D):
    _case(m, 2, 256, 2, np.array([256, 130], np.int32), False, m.BF16, seed=5, D=D)


def test_config_shapes(m, capsys):
    # encoder-layer config at its full size: batch 32, 12 heads x 64, S = 384, lengths uniform
    # in [192, 384]; the stack config: 12 heads x 64, S = 128, 64 of its 256 sequences
    rng = np.random.default_rng(6)
    lens = rng.integers(192, 385, 32).astype(np.int32)
    _case(m, 32, 384, 12, lens, False, m.F16, seed=6, name="attention B=32 S=384 12x64 (padding), fp16", capsys=capsys)
    _case(m, 64, 128, 12, None, False, m.F16, seed=7, name="attention B=64 S=128 12x64, fp16", capsys=capsys)
    # the reference layer's own head geometry: 8 heads x 128, causal (lib/Kernels/GPU/LLM.cu:18-19)
    _case(m, 8, 256, 8, None, True, m.F16, seed=9, D=128, name="attention B=8 S=256 8x128 causal, fp16", capsys=capsys)


@pytest.mark.parametrize("D", [64, 128])
def test_large_scores_do_not_overflow(m, D):
    B, S, H = 1, 128, 1
    rng = np.random.default_rng(8)
    qkv = rng.standard_normal((B * S, 3, H, D)).astype(np.float32)
    qkv[:, 0] *= 30.0  # scores of several hundred: exp() must be taken relative to the row max
    qkv = oracle.round_array(qkv, oracle.ROUND_F16)
    got = m.attention(qkv, None, B, S, H, D)
    ref = oracle.attention(qkv, None, B, S, H, D, round_mode=oracle.ROUND_F16)
    assert np.all(np.isfinite(got))
    assert oracle.max_rel_err(ref, got, floor_frac=1.0) <= TOL
