"""The CPU oracle must reproduce the fixtures made from the reference's PyTorch models
(tests/golden/make_golden.py) before anything is compared against it."""
import numpy as np

import oracle

W_KEYS = ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2", "ln1_g", "ln1_b", "ln2_g", "ln2_b")


def _weights(g, prefix):
    return {k: g[prefix + k] for k in W_KEYS}


def test_reference_decoder_layer_fp32(golden):
    # benchmark/PyTorch/Models/LLM.py: pre-LN, causal mask, ReLU
    y = oracle.encoder_layer(golden["dec_x"], _weights(golden, "dec_"), None, int(golden["dec_heads"]),
                             norm_first=True, causal=True, act=oracle.ACT_RELU,
                             round_mode=oracle.ROUND_NONE)
    assert np.max(np.abs(y - golden["dec_y"])) <= 2e-5


def test_reference_decoder_layer_fp16_storage_within_tolerance(golden):
    y = oracle.encoder_layer(golden["dec_x"], _weights(golden, "dec_"), None, int(golden["dec_heads"]),
                             norm_first=True, causal=True, act=oracle.ACT_RELU,
                             round_mode=oracle.ROUND_F16)
    # fp16 storage against the fp32 model: elements near zero are judged against 5 % of the rms
    assert oracle.max_rel_err(golden["dec_y"], y, floor_frac=5e-2) <= 2e-2


def test_reference_linear_relu(golden):
    # benchmark/PyTorch/Models/Linear.py; shape of test/End2End/GPU/linear.mlir
    y = oracle.matmul(golden["lin_x"], golden["lin_w"], golden["lin_b"], act=oracle.ACT_RELU)
    assert y.shape == golden["lin_y"].shape
    assert np.max(np.abs(y - golden["lin_y"])) <= 1e-5
    y64 = oracle.matmul(golden["lin_x"], golden["lin_w"], golden["lin_b"], act=oracle.ACT_RELU,
                        accum64=True)
    assert np.max(np.abs(y64 - golden["lin_y"])) <= 1e-5


def test_crosscheck_postln_gelu_padding(golden):
    lens = golden["enc_lens"]
    y = oracle.encoder_layer(golden["enc_x"], _weights(golden, "enc_"), lens, int(golden["enc_heads"]),
                             norm_first=False, causal=False, act=oracle.ACT_GELU_ERF,
                             round_mode=oracle.ROUND_NONE)
    ref = golden["enc_y"]
    for b, n in enumerate(lens):  # padded query rows are excluded from parity
        assert np.max(np.abs(y[b, :n] - ref[b, :n])) <= 2e-5
    assert np.all(np.isfinite(y))


def test_crosscheck_layernorm(golden):
    y = oracle.layernorm(golden["ln_x"], golden["ln_g"], golden["ln_b"], eps=1e-5)
    assert np.max(np.abs(y - golden["ln_y"])) <= 1e-5


def test_add_is_ieee_fp32():
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32)
    b = rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32)
    assert np.array_equal(oracle.add(a, b), a + b)


def test_matmul_fast_path_matches_double_accumulate():
    rng = np.random.default_rng(1)
    M, K, N = 37, 129, 70  # ragged against the 4x32 micro-tile
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (0.02 * rng.standard_normal((K, N))).astype(np.float32)
    b = (0.02 * rng.standard_normal(N)).astype(np.float32)
    fast = oracle.matmul(a, w, b)
    slow = oracle.matmul(a, w, b, accum64=True)
    ref = (a.astype(np.float64) @ w.astype(np.float64) + b).astype(np.float32)
    assert np.max(np.abs(slow - ref)) <= 1e-6
    assert np.max(np.abs(fast - ref)) <= 1e-5


def test_rounding_modes():
    x = np.array([1.0, 1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -2.5], dtype=np.float32)
    assert np.array_equal(oracle.round_array(x, oracle.ROUND_F16), x.astype(np.float16).astype(np.float32))
    import torch
    bf = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(oracle.round_array(x, oracle.ROUND_BF16), bf)


def test_attention_masks():
    rng = np.random.default_rng(2)
    B, S, H, D = 2, 9, 2, 8
    qkv = rng.standard_normal((B * S, 3, H, D)).astype(np.float32)
    lens = np.array([9, 5], dtype=np.int32)
    out = oracle.attention(qkv, lens, B, S, H, D)
    # brute force in float64
    q = qkv[:, 0].reshape(B, S, H, D).astype(np.float64)
    k = qkv[:, 1].reshape(B, S, H, D).astype(np.float64)
    v = qkv[:, 2].reshape(B, S, H, D).astype(np.float64)
    for b in range(B):
        n = lens[b]
        s = np.einsum("ihd,jhd->hij", q[b], k[b, :n]) / np.sqrt(D)
        p = np.exp(s - s.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        o = np.einsum("hij,jhd->ihd", p, v[b, :n]).reshape(S, H * D)
        assert np.max(np.abs(out.reshape(B, S, H * D)[b] - o)) <= 1e-5
    # causal: first row attends only to itself
    outc = oracle.attention(qkv, lens, B, S, H, D, causal=True)
    assert np.allclose(outc.reshape(B, S, H, D)[0, 0], v[0, 0], atol=1e-6)


def test_reference_conv_layer(golden_cnn):
    # benchmark/PyTorch/Models/Conv.py: Conv2d(3, 64, 3, 1, 1), the layer of test/End2End/GPU/conv.mlir
    g = golden_cnn
    y = oracle.conv2d(g["conv_x"], g["conv_w"], g["conv_b"], pad=(1, 1, 1, 1))
    assert y.shape == g["conv_y"].shape
    assert np.max(np.abs(y - g["conv_y"])) <= 2e-5
    y64 = oracle.conv2d(g["conv_x"], g["conv_w"], g["conv_b"], pad=(1, 1, 1, 1), accum64=True)
    assert np.max(np.abs(y64 - g["conv_y"])) <= 2e-5


def test_reference_maxpool_layer(golden_cnn):
    # benchmark/PyTorch/Models/MaxPool.py: MaxPool2d(4), the layer of test/End2End/GPU/pool.mlir
    g = golden_cnn
    y = oracle.pool2d(g["maxpool_x"], (4, 4), (4, 4))
    assert np.array_equal(y, g["maxpool_y"])


def test_crosscheck_conv_variants(golden_cnn):
    g = golden_cnn
    y = oracle.conv2d(g["res_x"], g["res_w"], g["res_b"], post_add=g["res_add"], stride=(2, 2),
                      pad=(1, 1, 1, 1), relu=True)
    assert y.shape == g["res_y"].shape and np.max(np.abs(y - g["res_y"])) <= 2e-5
    y = oracle.conv2d(g["dil_x"], g["dil_w"], g["dil_b"], stride=(1, 2), dilation=(2, 3))
    assert y.shape == g["dil_y"].shape and np.max(np.abs(y - g["dil_y"])) <= 2e-5


def test_crosscheck_pool_variants(golden_cnn):
    g = golden_cnn
    y = oracle.pool2d(g["pool_x"], (3, 3), (2, 2), pad=(1, 1, 1, 1), method=0)
    assert np.array_equal(y, g["pool_max_y"])
    y = oracle.pool2d(g["pool_x"], (3, 3), (2, 2), pad=(1, 1, 1, 1), method=1)
    assert y.shape == g["pool_avg_y"].shape and np.max(np.abs(y - g["pool_avg_y"])) <= 1e-6
