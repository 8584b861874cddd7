"""Generates tests/golden/reference_models.npz.

Run once, in a container that has the reference checkout:
    python tests/golden/make_golden.py <checkout of the reference project>
It imports the reference's own PyTorch model definitions
(benchmark/PyTorch/Models/LLM.py:5-21 `Decoder`, benchmark/PyTorch/Models/Linear.py:5-19
`Linear`), runs them in fp32 on seeded inputs and stores inputs, weights (transposed to the
row-major [in, out] layout the C ABI passes) and outputs.  The tests then require the CPU
oracle to reproduce those outputs; the fixture travels, the reference checkout does not.

A second group (`enc_*`) comes from torch.nn.TransformerEncoderLayer configured like the
encoder benchmark configs (post-LN, GELU, key-padding mask).  That module is not part of the
reference; it is an independent implementation used as a cross-check and is labelled so.
"""
import os
import sys

import numpy as np
import torch
from torch import nn


def layer_weights(enc: nn.TransformerEncoderLayer, prefix: str, out: dict):
    sa = enc.self_attn
    out[prefix + "wqkv"] = sa.in_proj_weight.detach().numpy().T.copy()
    out[prefix + "bqkv"] = sa.in_proj_bias.detach().numpy().copy()
    out[prefix + "wo"] = sa.out_proj.weight.detach().numpy().T.copy()
    out[prefix + "bo"] = sa.out_proj.bias.detach().numpy().copy()
    out[prefix + "w1"] = enc.linear1.weight.detach().numpy().T.copy()
    out[prefix + "b1"] = enc.linear1.bias.detach().numpy().copy()
    out[prefix + "w2"] = enc.linear2.weight.detach().numpy().T.copy()
    out[prefix + "b2"] = enc.linear2.bias.detach().numpy().copy()
    out[prefix + "ln1_g"] = enc.norm1.weight.detach().numpy().copy()
    out[prefix + "ln1_b"] = enc.norm1.bias.detach().numpy().copy()
    out[prefix + "ln2_g"] = enc.norm2.weight.detach().numpy().copy()
    out[prefix + "ln2_b"] = enc.norm2.bias.detach().numpy().copy()


def main(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "benchmark", "PyTorch"))
    from Models import LLM, Linear  # the reference's model files

    torch.manual_seed(20240229)
    torch.set_num_threads(1)
    out = {}

    # --- reference Decoder: pre-LN, causal, ReLU, dim_feedforward 2048 (torch default) ---
    d_model, heads, B, S = 64, 1, 2, 12  # head_dim 64: the GPU attention kernel can run it
    dec = LLM.Decoder(d_model, heads).eval()
    with torch.no_grad():
        # make LN affine and biases non-trivial so the fixture exercises them
        for p in (dec.encoder.norm1.weight, dec.encoder.norm2.weight):
            p.copy_(1.0 + 0.1 * torch.randn_like(p))
        for p in (dec.encoder.norm1.bias, dec.encoder.norm2.bias, dec.encoder.self_attn.in_proj_bias,
                  dec.encoder.self_attn.out_proj.bias):
            p.copy_(0.1 * torch.randn_like(p))
        x = torch.randn(B, S, d_model)
        y = dec(x)
    out["dec_x"] = x.numpy()
    out["dec_y"] = y.numpy()
    out["dec_heads"] = np.int64(heads)
    layer_weights(dec.encoder, "dec_", out)

    # --- reference Linear: y = relu(x W^T + b), the shape of test/End2End/GPU/linear.mlir ---
    lin = Linear.Linear(32, 64).eval()
    with torch.no_grad():
        x = torch.randn(3, 32, 32)
        y = lin(x)
    out["lin_x"] = x.numpy()
    out["lin_w"] = lin.linear.weight.detach().numpy().T.copy()
    out["lin_b"] = lin.linear.bias.detach().numpy().copy()
    out["lin_y"] = y.numpy()

    # --- cross-check (NOT reference code): post-LN, GELU(erf), key padding mask ---
    d_model, heads, B, S, F = 32, 4, 3, 10, 64
    enc = nn.TransformerEncoderLayer(d_model, heads, dim_feedforward=F, dropout=0.0,
                                     activation="gelu", batch_first=True, norm_first=False).eval()
    lens = np.array([10, 7, 4], dtype=np.int32)
    with torch.no_grad():
        for p in (enc.norm1.weight, enc.norm2.weight):
            p.copy_(1.0 + 0.1 * torch.randn_like(p))
        for p in (enc.norm1.bias, enc.norm2.bias, enc.self_attn.in_proj_bias):
            p.copy_(0.1 * torch.randn_like(p))
        x = torch.randn(B, S, d_model)
        pad = torch.arange(S)[None, :] >= torch.tensor(lens.astype(np.int64))[:, None]
        # the math path (no nested-tensor fast path) so padded rows stay defined
        h = x
        a, _ = enc.self_attn(h, h, h, key_padding_mask=pad, need_weights=False)
        h = enc.norm1(h + a)
        f = enc.linear2(torch.nn.functional.gelu(enc.linear1(h)))
        y = enc.norm2(h + f)
    out["enc_x"] = x.numpy()
    out["enc_y"] = y.numpy()
    out["enc_lens"] = lens
    out["enc_heads"] = np.int64(heads)
    layer_weights(enc, "enc_", out)

    # --- cross-check (NOT reference code): fp32 LayerNorm with affine ---
    ln = nn.LayerNorm(48, eps=1e-5)
    with torch.no_grad():
        ln.weight.copy_(1.0 + 0.1 * torch.randn(48))
        ln.bias.copy_(0.1 * torch.randn(48))
        x = torch.randn(5, 7, 48)
        y = ln(x)
    out["ln_x"], out["ln_g"], out["ln_b"], out["ln_y"] = (x.numpy(), ln.weight.detach().numpy().copy(),
                                                          ln.bias.detach().numpy().copy(), y.numpy())

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_models.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")
    cnn_fixtures()


def cnn_fixtures():
    """Conv2d / Pool2d fixtures -> reference_cnn.npz (own seed, so the file above never changes)."""
    from Models import Conv, MaxPool  # the reference's model files
    import torch.nn.functional as F

    torch.manual_seed(20240301)
    out = {}
    # --- reference Conv(3, 64): 3x3, stride 1, padding 1 (test/End2End/GPU/conv.mlir's layer) ---
    conv = Conv.Conv(3, 64).eval()
    with torch.no_grad():
        x = torch.randn(2, 3, 20, 24)
        y = conv(x)
    out["conv_x"], out["conv_y"] = x.numpy(), y.numpy()
    out["conv_w"] = conv.conv.weight.detach().numpy().copy()
    out["conv_b"] = conv.conv.bias.detach().numpy().copy()
    # --- reference MaxPool(): 4x4 window, stride 4 (test/End2End/GPU/pool.mlir's layer) ---
    with torch.no_grad():
        x = torch.randn(2, 3, 16, 24)
        y = MaxPool.MaxPool().eval()(x)
    out["maxpool_x"], out["maxpool_y"] = x.numpy(), y.numpy()
    # --- cross-checks (NOT reference code) ---
    with torch.no_grad():
        # residual block tail: relu(conv(x) + b + identity), stride 2, padding 1
        x, w, b = torch.randn(2, 8, 15, 17), 0.2 * torch.randn(16, 8, 3, 3), 0.1 * torch.randn(16)
        y0 = F.conv2d(x, w, b, stride=2, padding=1)
        add = torch.randn_like(y0)
        out["res_x"], out["res_w"], out["res_b"], out["res_add"] = x.numpy(), w.numpy(), b.numpy(), add.numpy()
        out["res_y"] = torch.relu(y0 + add).numpy()
        # dilation 2, rectangular filter, no padding
        x, w, b = torch.randn(1, 5, 14, 19), 0.2 * torch.randn(7, 5, 3, 2), 0.1 * torch.randn(7)
        out["dil_x"], out["dil_w"], out["dil_b"] = x.numpy(), w.numpy(), b.numpy()
        out["dil_y"] = F.conv2d(x, w, b, stride=(1, 2), dilation=(2, 3)).numpy()
        # pooling: the ResNet stem's 3x3 / stride 2 / padding 1 max pool, and an average pool
        # that counts its padding
        x = torch.randn(2, 4, 13, 18)
        out["pool_x"] = x.numpy()
        out["pool_max_y"] = F.max_pool2d(x, 3, 2, 1).numpy()
        out["pool_avg_y"] = F.avg_pool2d(x, 3, 2, 1, count_include_pad=True).numpy()
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cnn.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
