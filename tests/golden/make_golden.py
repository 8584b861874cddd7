"""Generates tests/golden/reference_models.npz.

Run once, in a container that has the reference checkout:
    python tests/golden/make_golden.py /root/reference
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


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
