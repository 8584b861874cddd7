"""Small ONNX models (built with the package's own protobuf writer) shared by the graph
generator tests: the reference's example graphs (examples/genonnx.py:10-64), the layers of its
End2End tests (test/End2End/GPU/{linear,conv,pool}.mlir) at reduced size, and an encoder layer."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GRAPHGEN = os.path.join(ROOT, "multi-device-model-compiler_b200", "graphgen")


def load_graphgen():
    import importlib.util
    import sys
    if GRAPHGEN not in sys.path:
        sys.path.insert(0, GRAPHGEN)
    out = []
    for name in ("onnx_wire", "onnx2graph"):
        if name in sys.modules:
            out.append(sys.modules[name])
            continue
        spec = importlib.util.spec_from_file_location(name, os.path.join(GRAPHGEN, name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        out.append(mod)
    return out


def _model(ow, nodes, inputs, outputs, inits, opsets=None):
    g = ow.Graph(nodes, [ow.ValueInfo(n, list(s)) for n, s in inputs], [ow.ValueInfo(n, list(s)) for n, s in outputs],
                 {k: np.ascontiguousarray(v) for k, v in inits.items()})
    return ow.Model(g, opsets=opsets or {"": 18})


def add_model(ow, shape=(3, 64, 64)):
    return _model(ow, [ow.Node("Add", ["A", "B"], ["C"])], [("A", shape), ("B", shape)], [("C", shape)], {})


def add_constant_model(ow, rng, shape=(3, 32, 32)):
    b = rng.uniform(0, 1, shape).astype(np.float32)
    return _model(ow, [ow.Node("Add", ["A", "B"], ["C"])], [("A", shape)], [("C", shape)], {"B": b}), b


def gemm_inputs_model(ow):
    """examples/genonnx.py:52-64: Gemm of two run-time inputs, no bias."""
    return _model(ow, [ow.Node("Gemm", ["A", "B"], ["C"])], [("A", (20, 10)), ("B", (10, 20))], [("C", (20, 20))], {})


def linear_relu_model(ow, rng, batch=(3, 32), K=32, N=64, as_gemm=False):
    """y = relu(x W^T + b): torch.nn.Linear exported either as Gemm(transB=1) on a 2-D input or as
    MatMul + Add on a higher-rank one (the shape of test/End2End/GPU/linear.mlir)."""
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)   # torch layout [out, in]
    b = (0.1 * rng.standard_normal(N)).astype(np.float32)
    if as_gemm:
        nodes = [ow.Node("Gemm", ["x", "W", "b"], ["h"], {"transB": 1, "alpha": 1.0, "beta": 1.0}), ow.Node("Relu", ["h"], ["y"])]
        inits = {"W": w, "b": b}
    else:
        nodes = [ow.Node("MatMul", ["x", "Wt"], ["h0"]), ow.Node("Add", ["b", "h0"], ["h"]), ow.Node("Relu", ["h"], ["y"])]
        inits = {"Wt": np.ascontiguousarray(w.T), "b": b}
    shape_in, shape_out = tuple(batch) + (K,), tuple(batch) + (N,)
    return _model(ow, nodes, [("x", shape_in)], [("y", shape_out)], inits), w, b


def layernorm_model(ow, rng, shape=(4, 16, 48)):
    g = (1 + 0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
    b = (0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
    n = ow.Node("LayerNormalization", ["x", "gamma", "beta"], ["y"], {"axis": -1, "epsilon": 1e-5})
    return _model(ow, [n], [("x", shape)], [("y", shape)], {"gamma": g, "beta": b}), g, b


def cnn_model(ow, rng, N=2, C=3, H=20, W=24, OC=16):
    """conv3x3(pad 1) + relu -> conv3x3 + residual add + relu -> maxpool 2x2 -> global average pool -> flatten"""
    w1 = (rng.standard_normal((OC, C, 3, 3)) / np.sqrt(C * 9)).astype(np.float32)
    b1 = (0.1 * rng.standard_normal(OC)).astype(np.float32)
    w2 = (rng.standard_normal((OC, OC, 3, 3)) / np.sqrt(OC * 9)).astype(np.float32)
    conv = dict(kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1], dilations=[1, 1], group=1)
    nodes = [ow.Node("Conv", ["x", "w1", "b1"], ["c1"], dict(conv)), ow.Node("Relu", ["c1"], ["r1"]),
             ow.Node("Conv", ["r1", "w2"], ["c2"], dict(conv)), ow.Node("Add", ["c2", "r1"], ["s"]), ow.Node("Relu", ["s"], ["r2"]),
             ow.Node("MaxPool", ["r2"], ["p"], dict(kernel_shape=[2, 2], strides=[2, 2])),
             ow.Node("GlobalAveragePool", ["p"], ["gap"]), ow.Node("Flatten", ["gap"], ["y"], {"axis": 1})]
    return _model(ow, nodes, [("x", (N, C, H, W))], [("y", (N, OC))], {"w1": w1, "b1": b1, "w2": w2}), (w1, b1, w2)


ENC_KEYS = ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2", "ln1_g", "ln1_b", "ln2_g", "ln2_b")


def encoder_model(ow, rng, B=4, S=32, D=128, F=256, heads=2, with_lens=True):
    w = {"wqkv": 0.05 * rng.standard_normal((D, 3 * D)), "bqkv": 0.02 * rng.standard_normal(3 * D),
         "wo": 0.05 * rng.standard_normal((D, D)), "bo": 0.02 * rng.standard_normal(D),
         "w1": 0.05 * rng.standard_normal((D, F)), "b1": 0.02 * rng.standard_normal(F),
         "w2": 0.05 * rng.standard_normal((F, D)), "b2": 0.02 * rng.standard_normal(D),
         "ln1_g": 1 + 0.1 * rng.standard_normal(D), "ln1_b": 0.1 * rng.standard_normal(D),
         "ln2_g": 1 + 0.1 * rng.standard_normal(D), "ln2_b": 0.1 * rng.standard_normal(D)}
    w = {k: v.astype(np.float32) for k, v in w.items()}
    ins = ["x"] + list(ENC_KEYS) + (["lens"] if with_lens else [])
    n = ow.Node("TransformerEncoderLayer", ins, ["y"], {"num_heads": heads, "norm_first": 0, "causal": 0,
                                                        "activation": "gelu", "epsilon": 1e-5, "dtype": "f16"}, domain="mdc")
    inputs = [("x", (B, S, D))] + ([("lens", (B,))] if with_lens else [])
    return _model(ow, [n], inputs, [("y", (B, S, D))], w, opsets={"": 18, "mdc": 1}), w
