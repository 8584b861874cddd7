"""Generated lowered graphs (graphgen/onnx2graph.py) executed by multi-device-gpu-runner on
the GPU and compared with the CPU oracle: the reference's example graphs
(examples/genonnx.py:10-64), the layers of its End2End tests and an encoder layer."""
import os
import subprocess

import numpy as np
import pytest

import graph_models as gm
import oracle

pytestmark = pytest.mark.gpu

ow, o2g = gm.load_graphgen()
RUNNER = os.path.join(gm.ROOT, "multi-device-model-compiler_b200", "bin", "multi-device-gpu-runner")


@pytest.fixture(scope="module", autouse=True)
def built(mdc):
    mdc.build()


def run_model(tmp_path, model, inputs, out_shape, extra=()):
    path = str(tmp_path / "m.onnx")
    ow.save(model, path)
    so = str(tmp_path / "graph_m.so")
    o2g.build(path, so, keep_cpp=str(tmp_path))
    names = []
    for i, a in enumerate(inputs):
        p = str(tmp_path / f"in{i}.dat")
        np.ascontiguousarray(a, dtype=np.float32).tofile(p)
        names.append(p)
    out = str(tmp_path / "out.dat")
    shp = lambda s: "_".join(str(d) for d in s)
    r = subprocess.run([RUNNER, so, "--input", ",".join(shp(a.shape) for a in inputs), "--output", shp(out_shape),
                        "--data", ",".join(names), "--out-data", out, "--rerun", "2"] + list(extra),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return np.fromfile(out, np.float32).reshape(out_shape)


def test_add_graphs(tmp_path):
    rng = np.random.default_rng(0)
    a, b = rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32), rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32)
    assert np.array_equal(run_model(tmp_path, gm.add_model(ow, a.shape), [a, b], a.shape), a + b)
    model, c = gm.add_constant_model(ow, rng)
    x = rng.uniform(-1, 1, c.shape).astype(np.float32)
    assert np.array_equal(run_model(tmp_path, model, [x], x.shape), x + c)


def test_gemm_of_two_inputs(tmp_path):
    rng = np.random.default_rng(1)
    a, w = rng.standard_normal((20, 10)).astype(np.float32), rng.standard_normal((10, 20)).astype(np.float32)
    got = run_model(tmp_path, gm.gemm_inputs_model(ow), [a, w], (20, 20))
    ref = oracle.matmul(a, w, None, round_mode=oracle.ROUND_F16)
    assert oracle.max_rel_err(ref, got, floor_frac=1e-2) <= 2e-2


@pytest.mark.parametrize("as_gemm", [False, True])
def test_linear_relu(tmp_path, as_gemm):
    rng = np.random.default_rng(2)
    batch = (96,) if as_gemm else (3, 32)
    model, w, b = gm.linear_relu_model(ow, rng, batch=batch, as_gemm=as_gemm)
    x = rng.standard_normal(batch + (32,)).astype(np.float32)
    got = run_model(tmp_path, model, [x], batch + (64,))
    ref = oracle.matmul(x, np.ascontiguousarray(w.T), b, act=oracle.ACT_RELU, round_mode=oracle.ROUND_F16).reshape(got.shape)
    assert oracle.max_rel_err(ref, got, floor_frac=1e-2) <= 2e-2


def test_layernorm(tmp_path):
    rng = np.random.default_rng(3)
    model, g, b = gm.layernorm_model(ow, rng, shape=(8, 64, 768))
    x = rng.standard_normal((8, 64, 768)).astype(np.float32)
    got = run_model(tmp_path, model, [x], x.shape)
    assert np.max(np.abs(got - oracle.layernorm(x, g, b))) <= 1e-5


def test_cnn(tmp_path):
    rng = np.random.default_rng(4)
    model, (w1, b1, w2) = gm.cnn_model(ow, rng, N=4)
    x = rng.standard_normal((4, 3, 20, 24)).astype(np.float32)
    got = run_model(tmp_path, model, [x], (4, 16))
    r1 = oracle.conv2d(x, w1, b1, pad=(1, 1, 1, 1), relu=True, round_mode=oracle.ROUND_F16)
    r2 = oracle.conv2d(r1, w2, None, post_add=r1, pad=(1, 1, 1, 1), relu=True, round_mode=oracle.ROUND_F16)
    p = oracle.pool2d(r2, (2, 2), (2, 2))
    ref = oracle.pool2d(p, (p.shape[2], p.shape[3]), (1, 1), method=1).reshape(4, 16)
    assert oracle.max_rel_err(ref, got, floor_frac=1e-2) <= 2e-2


@pytest.mark.parametrize("with_lens", [True, False])
def test_encoder_layer_node(tmp_path, with_lens):
    rng = np.random.default_rng(5)
    B, S, D, heads = 4, 32, 128, 2
    model, w = gm.encoder_model(ow, rng, B=B, S=S, D=D, F=256, heads=heads, with_lens=with_lens)
    x = rng.standard_normal((B, S, D)).astype(np.float32)
    lens = np.array([32, 17, 5, 28], np.int32)
    inputs = [x] + ([lens.astype(np.float32)] if with_lens else [])
    got = run_model(tmp_path, model, inputs, x.shape)
    ref = oracle.encoder_layer(x, w, lens if with_lens else None, heads, norm_first=False, causal=False,
                               act=oracle.ACT_GELU_ERF, round_mode=oracle.ROUND_F16)
    # 16-bit intermediates: errors are judged against the rms (see tests/test_gpu_encoder.py)
    if with_lens:
        valid = np.arange(S)[None, :] < lens[:, None]
        assert np.all(np.isfinite(got))
        assert oracle.max_rel_err(ref[valid], got[valid], floor_frac=1.0) <= 2e-2
    else:
        assert oracle.max_rel_err(ref, got, floor_frac=1.0) <= 2e-2


def test_generated_graph_serves_other_batch_sizes(tmp_path):
    """The batch is read from the descriptor: a module generated for 8 rows runs 5 and 16."""
    rng = np.random.default_rng(6)
    model, g, b = gm.layernorm_model(ow, rng, shape=(8, 16, 48))
    for rows in (5, 16):
        x = rng.standard_normal((rows, 16, 48)).astype(np.float32)
        got = run_model(tmp_path, model, [x], x.shape)
        assert np.max(np.abs(got - oracle.layernorm(x, g, b))) <= 1e-5


def test_generated_graph_sharded_over_two_devices(tmp_path):
    """The runner's --gpus 2 cuts input 0 along dimension 0 and gathers the rows of output 0: a
    generated module, which reads its batch from the descriptor, needs nothing special."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rng = np.random.default_rng(9)
    model, w, b = gm.linear_relu_model(ow, rng, batch=(64, 8), K=32, N=64)
    x = rng.standard_normal((64, 8, 32)).astype(np.float32)
    one = run_model(tmp_path, model, [x], (64, 8, 64))
    two = run_model(tmp_path, model, [x], (64, 8, 64), extra=["--gpus", "2"])
    assert np.array_equal(one, two)
