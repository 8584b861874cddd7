"""multi-device-gpu-runner: command line, memref plumbing, raw fp32 files, batch sharding
over worker processes and host-side failure detection (CPU graphs, no GPU needed); and the
same configs through the GPU graphs (-m gpu)."""
import os
import subprocess

import numpy as np
import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "multi-device-model-compiler_b200")
RUNNER = os.path.join(PKG, "bin", "multi-device-gpu-runner")
ORACLE_DIR = os.path.join(ROOT, "oracle")


@pytest.fixture(scope="module", autouse=True)
def built(mdc):
    if not os.path.exists(RUNNER):
        mdc.build()
    oracle.build()


def run(args, **kw):
    return subprocess.run([RUNNER] + args, capture_output=True, text=True, timeout=600, **kw)


def files(tmp_path, arrays):
    names = []
    for i, a in enumerate(arrays):
        p = str(tmp_path / f"in{i}.dat")
        np.ascontiguousarray(a, dtype=np.float32).tofile(p)  # raw little-endian fp32, examples/data_util.py:52-54
        names.append(p)
    return ",".join(names)


def shape(a):
    return "_".join(str(s) for s in a.shape)


# ------------------------------------------------------------------ CPU graphs
def test_cpu_add_graph_roundtrip(tmp_path):
    rng = np.random.default_rng(0)
    a, b = rng.uniform(-1, 1, (3, 64, 64)).astype(np.float32), rng.uniform(-1, 1, (3, 64, 64)).astype(np.float32)
    out = str(tmp_path / "out.dat")
    r = run([os.path.join(ORACLE_DIR, "libcpu_graph_add.so"), "--device", "cpu", "--input", f"{shape(a)},{shape(b)}",
             "--output", shape(a), "--data", files(tmp_path, [a, b]), "--out-data", out, "--rerun", "2"])
    assert r.returncode == 0, r.stderr
    assert "Average time" in r.stdout
    assert np.array_equal(np.fromfile(out, np.float32).reshape(a.shape), a + b)


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_batch_sharding_matches_single_process(tmp_path, world):
    # N worker processes each take a contiguous slice of dimension 0; the gathered file must
    # equal the single-process result (the multi-GPU path of the runner, minus the GPU)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 5, 48)).astype(np.float32)
    g, b = rng.standard_normal(48).astype(np.float32), rng.standard_normal(48).astype(np.float32)
    lib = os.path.join(ORACLE_DIR, "libcpu_graph_layernorm.so")
    common = ["--device", "cpu", "--input", f"{shape(x)},48,48", "--output", shape(x), "--data", files(tmp_path, [x, g, b])]
    one, many = str(tmp_path / "one.dat"), str(tmp_path / "many.dat")
    assert run([lib] + common + ["--out-data", one]).returncode == 0
    r = run([lib] + common + ["--out-data", many, "--gpus", str(world), "--json"])
    assert r.returncode == 0, r.stderr
    assert np.array_equal(np.fromfile(one, np.float32), np.fromfile(many, np.float32))
    assert np.max(np.abs(np.fromfile(many, np.float32).reshape(x.shape) - oracle.layernorm(x, g, b))) <= 1e-6


def test_cpu_gemm_graph(tmp_path):
    rng = np.random.default_rng(2)
    a, w, b = (rng.standard_normal((20, 10)).astype(np.float32), rng.standard_normal((10, 20)).astype(np.float32),
               rng.standard_normal(20).astype(np.float32))
    out = str(tmp_path / "o.dat")
    r = run([os.path.join(ORACLE_DIR, "libcpu_graph_gemm.so"), "--device", "cpu", "--input", "20_10,10_20,20",
             "--output", "20_20", "--data", files(tmp_path, [a, w, b]), "--out-data", out])
    assert r.returncode == 0, r.stderr
    assert np.allclose(np.fromfile(out, np.float32).reshape(20, 20), a @ w + b, atol=1e-5)


def test_bad_arguments_are_rejected(tmp_path):
    lib = os.path.join(ORACLE_DIR, "libcpu_graph_add.so")
    assert run([]).returncode != 0                                          # <lib> is required
    assert run([lib, "--device", "cpu", "--input", "3_x_4"]).returncode != 0  # not a shape
    assert run([lib, "--device", "cpu", "--input", "2_2,2_2", "--output", "2_2", "--data", "only_one.dat"]).returncode != 0
    short = str(tmp_path / "short.dat")
    np.zeros(3, np.float32).tofile(short)                                   # truncated input file
    r = run([lib, "--device", "cpu", "--input", "2_2_2,2_2_2", "--output", "2_2_2", "--data", f"{short},{short}"])
    assert r.returncode != 0 and "Wrong File size" in r.stderr
    assert run([str(tmp_path / "missing.so"), "--device", "cpu"]).returncode != 0
    r = run([lib, "--device", "cpu", "--func", "no_such_symbol", "--input", "1_1_1,1_1_1", "--output", "1_1_1"])
    assert r.returncode != 0 and "Failed to find run function" in r.stderr


def test_failed_worker_is_detected_on_the_host(tmp_path):
    # fault injected on the host: worker 1's slice cannot be produced because the library
    # has no such entry point -> the parent must report the failure and exit non-zero
    lib = os.path.join(ORACLE_DIR, "libcpu_graph_add.so")
    r = run([lib, "--device", "cpu", "--gpus", "2", "--func", "nope", "--input", "4_2_2,4_2_2", "--output", "4_2_2"])
    assert r.returncode != 0
    assert "workers failed" in r.stderr


def test_hung_worker_hits_the_deadline(tmp_path):
    # a graph that never returns (host-side sleep): the parent kills it at the deadline
    src = tmp_path / "hang.c"
    src.write_text("#include <unistd.h>\nvoid _mlir_ciface_main_graph(void*a,void*b,void*c){ for(;;) sleep(1); }\n")
    lib = str(tmp_path / "libhang.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", lib, str(src)], check=True)
    r = run([lib, "--device", "cpu", "--gpus", "2", "--timeout", "2", "--input", "4_2_2,4_2_2", "--output", "4_2_2"])
    assert r.returncode != 0
    assert "deadline" in r.stderr


def test_without_a_gpu_the_gpu_path_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    r = run([os.path.join(PKG, "lib", "graph_add.so")])
    assert r.returncode != 0
    assert "failed" in r.stderr


# ------------------------------------------------------------------ GPU graphs
@pytest.mark.gpu
def test_gpu_add_graph_bit_exact(tmp_path):
    rng = np.random.default_rng(3)
    a, b = rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32), rng.uniform(-1, 1, (3, 640, 640)).astype(np.float32)
    out = str(tmp_path / "out.dat")
    r = run([os.path.join(PKG, "lib", "graph_add.so"), "--data", files(tmp_path, [a, b]), "--out-data", out, "--rerun", "3"])
    assert r.returncode == 0, r.stderr + r.stdout
    assert np.array_equal(np.fromfile(out, np.float32).reshape(a.shape), oracle.add(a, b))


@pytest.mark.gpu
def test_gpu_gemm_and_layernorm_graphs(tmp_path):
    rng = np.random.default_rng(4)
    a, w, b = (rng.standard_normal((256, 512)).astype(np.float32), (0.02 * rng.standard_normal((512, 384))).astype(np.float32),
               (0.02 * rng.standard_normal(384)).astype(np.float32))
    out = str(tmp_path / "g.dat")
    r = run([os.path.join(PKG, "lib", "graph_gemm.so"), "--input", "256_512,512_384,384", "--output", "256_384",
             "--data", files(tmp_path, [a, w, b]), "--out-data", out, "--rerun", "2"])
    assert r.returncode == 0, r.stderr + r.stdout
    ref = oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16)
    assert oracle.max_rel_err(ref, np.fromfile(out, np.float32).reshape(256, 384)) <= 2e-2
    x = rng.standard_normal((4, 64, 768)).astype(np.float32)
    g, be = (1 + 0.1 * rng.standard_normal(768)).astype(np.float32), (0.1 * rng.standard_normal(768)).astype(np.float32)
    out = str(tmp_path / "l.dat")
    r = run([os.path.join(PKG, "lib", "graph_layernorm.so"), "--input", "4_64_768,768,768", "--output", "4_64_768",
             "--data", files(tmp_path, [x, g, be]), "--out-data", out])
    assert r.returncode == 0, r.stderr + r.stdout
    assert np.max(np.abs(np.fromfile(out, np.float32).reshape(x.shape) - oracle.layernorm(x, g, be))) <= 1e-5


@pytest.mark.gpu
def test_gpu_encoder_graph_with_baked_weights(tmp_path):
    import ctypes
    lib_path = os.path.join(PKG, "lib", "graph_encoder.so")
    B, S, d, F = 4, 128, 768, 3072
    rng = np.random.default_rng(5)
    x = rng.standard_normal((B, S, d)).astype(np.float32)
    lens = np.array([128, 100, 128, 64], np.float32)
    out = str(tmp_path / "e.dat")
    r = run([lib_path, "--input", f"{B}_{S}_{d},{B}", "--output", f"{B}_{S}_{d}", "--data", files(tmp_path, [x, lens]),
             "--out-data", out, "--rerun", "2"], env=dict(os.environ, MDC_GRAPH_LAYERS="2"))
    assert r.returncode == 0, r.stderr + r.stdout
    got = np.fromfile(out, np.float32).reshape(B, S, d)
    # rebuild the constants the graph carries with the generator it exports
    g = ctypes.CDLL(lib_path)
    g.mdc_graph_weight_seed.restype = ctypes.c_uint64
    g.mdc_graph_weight_seed.argtypes = [ctypes.c_int64, ctypes.c_int64]
    g.mdc_graph_fill_normal.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float]
    layers = []
    for l in range(2):
        lw = {}
        for which, (name, shp) in enumerate((("wqkv", (d, 3 * d)), ("wo", (d, d)), ("w1", (d, F)), ("w2", (F, d)))):
            arr = np.empty(shp, np.float32)
            g.mdc_graph_fill_normal(arr.ctypes.data, arr.size, g.mdc_graph_weight_seed(l, which), 0.02)
            lw[name] = arr
        layers.append(lw)
    assert abs(float(np.std(layers[0]["w1"])) - 0.02) < 1e-3
    ref = oracle.encoder_stack(x, layers, lens.astype(np.int32), 12, round_mode=oracle.ROUND_F16)
    for b in range(B):
        n = int(lens[b])
        assert oracle.max_rel_err(ref[b, :n], got[b, :n], floor_frac=1.0) <= 2e-2


@pytest.mark.gpu
def test_gpu_batch_sharding_over_two_devices(tmp_path):
    # one worker process per GPU, each computing its rows of the batch; the gathered file
    # must equal the single-GPU result bit for bit (sequences do not interact)
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib_path = os.path.join(PKG, "lib", "graph_encoder.so")
    B, S, d = 8, 128, 768
    rng = np.random.default_rng(6)
    x = rng.standard_normal((B, S, d)).astype(np.float32)
    lens = np.full(B, S, np.float32)
    common = [lib_path, "--input", f"{B}_{S}_{d},{B}", "--output", f"{B}_{S}_{d}", "--data", files(tmp_path, [x, lens])]
    one, two = str(tmp_path / "one.dat"), str(tmp_path / "two.dat")
    r1 = run(common + ["--out-data", one])
    assert r1.returncode == 0, r1.stderr + r1.stdout
    r2 = run(common + ["--out-data", two, "--gpus", "2", "--rerun", "2", "--json"])
    assert r2.returncode == 0, r2.stderr + r2.stdout
    assert np.array_equal(np.fromfile(one, np.float32), np.fromfile(two, np.float32))


@pytest.mark.gpu
def test_gpu_gemm_config_with_constant_cache(tmp_path):
    # the Gemm config (A [2048,4096], W [4096,4096] passed as [K,N], bias [4096]) through the
    # runner; with --constants the weights are uploaded once and re-runs get faster, with the
    # same bytes out
    import json
    rng = np.random.default_rng(7)
    a = rng.standard_normal((2048, 4096)).astype(np.float32)
    w = (0.02 * rng.standard_normal((4096, 4096))).astype(np.float32)
    b = (0.02 * rng.standard_normal(4096)).astype(np.float32)
    common = [os.path.join(PKG, "lib", "graph_gemm.so"), "--input", "2048_4096,4096_4096,4096", "--output", "2048_4096",
              "--data", files(tmp_path, [a, w, b]), "--rerun", "5", "--json"]
    plain, cached = str(tmp_path / "p.dat"), str(tmp_path / "c.dat")
    r1 = run(common + ["--out-data", plain])
    r2 = run(common + ["--out-data", cached, "--constants"])
    assert r1.returncode == 0 and r2.returncode == 0, r1.stderr + r2.stderr
    assert np.array_equal(np.fromfile(plain, np.float32), np.fromfile(cached, np.float32))
    ref = oracle.matmul(a, w, b, round_mode=oracle.ROUND_F16)
    assert oracle.max_rel_err(ref, np.fromfile(cached, np.float32).reshape(2048, 4096)) <= 2e-2
    t1 = json.loads(r1.stdout.strip().splitlines()[-1])["avg_ms"]
    t2 = json.loads(r2.stdout.strip().splitlines()[-1])["avg_ms"]
    assert t2 < t1, (t1, t2)
