"""ONNX -> lowered-graph generator (graphgen/): the protobuf reader / writer, the emitted call
sequence and that every generated module compiles, links against the two libraries and
exports the model entry point.  No GPU needed: nothing is executed."""
import ctypes
import os

import numpy as np
import pytest

import graph_models as gm

ow, o2g = gm.load_graphgen()


@pytest.fixture(scope="module", autouse=True)
def built(mdc):
    mdc.build()


def test_wire_roundtrip_attributes_and_tensors():
    rng = np.random.default_rng(0)
    n = ow.Node("Conv", ["x", "w", ""], ["y"], {"pads": [1, 0, 1, 2], "axis": -1, "epsilon": 1e-5, "auto_pad": "NOTSET",
                                                "scales": [0.5, 2.0], "value": np.arange(6, dtype=np.int64).reshape(2, 3)},
                name="n0", domain="mdc")
    inits = {"w": rng.standard_normal((4, 3, 3, 3)).astype(np.float32), "shape": np.array([0, -1], dtype=np.int64),
             "i32": np.array([[1, -2], [3, 4]], dtype=np.int32)}
    g = ow.Graph([n], [ow.ValueInfo("x", [2, 3, 8, 8]), ow.ValueInfo("dyn", [None, 4])], [ow.ValueInfo("y", [2, 4, 8, 7])], inits)
    m = ow.load(ow.dumps(ow.Model(g, opsets={"": 18, "mdc": 1})))
    n2 = m.graph.nodes[0]
    assert (n2.op_type, n2.inputs, n2.outputs, n2.name, n2.domain) == ("Conv", ["x", "w", ""], ["y"], "n0", "mdc")
    assert n2.attrs["pads"] == [1, 0, 1, 2] and n2.attrs["axis"] == -1 and n2.attrs["auto_pad"] == "NOTSET"
    assert abs(n2.attrs["epsilon"] - 1e-5) < 1e-12 and n2.attrs["scales"] == [0.5, 2.0]
    assert np.array_equal(n2.attrs["value"], np.arange(6).reshape(2, 3))
    assert m.opsets == {"": 18, "mdc": 1}
    assert [(v.name, v.shape) for v in m.graph.inputs] == [("x", [2, 3, 8, 8]), ("dyn", [None, 4])]
    for k, a in inits.items():
        assert m.graph.initializers[k].dtype == a.dtype and np.array_equal(m.graph.initializers[k], a)


def test_typed_tensor_storage_is_read():
    # float_data / int64_data instead of raw_data, as some exporters write small tensors
    import struct
    t = ow._vi(1, 3) + ow._vi(2, ow.FLOAT) + ow._ld(4, struct.pack("<3f", 1.5, -2.0, 3.25)) + ow._ld(8, b"t")
    name, arr = ow._tensor(t)
    assert name == "t" and np.array_equal(arr, np.array([1.5, -2.0, 3.25], np.float32))
    t = ow._vi(1, 2) + ow._vi(2, ow.INT64) + ow._ld(7, ow._enc_varint(7) + ow._enc_varint(-1)) + ow._ld(8, b"s")
    assert np.array_equal(ow._tensor(t)[1], np.array([7, -1]))


def _calls(src):
    return [ln.strip().split("(")[0] for ln in src.splitlines() if ln.strip().startswith("mgpu")]


def test_emitted_sequence_for_linear(tmp_path):
    rng = np.random.default_rng(1)
    model, w, b = gm.linear_relu_model(ow, rng)
    src, weights = o2g.emit_cpp(model, "w.bin")
    # MatMul + Add(bias) became one mgpuMatmul; the weight is embedded as [K,N]; bias follows
    ops = [c for c in _calls(src) if c in ("mgpuMatmul", "mgpuAdd", "mgpuBiasAdd", "mgpuActivation")]
    assert ops == ["mgpuMatmul", "mgpuActivation"]
    assert src.index("GraphStreams st;") < src.index("st.data_to_kernel();") < src.index("mgpuMatmul(") < \
        src.index("st.kernel_to_data();") < src.index("mgpuMemcpy(host_out") < src.index("st.end();")
    assert src.count("mgpuRegisterConstant(") == 2
    wt = np.frombuffer(weights[:w.size * 4], np.float32).reshape(32, 64)
    assert np.array_equal(wt, w.T)
    # the Gemm(transB=1) form embeds the same transposed weight
    model2, w2, _ = gm.linear_relu_model(ow, np.random.default_rng(1), batch=(6,), as_gemm=True)
    _, weights2 = o2g.emit_cpp(model2, "w.bin")
    assert np.array_equal(np.frombuffer(weights2[:w2.size * 4], np.float32).reshape(32, 64), w2.T)


def test_conv_chain_is_fused():
    model, _ = gm.cnn_model(ow, np.random.default_rng(2))
    src, _ = o2g.emit_cpp(model, "w.bin")
    ops = [c for c in _calls(src) if c in ("mgpuConv2d", "mgpuAdd", "mgpuActivation", "mgpuPool2d")]
    assert ops == ["mgpuConv2d", "mgpuConv2d", "mgpuPool2d", "mgpuPool2d"]
    convs = [ln for ln in src.splitlines() if "mgpuConv2d(" in ln]
    assert convs[0].rstrip().endswith("false, true, st.kernel);")   # conv + relu
    assert convs[1].rstrip().endswith("true, true, st.kernel);")    # conv + residual + relu


def test_unsupported_models_are_rejected():
    m = gm._model(ow, [ow.Node("Softmax", ["x"], ["y"])], [("x", (2, 4))], [("y", (2, 4))], {})
    with pytest.raises(o2g.Unsupported, match="Softmax"):
        o2g.emit_cpp(m, "w.bin")
    m = gm._model(ow, [ow.Node("Add", ["x", "b"], ["y"])], [("x", (2, 4))], [("y", (2, 4))], {"b": np.zeros((2, 1), np.float32)})
    with pytest.raises(o2g.Unsupported, match="Add"):
        o2g.emit_cpp(m, "w.bin")
    m = gm._model(ow, [ow.Node("Conv", ["x", "w"], ["y"], {"group": 2, "kernel_shape": [1, 1]})], [("x", (1, 4, 4, 4))],
                  [("y", (1, 4, 4, 4))], {"w": np.zeros((4, 2, 1, 1), np.float32)})
    with pytest.raises(o2g.Unsupported, match="group"):
        o2g.emit_cpp(m, "w.bin")


@pytest.mark.parametrize("which", ["add", "add_constant", "gemm_inputs", "linear", "layernorm", "cnn", "encoder"])
def test_generated_module_compiles_and_exports_the_entry_point(tmp_path, which):
    rng = np.random.default_rng(3)
    model = {"add": lambda: gm.add_model(ow), "add_constant": lambda: gm.add_constant_model(ow, rng)[0],
             "gemm_inputs": lambda: gm.gemm_inputs_model(ow), "linear": lambda: gm.linear_relu_model(ow, rng)[0],
             "layernorm": lambda: gm.layernorm_model(ow, rng)[0], "cnn": lambda: gm.cnn_model(ow, rng)[0],
             "encoder": lambda: gm.encoder_model(ow, rng)[0]}[which]()
    path = str(tmp_path / f"{which}.onnx")
    ow.save(model, path)
    so = str(tmp_path / f"graph_{which}.so")
    o2g.build(path, so, keep_cpp=str(tmp_path))
    lib = ctypes.CDLL(so)
    assert hasattr(lib, "_mlir_ciface_main_graph")
    assert os.path.getsize(str(tmp_path / f"graph_{which}.weights.bin")) >= 0
