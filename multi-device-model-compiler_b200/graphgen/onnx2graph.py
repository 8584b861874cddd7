#!/usr/bin/env python3
"""ONNX -> lowered-graph module for multi-device-gpu-runner, without MLIR.

The reference lowers an ONNX model through its MLIR pipeline (lib/Pipelines/MLIRToGPU.cpp:48-193)
into a shared library exporting `_mlir_ciface_main_graph(out*, in*...)` whose body is a
sequence of runtime / op-library calls.  This script produces the same kind of module for the
operator subset the op library serves, by emitting that call sequence as C++ and compiling
it with g++:

    Add (same shape, or a trailing-dimension bias), Relu, Gelu, Gemm, MatMul (+ bias Add),
    LayerNormalization, Conv (+ residual Add, + Relu), MaxPool, AveragePool,
    GlobalAveragePool, Flatten / Reshape / Identity (views), and the fused node
    `TransformerEncoderLayer` of domain "mdc" (the reference recognises the exported attention
    subgraph instead, lib/Conversion/ConvertONNXToDevice/MultiHeadAttentionLayer.cpp:133-172).

What the emitted module does per call, in the reference's order: two streams linked by events,
device allocation + upload of every input and constant, the op calls on the kernel stream,
download of the result, frees, stream teardown.  Initializers are embedded in the module's
read-only data (as the reference embeds constants in the model library) and declared to the
runtime with mgpuRegisterConstant, so after the first call their "upload" is a
device-to-device copy.  Gemm weights stored [N,K] (transB = 1) are transposed at generation
time, as lib/Conversion/ConvertTosaToDevice/Matmul.cpp:57-70 does.  The leading dimension of
the first input is read from its descriptor at run time, so one module serves any batch size
(and the runner's --gpus batch sharding).

Usage:  onnx2graph.py model.onnx -o graph_model.so [--keep-cpp DIR]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import onnx_wire as ow  # noqa: E402

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REPO = os.path.dirname(PKG)


class Unsupported(Exception):
    pass


class Val:
    """A tensor of the graph: shape[0] scales with the run-time batch when `batched`."""

    def __init__(self, name, shape, batched, kind):
        self.name, self.shape, self.batched, self.kind = name, list(shape), batched, kind
        self.alias = None       # a view of another Val (Reshape / Flatten / Identity)
        self.var = None         # C++ identifier of the device pointer
        self.const_off = None   # byte offset inside the embedded weights
        self.input_index = None

    def root(self):
        v = self
        while v.alias is not None:
            v = v.alias
        return v

    def inner(self):
        """elements per batch entry (batched) or in total (not batched)"""
        n = 1
        for d in (self.shape[1:] if self.batched else self.shape):
            n *= d
        return n

    def count_expr(self):
        return f"(B * {self.inner()}LL)" if self.batched else f"{self.inner()}LL"


class Lowering:
    def __init__(self, model: ow.Model):
        self.g = model.graph
        self.vals = {}
        self.steps = []          # C++ statements on the kernel stream
        self.weights = bytearray()
        self.consts = []         # Vals backed by embedded data
        self.temps = []          # Vals needing a device allocation
        self.consumers = {}
        self.fused = set()       # ids of nodes folded into an earlier one
        for n in self.g.nodes:
            for i in n.inputs:
                if i:
                    self.consumers.setdefault(i, []).append(n)
        if len(self.g.outputs) != 1:
            raise Unsupported("exactly one graph output is supported (the runner saves output 0)")
        if not self.g.inputs:
            raise Unsupported("the graph has no run-time input")
        for k, vi in enumerate(self.g.inputs):
            if vi.elem_type != ow.FLOAT or any(d is None or d <= 0 for d in vi.shape) or not 1 <= len(vi.shape) <= 4:
                raise Unsupported(f"input {vi.name!r}: static fp32 shapes of rank 1-4 only")
            v = Val(vi.name, vi.shape, False, "input")
            v.input_index = k
            self.vals[vi.name] = v
        self.batch = self.g.inputs[0].shape[0]
        # inputs shaped like input 0 share its run-time batch (an elementwise partner)
        for vi in self.g.inputs:
            if list(vi.shape) == list(self.g.inputs[0].shape):
                self.vals[vi.name].batched = True
        for name, arr in self.g.initializers.items():
            self.vals[name] = Val(name, arr.shape, False, "const")

    # ---------------------------------------------------------------- helpers
    def val(self, name):
        if name not in self.vals:
            raise Unsupported(f"tensor {name!r} is used before it is produced")
        return self.vals[name]

    def const_array(self, name):
        if name not in self.g.initializers:
            raise Unsupported(f"{name!r} must be an initializer")
        return self.g.initializers[name]

    def embed(self, v: Val, arr: np.ndarray):
        """Place fp32 data in the embedded weights (256-byte aligned) and mark v as a device constant."""
        root = v.root()
        if root.const_off is None:
            while len(self.weights) % 256:
                self.weights.append(0)
            root.const_off = len(self.weights)
            data = np.ascontiguousarray(arr, dtype="<f4")
            root.nbytes = data.nbytes
            self.weights += data.tobytes()
            self.consts.append(root)
        return root

    def device(self, name):
        """C++ expression of the device pointer of tensor `name` (uploading constants on demand)."""
        v = self.val(name).root()
        if v.kind == "const":
            self.embed(v, self.const_array(v.name))
        return v.var_name()

    def new(self, name, shape, batched):
        v = Val(name, shape, batched, "temp")
        self.vals[name] = v
        self.temps.append(v)
        return v

    def sole_consumer(self, name, op_types):
        users = self.consumers.get(name, [])
        if len(users) == 1 and users[0].op_type in op_types and name != self.g.outputs[0].name:
            return users[0]
        return None

    # ---------------------------------------------------------------- operators
    def lower(self):
        for n in self.g.nodes:
            if id(n) in self.fused:
                continue
            fn = getattr(self, "op_" + n.op_type, None)
            if fn is None or (n.domain not in ("", "ai.onnx", "mdc")):
                raise Unsupported(f"operator {n.domain or 'ai.onnx'}.{n.op_type} is outside the supported subset")
            fn(n)
        out = self.val(self.g.outputs[0].name)
        if out.root().kind != "temp":
            raise Unsupported("the graph output must be computed by an operator")
        return out

    def op_Identity(self, n):
        self.view(n, self.val(n.inputs[0]).shape)

    def view(self, n, shape):
        src = self.val(n.inputs[0])
        v = Val(n.outputs[0], shape, src.batched, "view")
        v.alias = src
        if int(np.prod(shape)) != int(np.prod(src.shape)):
            raise Unsupported(f"{n.op_type}: element count changes")
        if src.batched and shape[0] != src.shape[0]:
            raise Unsupported(f"{n.op_type}: the batch dimension must stay in front")
        self.vals[n.outputs[0]] = v

    def op_Flatten(self, n):
        src = self.val(n.inputs[0])
        axis = n.attrs.get("axis", 1)
        axis += len(src.shape) if axis < 0 else 0
        self.view(n, [int(np.prod(src.shape[:axis])), int(np.prod(src.shape[axis:]))])

    def op_Reshape(self, n):
        src = self.val(n.inputs[0])
        shape = [int(x) for x in self.const_array(n.inputs[1]).ravel()]
        shape = [src.shape[i] if d == 0 else d for i, d in enumerate(shape)]
        if -1 in shape:
            known = int(np.prod([d for d in shape if d != -1]))
            shape[shape.index(-1)] = int(np.prod(src.shape)) // max(known, 1)
        self.view(n, shape)

    def op_Add(self, n):
        a, b = self.val(n.inputs[0]), self.val(n.inputs[1])
        if b.kind != "const" and a.kind == "const":
            a, b = b, a
            n = ow.Node("Add", [n.inputs[1], n.inputs[0]], n.outputs, n.attrs)
        out = self.new(n.outputs[0], a.shape, a.batched or b.batched)
        if list(a.shape) == list(b.shape) and (a.batched == b.batched or b.kind == "const"):
            if b.root().kind == "const" and a.batched:
                # a constant of the full (compile-time) shape only matches at that batch size
                self.steps.append(f'  if (B != {self.batch}) {{ mgpuSetLastError(-1, "{n.outputs[0]}: constant operand fixes the batch at {self.batch}"); }}')
            self.steps.append(f"  mgpuAdd({self.device(n.inputs[0])}, {self.device(n.inputs[1])}, {out.var_name()}, {out.count_expr()}, st.kernel);")
        elif len(b.shape) == 1 and b.shape[0] == a.shape[-1] and not b.batched:
            cols = a.shape[-1]
            self.steps.append(f"  mgpuBiasAdd({self.device(n.inputs[0])}, {self.device(n.inputs[1])}, {out.var_name()}, {out.count_expr()} / {cols}, {cols}, st.kernel);")
        else:
            raise Unsupported(f"Add: shapes {a.shape} and {b.shape} (only equal shapes or a trailing-dimension bias)")

    def activation(self, n, act):
        a = self.val(n.inputs[0])
        out = self.new(n.outputs[0], a.shape, a.batched)
        self.steps.append(f"  mgpuActivation({self.device(n.inputs[0])}, {out.var_name()}, {out.count_expr()}, {act}, st.kernel);")

    def op_Relu(self, n):
        self.activation(n, "MGPU_ACT_RELU")

    def op_Gelu(self, n):
        approx = n.attrs.get("approximate", "none")
        self.activation(n, "MGPU_ACT_GELU_TANH" if approx == "tanh" else "MGPU_ACT_GELU_ERF")

    def matmul(self, n, a_name, w_name, bias_name, trans_b):
        a, w = self.val(a_name), self.val(w_name)
        if len(w.shape) != 2:
            raise Unsupported(f"{n.op_type}: the second operand must be a matrix")
        K = a.shape[-1]
        if w.root().kind == "const":
            arr = self.const_array(w.root().name)
            if trans_b:
                arr = arr.T  # stored [N,K]: hand the op its [K,N] layout
            if arr.shape[0] != K:
                raise Unsupported(f"{n.op_type}: inner dimensions {K} and {arr.shape[0]} differ")
            N = arr.shape[1]
            wv = Val(w.name + ("__kn" if trans_b else ""), arr.shape, False, "const")
            self.embed(wv, arr)
            w_expr = wv.var_name()
        else:
            if trans_b:
                raise Unsupported("Gemm: transB = 1 needs a constant weight")
            w.root().batched = False  # a weight that arrives as an input is always passed whole
            if w.shape[0] != K:
                raise Unsupported(f"{n.op_type}: inner dimensions {K} and {w.shape[0]} differ")
            N = w.shape[1]
            w_expr = self.device(w_name)
        bias_expr = "nullptr"
        if bias_name:
            b = self.val(bias_name)
            if int(np.prod(b.shape)) != N:
                raise Unsupported(f"{n.op_type}: bias of {b.shape} for {N} columns")
            bias_expr = self.device(bias_name)
        out_name = n.outputs[0]
        out = self.new(out_name, a.shape[:-1] + [N], a.batched)
        self.steps.append(f"  mgpuMatmul(mut({self.device(a_name)}), mut({w_expr}), "
                          f"mut({bias_expr}), {out.var_name()}, {a.count_expr()} / {K}, {N}, {K}, st.kernel);")
        return out

    def op_Gemm(self, n):
        if n.attrs.get("transA", 0) or n.attrs.get("alpha", 1.0) != 1.0 or n.attrs.get("beta", 1.0) != 1.0:
            raise Unsupported("Gemm: transA, alpha and beta must be at their defaults")
        self.matmul(n, n.inputs[0], n.inputs[1], n.inputs[2] if len(n.inputs) > 2 and n.inputs[2] else None,
                    bool(n.attrs.get("transB", 0)))

    def op_MatMul(self, n):
        # MatMul followed by Add of a constant vector is one device.matmul with bias
        nxt = self.sole_consumer(n.outputs[0], ("Add",))
        bias = None
        if nxt is not None:
            other = [i for i in nxt.inputs if i != n.outputs[0]]
            if len(other) == 1 and other[0] in self.g.initializers and self.g.initializers[other[0]].ndim == 1:
                bias = other[0]
                self.fused.add(id(nxt))
                n = ow.Node("MatMul", n.inputs, nxt.outputs, n.attrs)
        self.matmul(n, n.inputs[0], n.inputs[1], bias, False)

    def op_LayerNormalization(self, n):
        a = self.val(n.inputs[0])
        axis = n.attrs.get("axis", -1)
        if axis not in (-1, len(a.shape) - 1):
            raise Unsupported("LayerNormalization: only the last axis")
        cols = a.shape[-1]
        gamma = self.device(n.inputs[1]) if len(n.inputs) > 1 and n.inputs[1] else "nullptr"
        beta = self.device(n.inputs[2]) if len(n.inputs) > 2 and n.inputs[2] else "nullptr"
        eps = float(n.attrs.get("epsilon", 1e-5))
        out = self.new(n.outputs[0], a.shape, a.batched)
        self.steps.append(f"  mgpuLayerNormF32({self.device(n.inputs[0])}, {gamma}, {beta}, {out.var_name()}, {eps!r}f, "
                          f"{a.count_expr()} / {cols}, {cols}, st.kernel);")

    @staticmethod
    def conv_geometry(n, x_shape, k_shape, dilations):
        if n.attrs.get("auto_pad", "NOTSET") != "NOTSET":
            raise Unsupported(f"{n.op_type}: auto_pad")
        if n.attrs.get("ceil_mode", 0):
            raise Unsupported(f"{n.op_type}: ceil_mode")
        strides = n.attrs.get("strides", [1, 1])
        pads = n.attrs.get("pads", [0, 0, 0, 0])  # top, left, bottom, right
        H, W = x_shape[2], x_shape[3]
        OH = (H + pads[0] + pads[2] - (k_shape[0] - 1) * dilations[0] - 1) // strides[0] + 1
        OW = (W + pads[1] + pads[3] - (k_shape[1] - 1) * dilations[1] - 1) // strides[1] + 1
        return strides, pads, OH, OW

    def op_Conv(self, n):
        x = self.val(n.inputs[0])
        w = self.const_array(n.inputs[1])
        if len(x.shape) != 4 or w.ndim != 4 or n.attrs.get("group", 1) != 1 or w.shape[1] != x.shape[1]:
            raise Unsupported("Conv: 2-D, group 1 only")
        dil = n.attrs.get("dilations", [1, 1])
        strides, pads, OH, OW = self.conv_geometry(n, x.shape, w.shape[2:], dil)
        OC, IC, KH, KW = w.shape
        if len(n.inputs) > 2 and n.inputs[2]:
            bias = self.device(n.inputs[2])
        else:
            zb = Val(n.outputs[0] + "__zero_bias", [OC], False, "const")
            self.embed(zb, np.zeros(OC, np.float32))
            bias = zb.var_name()
        # Conv -> [Add residual] -> [Relu] is one device.conv2d (hasPostAdd / hasContainRelu)
        cur, post, relu = n, None, False
        nxt = self.sole_consumer(cur.outputs[0], ("Add",))
        if nxt is not None:
            other = [i for i in nxt.inputs if i != cur.outputs[0]]
            if len(other) == 1 and list(self.val(other[0]).shape) == [x.shape[0], OC, OH, OW] and \
                    self.val(other[0]).root().kind != "const":
                post, cur = other[0], nxt
                self.fused.add(id(nxt))
        nxt = self.sole_consumer(cur.outputs[0], ("Relu",))
        if nxt is not None:
            relu, cur = True, nxt
            self.fused.add(id(nxt))
        out = self.new(cur.outputs[0], [x.shape[0], OC, OH, OW], x.batched)
        nb = "B" if x.batched else str(x.shape[0])
        self.steps.append(
            f"  mgpuConv2d(mut({self.device(n.inputs[0])}), mut({self.device(n.inputs[1])}), "
            f"mut({bias}), {out.var_name()}, {('mut(' + self.device(post) + ')') if post else 'nullptr'}, "
            f"{nb}, {IC}, {x.shape[2]}, {x.shape[3]}, {OC}, {KH}, {KW}, {OH}, {OW}, {pads[0]}, {pads[1]}, {pads[2]}, {pads[3]}, "
            f"{strides[0]}, {strides[1]}, {dil[0]}, {dil[1]}, {'true' if post else 'false'}, {'true' if relu else 'false'}, st.kernel);")

    def pool(self, n, method, kernel=None):
        x = self.val(n.inputs[0])
        if len(x.shape) != 4:
            raise Unsupported(f"{n.op_type}: NCHW input only")
        if kernel is None:
            kernel = n.attrs.get("kernel_shape")
            if n.attrs.get("dilations", [1, 1]) != [1, 1]:
                raise Unsupported(f"{n.op_type}: dilations")
            if method == 1 and not n.attrs.get("count_include_pad", 0) and any(n.attrs.get("pads", [0, 0, 0, 0])):
                raise Unsupported("AveragePool: padded windows need count_include_pad = 1")
            if "strides" not in n.attrs:
                n.attrs["strides"] = [1, 1]
            strides, pads, OH, OW = self.conv_geometry(n, x.shape, kernel, [1, 1])
        else:
            strides, pads, OH, OW = [1, 1], [0, 0, 0, 0], 1, 1
        out = self.new(n.outputs[0], [x.shape[0], x.shape[1], OH, OW], x.batched)
        nb = "B" if x.batched else str(x.shape[0])
        self.steps.append(
            f"  mgpuPool2d(mut({self.device(n.inputs[0])}), {out.var_name()}, {nb}, {x.shape[1]}, {x.shape[2]}, {x.shape[3]}, "
            f"{OH}, {OW}, {kernel[0]}, {kernel[1]}, {pads[0]}, {pads[1]}, {pads[2]}, {pads[3]}, {strides[0]}, {strides[1]}, {method}, st.kernel);")

    def op_MaxPool(self, n):
        if len(n.outputs) > 1 and n.outputs[1]:
            raise Unsupported("MaxPool: the indices output")
        self.pool(n, 0)

    def op_AveragePool(self, n):
        self.pool(n, 1)

    def op_GlobalAveragePool(self, n):
        x = self.val(n.inputs[0])
        self.pool(n, 1, kernel=[x.shape[2], x.shape[3]])

    def op_TransformerEncoderLayer(self, n):
        """domain "mdc": inputs x [B,S,D], wqkv [D,3D], bqkv, wo [D,D], bo, w1 [D,F], b1, w2 [F,D], b2,
        ln1_gamma, ln1_beta, ln2_gamma, ln2_beta, then optionally seq_lens [B] (fp32 valid lengths).
        attributes: num_heads, norm_first (0), causal (0), activation ("gelu" | "gelu_tanh" | "relu"),
        epsilon (1e-5), dtype ("f16" | "bf16")."""
        if n.domain != "mdc":
            raise Unsupported("TransformerEncoderLayer belongs to domain 'mdc'")
        x = self.val(n.inputs[0])
        if len(x.shape) != 3 or len(n.inputs) < 13:
            raise Unsupported("TransformerEncoderLayer: x [B,S,D] and 12 parameter tensors")
        Bc, S, D = x.shape
        F = self.val(n.inputs[5]).shape[1]
        heads = int(n.attrs["num_heads"])
        act = {"gelu": "MGPU_ACT_GELU_ERF", "gelu_tanh": "MGPU_ACT_GELU_TANH", "relu": "MGPU_ACT_RELU"}[n.attrs.get("activation", "gelu")]
        dtype = {"f16": "MGPU_DTYPE_F16", "bf16": "MGPU_DTYPE_BF16"}[n.attrs.get("dtype", "f16")]
        params = [self.device(i) if i else "nullptr" for i in n.inputs[1:13]]
        lens = "nullptr"
        if len(n.inputs) > 13 and n.inputs[13]:
            lv = self.val(n.inputs[13]).root()
            if lv.kind != "input":
                raise Unsupported("TransformerEncoderLayer: seq_lens must be a graph input")
            lens = f"lens_i32_{lv.input_index}"
            lv.as_lengths = True
        out = self.new(n.outputs[0], x.shape, x.batched)
        nb = "B" if x.batched else str(Bc)
        self.steps.append(
            f"  mgpuTransformerEncoderLayer({self.device(n.inputs[0])}, {', '.join(params)}, {lens}, {out.var_name()}, "
            f"{nb}, {S}, {D}, {F}, {heads}, {'true' if n.attrs.get('norm_first', 0) else 'false'}, "
            f"{'true' if n.attrs.get('causal', 0) else 'false'}, {act}, {dtype}, {float(n.attrs.get('epsilon', 1e-5))!r}f, st.kernel);")


_var_counter = [0]


def _var_name(self):
    r = self.root()
    if r.var is None:
        safe = "".join(c if c.isalnum() else "_" for c in r.name)[:40]
        r.var = f"d{_var_counter[0]}_{r.kind[0]}_{safe}"
        _var_counter[0] += 1
    return r.var


Val.var_name = _var_name


def emit_cpp(model: ow.Model, weights_path: str, func: str = "main_graph"):
    """Returns (C++ source, weights bytes)."""
    _var_counter[0] = 0
    lo = Lowering(model)
    out = lo.lower()
    g = lo.g
    inputs = [lo.vals[vi.name] for vi in g.inputs]
    L = []
    L.append("// Generated by graphgen/onnx2graph.py: the call sequence of a lowered graph (see graph_common.h).")
    L.append('#include "graph_common.h"')
    L.append("")
    L.append("// the reference's entry points take non-const pointers")
    L.append("static inline float *mut(const float *p) { return const_cast<float *>(p); }")
    L.append("")
    if lo.weights:
        L.append('__asm__(".section .rodata\\n.balign 256\\n.hidden mdc_weights_begin\\n.global mdc_weights_begin\\n"')
        L.append(f'        "mdc_weights_begin:\\n.incbin \\"{weights_path}\\"\\n.previous\\n");')
        L.append('extern "C" __attribute__((visibility("hidden"))) const unsigned char mdc_weights_begin[];')
        L.append("static const float *weight_at(size_t offset) { return reinterpret_cast<const float *>(mdc_weights_begin + offset); }")
        L.append("")
    args = ", ".join([f"MemRef<{len(out.shape)}> *out"] + [f"MemRef<{len(v.shape)}> *in{v.input_index}" for v in inputs])
    L.append(f"MDC_GRAPH_EXPORT void _mlir_ciface_{func}({args}) {{")
    L.append("  const int64_t B = in0->sizes[0];  // run-time batch: the leading dimension of input 0")
    for v in inputs[1:]:
        if v.shape and v.shape[0] == lo.batch and getattr(v, "as_lengths", False):
            v.batched = True
    # result descriptor
    dims = ", ".join(("static_cast<intptr_t>(B)" if (i == 0 and out.batched) else str(d)) for i, d in enumerate(out.shape))
    L.append(f"  const intptr_t out_sizes[{len(out.shape)}] = {{{dims}}};")
    L.append(f"  float *host_out = alloc_result<{len(out.shape)}>(out, out_sizes);")
    if lo.consts:
        L.append("  static bool constants_registered = false;")
        L.append("  if (!constants_registered) {  // embedded weights never change: later uploads are device-to-device")
        for c in lo.consts:
            L.append(f"    mgpuRegisterConstant(mut(weight_at({c.const_off})), {c.nbytes});")
        L.append("    constants_registered = true;")
        L.append("  }")
    L.append("  GraphStreams st;")
    frees = []
    for v in inputs:
        k = v.input_index
        if getattr(v, "as_lengths", False):
            # valid lengths arrive as fp32 (the runner only reads fp32 files): int32 on the device
            L.append(f"  int32_t *lens_host_{k} = static_cast<int32_t *>(malloc(sizeof(int32_t) * (B > 0 ? B : 1)));")
            L.append(f"  for (int64_t i = 0; i < B; ++i) lens_host_{k}[i] = static_cast<int32_t>(in{k}->data()[i]);")
            L.append(f"  int32_t *lens_i32_{k} = static_cast<int32_t *>(mgpuMemAlloc(sizeof(int32_t) * (B > 0 ? B : 1), st.data));")
            L.append(f"  mgpuMemcpy(lens_i32_{k}, lens_host_{k}, sizeof(int32_t) * B, st.data);")
            frees.append(f"lens_i32_{k}")
            continue
        if v.var is None:
            continue  # unused input
        L.append(f"  float *{v.var} = upload(in{k}->data(), {v.count_expr()}, st.data);")
        frees.append(v.var)
    for c in lo.consts:
        L.append(f"  float *{c.var_name()} = upload(weight_at({c.const_off}), {c.nbytes // 4}, st.data);")
        frees.append(c.var)
    for t in lo.temps:
        L.append(f"  float *{t.var_name()} = static_cast<float *>(mgpuMemAlloc(static_cast<uint64_t>({t.count_expr()}) * 4, st.data));")
        frees.append(t.var)
    L.append("  st.data_to_kernel();")
    L += lo.steps
    L.append("  st.kernel_to_data();")
    L.append(f"  mgpuMemcpy(host_out, {out.var_name()}, static_cast<size_t>({out.count_expr()}) * 4, st.data);")
    for f in frees:
        L.append(f"  mgpuMemFree({f}, st.data);")
    L.append("  st.end();")
    for v in inputs:
        if getattr(v, "as_lengths", False):
            L.append(f"  free(lens_host_{v.input_index});")
    L.append("}")
    return "\n".join(L) + "\n", bytes(lo.weights)


def build(onnx_path, out_so, keep_cpp=None, func="main_graph", cxx=None):
    """Generate and compile; returns the path of the C++ source that was compiled."""
    model = ow.load(onnx_path)
    work = keep_cpp or tempfile.mkdtemp(prefix="mdc_graphgen_")
    os.makedirs(work, exist_ok=True)
    base = os.path.splitext(os.path.basename(out_so))[0]
    wpath = os.path.abspath(os.path.join(work, base + ".weights.bin"))
    src, weights = emit_cpp(model, wpath, func)
    with open(wpath, "wb") as f:
        f.write(weights)
    cpp = os.path.join(work, base + ".cpp")
    with open(cpp, "w") as f:
        f.write(src)
    cxx = cxx or os.environ.get("CXX", "g++")
    libdir = os.path.join(PKG, "lib")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", f"-I{os.path.join(REPO, 'include')}",
           f"-I{os.path.join(PKG, 'csrc', 'graphs')}", "-o", out_so, cpp, f"-L{libdir}", "-lMultiDeviceGPUOps",
           "-lMultiDeviceCUDARuntime", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compiling the generated graph failed:\n" + r.stderr)
    return cpp


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("onnx")
    ap.add_argument("-o", "--output", required=True, help="the graph module (.so) to write")
    ap.add_argument("--keep-cpp", default=None, help="directory for the generated .cpp and weights file")
    ap.add_argument("--func", default="main_graph")
    a = ap.parse_args()
    try:
        cpp = build(a.onnx, a.output, a.keep_cpp, a.func)
    except Unsupported as e:
        print(f"onnx2graph: unsupported model: {e}", file=sys.stderr)
        return 2
    print(f"wrote {a.output} (source: {cpp})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
