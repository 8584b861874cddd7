"""Minimal reader / writer of the ONNX protobuf wire format (no `onnx` package needed).

Only what the graph generator uses is decoded: ModelProto.graph, opset imports, nodes with
their attributes, initializers (float / int32 / int64 tensors, raw or typed storage) and the
value infos of graph inputs / outputs with static shapes.  Field numbers are those of the
published onnx.proto3 schema.  The writer exists so tests and examples can build small models.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

# TensorProto.DataType
FLOAT, INT32, INT64 = 1, 6, 7
_NP = {FLOAT: np.float32, INT32: np.int32, INT64: np.int64}
# AttributeProto.AttributeType
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_FLOATS, A_INTS, A_STRINGS = 1, 2, 3, 4, 6, 7, 8


# ------------------------------------------------------------------ wire primitives
def _varint(buf: bytes, pos: int):
    out = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        out |= (b & 0x7F) << shift
        if not b & 0x80:
            return out, pos
        shift += 7


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def fields(buf: bytes):
    """Yield (field number, wire type, value); value is int (varint), bytes (length-delimited,
    fixed32, fixed64)."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        no, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 1:
            v, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            v, pos = buf[pos:pos + ln], pos + ln
        elif wt == 5:
            v, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        yield no, wt, v


def _packed_varints(v: bytes):
    pos, out = 0, []
    while pos < len(v):
        x, pos = _varint(v, pos)
        out.append(_signed(x))
    return out


def _enc_varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(no: int, wt: int) -> bytes:
    return _enc_varint((no << 3) | wt)


def _ld(no: int, payload: bytes) -> bytes:
    return _key(no, 2) + _enc_varint(len(payload)) + payload


def _vi(no: int, v: int) -> bytes:
    return _key(no, 0) + _enc_varint(v)


# ------------------------------------------------------------------ data model
@dataclass
class Node:
    op_type: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)
    name: str = ""
    domain: str = ""


@dataclass
class ValueInfo:
    name: str
    shape: list          # ints; None for a symbolic / unknown dimension
    elem_type: int = FLOAT


@dataclass
class Graph:
    nodes: list
    inputs: list         # ValueInfo, initializers excluded
    outputs: list        # ValueInfo
    initializers: dict   # name -> np.ndarray
    name: str = "main_graph"


@dataclass
class Model:
    graph: Graph
    opsets: dict = field(default_factory=lambda: {"": 17})
    ir_version: int = 8
    producer: str = "mdc-graphgen"


# ------------------------------------------------------------------ reader
def _tensor(buf: bytes):
    dims, dtype, name, raw = [], FLOAT, "", None
    floats, i32, i64 = [], [], []
    for no, wt, v in fields(buf):
        if no == 1:
            dims += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif no == 2:
            dtype = v
        elif no == 4:
            floats += list(struct.unpack(f"<{len(v) // 4}f", v))
        elif no == 5:
            i32 += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif no == 7:
            i64 += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif no == 8:
            name = v.decode()
        elif no == 9:
            raw = v
        elif no in (13, 14) and (no == 13 or v):
            raise ValueError(f"tensor {name!r}: external data is not supported")
    if dtype not in _NP:
        raise ValueError(f"tensor {name!r}: unsupported data type {dtype}")
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(_NP[dtype]).newbyteorder("<")).astype(_NP[dtype])
    else:
        arr = np.array(floats if dtype == FLOAT else i32 if dtype == INT32 else i64, dtype=_NP[dtype])
    return name, arr.reshape(dims)


def _attribute(buf: bytes):
    name, atype = "", None
    f = i = s = t = None
    floats, ints, strings = [], [], []
    for no, wt, v in fields(buf):
        if no == 1:
            name = v.decode()
        elif no == 2:
            f = struct.unpack("<f", v)[0]
        elif no == 3:
            i = _signed(v)
        elif no == 4:
            s = v
        elif no == 5:
            t = _tensor(v)[1]
        elif no == 7:
            floats += list(struct.unpack(f"<{len(v) // 4}f", v))
        elif no == 8:
            ints += _packed_varints(v) if wt == 2 else [_signed(v)]
        elif no == 9:
            strings.append(v)
        elif no == 20:
            atype = v
    if atype is None:  # older writers omit the type: infer it
        atype = (A_FLOAT if f is not None else A_INT if i is not None else A_STRING if s is not None else
                 A_TENSOR if t is not None else A_FLOATS if floats else A_INTS if ints else A_STRINGS)
    value = {A_FLOAT: f, A_INT: i, A_STRING: s.decode() if s is not None else None, A_TENSOR: t,
             A_FLOATS: floats, A_INTS: ints, A_STRINGS: [x.decode() for x in strings]}.get(atype)
    if atype not in (A_FLOAT, A_INT, A_STRING, A_TENSOR, A_FLOATS, A_INTS, A_STRINGS):
        raise ValueError(f"attribute {name!r}: unsupported type {atype}")
    return name, value


def _node(buf: bytes) -> Node:
    n = Node("", [], [])
    for no, _, v in fields(buf):
        if no == 1:
            n.inputs.append(v.decode())
        elif no == 2:
            n.outputs.append(v.decode())
        elif no == 3:
            n.name = v.decode()
        elif no == 4:
            n.op_type = v.decode()
        elif no == 5:
            k, val = _attribute(v)
            n.attrs[k] = val
        elif no == 7:
            n.domain = v.decode()
    return n


def _value_info(buf: bytes) -> ValueInfo:
    name, shape, elem = "", [], FLOAT
    for no, _, v in fields(buf):
        if no == 1:
            name = v.decode()
        elif no == 2:                                   # TypeProto
            for no2, _, v2 in fields(v):
                if no2 == 1:                            # tensor_type
                    for no3, _, v3 in fields(v2):
                        if no3 == 1:
                            elem = v3
                        elif no3 == 2:                  # TensorShapeProto
                            for no4, _, v4 in fields(v3):
                                if no4 == 1:            # Dimension
                                    dim = None
                                    for no5, _, v5 in fields(v4):
                                        if no5 == 1:
                                            dim = _signed(v5)
                                    shape.append(dim)
    return ValueInfo(name, shape, elem)


def load(src) -> Model:
    """src: a path or the serialized bytes of a ModelProto."""
    buf = src if isinstance(src, (bytes, bytearray)) else open(src, "rb").read()
    model = Model(Graph([], [], [], {}), opsets={})
    for no, _, v in fields(bytes(buf)):
        if no == 1:
            model.ir_version = v
        elif no == 2:
            model.producer = v.decode()
        elif no == 8:
            dom, ver = "", 0
            for no2, _, v2 in fields(v):
                if no2 == 1:
                    dom = v2.decode()
                elif no2 == 2:
                    ver = v2
            model.opsets[dom] = ver
        elif no == 7:
            g = model.graph
            inputs = []
            for no2, _, v2 in fields(v):
                if no2 == 1:
                    g.nodes.append(_node(v2))
                elif no2 == 2:
                    g.name = v2.decode()
                elif no2 == 5:
                    k, arr = _tensor(v2)
                    g.initializers[k] = arr
                elif no2 == 11:
                    inputs.append(_value_info(v2))
                elif no2 == 12:
                    g.outputs.append(_value_info(v2))
            g.inputs = [vi for vi in inputs if vi.name not in g.initializers]
    return model


# ------------------------------------------------------------------ writer
def _enc_tensor(name: str, arr: np.ndarray) -> bytes:
    arr = np.ascontiguousarray(arr)
    dtype = {np.dtype(np.float32): FLOAT, np.dtype(np.int32): INT32, np.dtype(np.int64): INT64}[arr.dtype]
    out = b"".join(_vi(1, int(d)) for d in arr.shape)
    out += _vi(2, dtype) + _ld(8, name.encode()) + _ld(9, arr.astype(arr.dtype.newbyteorder("<")).tobytes())
    return out


def _enc_attr(name: str, v) -> bytes:
    out = _ld(1, name.encode())
    if isinstance(v, bool):
        v = int(v)
    if isinstance(v, float):
        out += _key(2, 5) + struct.pack("<f", v) + _vi(20, A_FLOAT)
    elif isinstance(v, (int, np.integer)):
        out += _vi(3, int(v)) + _vi(20, A_INT)
    elif isinstance(v, str):
        out += _ld(4, v.encode()) + _vi(20, A_STRING)
    elif isinstance(v, np.ndarray):
        out += _ld(5, _enc_tensor("", v)) + _vi(20, A_TENSOR)
    elif isinstance(v, (list, tuple)) and v and all(isinstance(x, float) for x in v):
        out += _ld(7, struct.pack(f"<{len(v)}f", *v)) + _vi(20, A_FLOATS)
    elif isinstance(v, (list, tuple)):
        out += b"".join(_vi(8, int(x)) for x in v) + _vi(20, A_INTS)
    else:
        raise TypeError(f"attribute {name!r}: cannot encode {type(v).__name__}")
    return out


def _enc_value_info(vi: ValueInfo) -> bytes:
    dims = b"".join(_ld(1, _vi(1, int(d)) if d is not None else _ld(2, b"N")) for d in vi.shape)
    tensor_type = _vi(1, vi.elem_type) + _ld(2, dims)
    return _ld(1, vi.name.encode()) + _ld(2, _ld(1, tensor_type))


def dumps(model: Model) -> bytes:
    g = model.graph
    body = b""
    for n in g.nodes:
        nb = b"".join(_ld(1, x.encode()) for x in n.inputs) + b"".join(_ld(2, x.encode()) for x in n.outputs)
        nb += _ld(3, n.name.encode()) + _ld(4, n.op_type.encode())
        nb += b"".join(_ld(5, _enc_attr(k, v)) for k, v in n.attrs.items())
        if n.domain:
            nb += _ld(7, n.domain.encode())
        body += _ld(1, nb)
    body += _ld(2, g.name.encode())
    body += b"".join(_ld(5, _enc_tensor(k, a)) for k, a in g.initializers.items())
    body += b"".join(_ld(11, _enc_value_info(vi)) for vi in g.inputs)
    body += b"".join(_ld(12, _enc_value_info(vi)) for vi in g.outputs)
    out = _vi(1, model.ir_version) + _ld(2, model.producer.encode()) + _ld(7, body)
    for dom, ver in model.opsets.items():
        out += _ld(8, _ld(1, dom.encode()) + _vi(2, ver))
    return out


def save(model: Model, path: str) -> None:
    with open(path, "wb") as f:
        f.write(dumps(model))
