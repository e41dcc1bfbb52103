"""Minimal reader and writer of ONNX model files (protobuf wire format): enough for the models of the test-suite and
for the benchmark configurations, which are written as ONNX files and handed to the C++ generator.

The `onnx` Python package is not available, and the reference carries its
own wire reader for the same reason (parsers/src/onnx.hxx:19-120).  Only the fields the hot-path
models use are decoded: graph nodes with attributes, initializers (float/int64/int32, raw or typed
storage), graph inputs and outputs with static shapes.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np


def _varint(buf: bytes, pos: int):
    result = shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _fields(buf: bytes):
    """Yields (field number, wire type, value) for one message."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val = buf[pos:pos + 8]
            pos += 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            val = buf[pos:pos + ln]
            pos += ln
        elif wt == 5:
            val = buf[pos:pos + 4]
            pos += 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        yield num, wt, val


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


def _packed_varints(val, wt):
    if wt == 0:
        return [_signed(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed(v))
    return out


def _packed_floats(val, wt):
    if wt == 5:
        return [struct.unpack("<f", val)[0]]
    return list(struct.unpack(f"<{len(val) // 4}f", val))


_NP = {1: np.float32, 2: np.uint8, 3: np.int8, 6: np.int32, 7: np.int64, 11: np.float64}


def _tensor(buf: bytes):
    dims, dtype, name, raw = [], 1, "", None
    floats, int32s, int64s = [], [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_varints(val, wt)
        elif num == 2:
            dtype = val
        elif num == 4:
            floats += _packed_floats(val, wt)
        elif num == 5:
            int32s += _packed_varints(val, wt)
        elif num == 7:
            int64s += _packed_varints(val, wt)
        elif num == 8:
            name = val.decode()
        elif num == 9:
            raw = bytes(val)
    npdt = _NP[dtype]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=npdt).copy()
    elif dtype == 1:
        arr = np.array(floats, dtype=np.float32)
    elif dtype == 7:
        arr = np.array(int64s, dtype=np.int64)
    else:
        arr = np.array(int32s, dtype=npdt)
    return name, arr.reshape(dims)


def _attribute(buf: bytes):
    name, f, i, s, t = "", None, None, None, None
    floats, ints = [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            f = struct.unpack("<f", val)[0]
        elif num == 3:
            i = _signed(val)
        elif num == 4:
            s = val.decode()
        elif num == 5:
            t = _tensor(val)[1]
        elif num == 7:
            floats += _packed_floats(val, wt)
        elif num == 8:
            ints += _packed_varints(val, wt)
    for v in (f, i, s, t):
        if v is not None:
            return name, v
    return name, (floats if floats else ints)


@dataclass
class Node:
    op_type: str
    inputs: list
    outputs: list
    attrs: dict = field(default_factory=dict)


def _node(buf: bytes) -> Node:
    n = Node("", [], [])
    for num, wt, val in _fields(buf):
        if num == 1:
            n.inputs.append(val.decode())
        elif num == 2:
            n.outputs.append(val.decode())
        elif num == 4:
            n.op_type = val.decode()
        elif num == 5:
            k, v = _attribute(val)
            n.attrs[k] = v
    return n


def _value_info(buf: bytes):
    name, shape = "", []
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:  # TypeProto
            for n2, _, v2 in _fields(val):
                if n2 == 1:  # tensor_type
                    for n3, _, v3 in _fields(v2):
                        if n3 == 2:  # shape
                            for n4, _, v4 in _fields(v3):
                                if n4 == 1:  # dim
                                    d = None
                                    for n5, _, v5 in _fields(v4):
                                        if n5 == 1:
                                            d = _signed(v5)
                                    shape.append(d)
    return name, shape


@dataclass
class Graph:
    nodes: list
    initializers: dict
    inputs: list   # [(name, shape)] without initializers
    outputs: list  # [name]


def load(path: str) -> Graph:
    data = open(path, "rb").read()
    graph = None
    for num, wt, val in _fields(data):
        if num == 7:
            graph = val
    if graph is None:
        raise ValueError(f"{path}: no graph")
    nodes, inits, inputs, outputs = [], {}, [], []
    for num, wt, val in _fields(graph):
        if num == 1:
            nodes.append(_node(val))
        elif num == 5:
            k, v = _tensor(val)
            inits[k] = v
        elif num == 11:
            inputs.append(_value_info(val))
        elif num == 12:
            outputs.append(_value_info(val)[0])
    inputs = [(n, s) for n, s in inputs if n not in inits]
    return Graph(nodes, inits, inputs, outputs)


# ---- writer: the inverse of load(), used to hand the fixtures' graphs to the C++ front-end ----------
def _enc_varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _field(num: int, wt: int, payload: bytes) -> bytes:
    key = _enc_varint((num << 3) | wt)
    if wt == 2:
        return key + _enc_varint(len(payload)) + payload
    return key + payload


_ONNX_DT = {np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.int32): 6, np.dtype(np.int64): 7}


def _enc_tensor(name: str, arr: np.ndarray, data_type: int | None = None) -> bytes:
    arr = np.ascontiguousarray(arr)
    out = b"".join(_field(1, 0, _enc_varint(int(d))) for d in arr.shape)
    out += _field(2, 0, _enc_varint(data_type if data_type is not None else _ONNX_DT[arr.dtype]))
    out += _field(8, 2, name.encode())
    out += _field(9, 2, arr.tobytes())
    return out


def _enc_attr(name: str, v) -> bytes:
    out = _field(1, 2, name.encode())
    if isinstance(v, float):
        out += _field(2, 5, struct.pack("<f", v)) + _field(20, 0, _enc_varint(1))
    elif isinstance(v, bool) or isinstance(v, int):
        out += _field(3, 0, _enc_varint(int(v))) + _field(20, 0, _enc_varint(2))
    elif isinstance(v, str):
        out += _field(4, 2, v.encode()) + _field(20, 0, _enc_varint(3))
    elif isinstance(v, (list, tuple)) and v and isinstance(v[0], float):
        out += b"".join(_field(7, 5, struct.pack("<f", x)) for x in v) + _field(20, 0, _enc_varint(6))
    elif isinstance(v, (list, tuple)):
        out += b"".join(_field(8, 0, _enc_varint(int(x))) for x in v) + _field(20, 0, _enc_varint(7))
    else:
        raise TypeError(f"attribute {name}: {type(v)}")
    return out


def _enc_value_info(name: str, shape, elem_type: int = 1) -> bytes:
    dims = b"".join(_field(1, 2, _field(1, 0, _enc_varint(int(d))) if not isinstance(d, str) else _field(2, 2, d.encode())) for d in shape)
    tensor_type = _field(1, 0, _enc_varint(elem_type)) + _field(2, 2, dims)
    return _field(1, 2, name.encode()) + _field(2, 2, _field(1, 2, tensor_type))


def save(path: str, nodes: list, initializers: dict, inputs: list, outputs: list, input_types: dict | None = None,
         initializer_types: dict | None = None) -> None:
    """Writes an ONNX file.  nodes: [{"op", "in", "out", "attrs"}]; inputs: [(name, shape)]; outputs: [name]."""
    g = b""
    for n in nodes:
        body = b"".join(_field(1, 2, i.encode()) for i in n["in"]) + b"".join(_field(2, 2, o.encode()) for o in n["out"])
        body += _field(4, 2, n["op"].encode())
        body += b"".join(_field(5, 2, _enc_attr(k, v)) for k, v in n.get("attrs", {}).items())
        g += _field(1, 2, body)
    g += _field(2, 2, b"graph")
    for k, v in initializers.items():
        g += _field(5, 2, _enc_tensor(k, v, (initializer_types or {}).get(k)))
    for name, shape in inputs:
        g += _field(11, 2, _enc_value_info(name, shape, (input_types or {}).get(name, 1)))
    for name in outputs:
        g += _field(12, 2, _enc_value_info(name, []))
    model = _field(1, 0, _enc_varint(8)) + _field(7, 2, g) + _field(8, 2, _field(2, 0, _enc_varint(17)))
    with open(path, "wb") as f:
        f.write(model)
