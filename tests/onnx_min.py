"""Minimal reader of ONNX model files (protobuf wire format), enough for the pinned test models.

Test infrastructure.  The `onnx` Python package is not available, and the reference carries its
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
