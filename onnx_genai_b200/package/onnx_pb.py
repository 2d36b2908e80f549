"""Dependency-free ONNX protobuf reader / writer (wire level) with external-data support.

Neither ``onnx`` nor ``onnxruntime`` is required: this module decodes and encodes the subset of
``onnx.proto3`` a decoder package uses (ModelProto, GraphProto, NodeProto, AttributeProto,
TensorProto, ValueInfoProto, StringStringEntry, OperatorSetId) directly from the protobuf wire
format.  Tensors stored as external data are memory-mapped, never copied.  Role of the
reference's `onnx-runtime-loader` (crates/onnx-runtime-loader/src/lib.rs:1-40, weights.rs) and
writer (writer.rs).
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass, field

import numpy as np

# TensorProto.DataType
FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL, FLOAT16, DOUBLE, UINT32, UINT64 = range(1, 14)
BFLOAT16 = 16
FLOAT8E4M3FN = 17
_NP = {FLOAT: np.float32, UINT8: np.uint8, INT8: np.int8, UINT16: np.uint16, INT16: np.int16, INT32: np.int32,
       INT64: np.int64, BOOL: np.bool_, FLOAT16: np.float16, DOUBLE: np.float64, UINT32: np.uint32, UINT64: np.uint64,
       BFLOAT16: np.uint16, FLOAT8E4M3FN: np.uint8}
_ITEM = {k: np.dtype(v).itemsize for k, v in _NP.items()}


# ---------------------------------------------------------------------------------------------
# wire primitives
# ---------------------------------------------------------------------------------------------
def _read_varint(buf, pos):
    result = 0
    shift = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _fields(buf, start=0, end=None):
    """Yield (field_number, wire_type, value) where value is int (varint/fixed) or a (start, end) span."""
    pos = start
    end = len(buf) if end is None else end
    while pos < end:
        key, pos = _read_varint(buf, pos)
        fn, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _read_varint(buf, pos)
            yield fn, wt, v
        elif wt == 1:
            yield fn, wt, struct.unpack_from("<Q", buf, pos)[0]
            pos += 8
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            yield fn, wt, (pos, pos + ln)
            pos += ln
        elif wt == 5:
            yield fn, wt, struct.unpack_from("<I", buf, pos)[0]
            pos += 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt} at offset {pos}")


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def _varint(v):
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


def _key(fn, wt):
    return _varint((fn << 3) | wt)


def _ld(fn, payload: bytes):
    return _key(fn, 2) + _varint(len(payload)) + payload


def _str(fn, s: str):
    return _ld(fn, s.encode("utf-8"))


def _int(fn, v: int):
    return _key(fn, 0) + _varint(int(v))


# ---------------------------------------------------------------------------------------------
# model objects
# ---------------------------------------------------------------------------------------------
@dataclass
class Tensor:
    name: str = ""
    dims: tuple = ()
    data_type: int = FLOAT
    array: np.ndarray | None = None         # raw element view (bf16 as uint16)
    external: dict = field(default_factory=dict)

    def numpy(self) -> np.ndarray:
        return self.array


@dataclass
class Attribute:
    name: str
    value: object


@dataclass
class Node:
    op_type: str
    inputs: list
    outputs: list
    name: str = ""
    domain: str = ""
    attrs: dict = field(default_factory=dict)


@dataclass
class ValueInfo:
    name: str
    elem_type: int = FLOAT
    shape: tuple = ()


@dataclass
class Graph:
    name: str = "decoder"
    nodes: list = field(default_factory=list)
    initializers: dict = field(default_factory=dict)   # name -> Tensor
    inputs: list = field(default_factory=list)
    outputs: list = field(default_factory=list)


@dataclass
class Model:
    graph: Graph = field(default_factory=Graph)
    ir_version: int = 10
    producer_name: str = "onnx_genai_b200"
    opsets: dict = field(default_factory=lambda: {"": 21, "com.microsoft": 1})
    metadata: dict = field(default_factory=dict)


# ---------------------------------------------------------------------------------------------
# decoding
# ---------------------------------------------------------------------------------------------
class _Mapped:
    """Keeps memory maps of external-data files alive for the arrays that view them."""

    def __init__(self):
        self.maps = {}

    def view(self, path):
        m = self.maps.get(path)
        if m is None:
            f = open(path, "rb")
            m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self.maps[path] = m
        return m


def _packed_ints(buf, span):
    out, pos = [], span[0]
    while pos < span[1]:
        v, pos = _read_varint(buf, pos)
        out.append(_signed(v))
    return out


def _decode_tensor(buf, span, base_dir, mapped) -> Tensor:
    t = Tensor()
    dims, raw, ext = [], None, {}
    f32, i32, i64 = [], [], []
    location = 0
    for fn, wt, v in _fields(buf, *span):
        if fn == 1:
            dims += _packed_ints(buf, v) if wt == 2 else [_signed(v)]
        elif fn == 2:
            t.data_type = v
        elif fn == 4:
            f32 += list(np.frombuffer(buf[v[0]:v[1]], dtype="<f4")) if wt == 2 else [struct.unpack("<f", struct.pack("<I", v))[0]]
        elif fn == 5:
            i32 += _packed_ints(buf, v) if wt == 2 else [_signed(v)]
        elif fn == 7:
            i64 += _packed_ints(buf, v) if wt == 2 else [_signed(v)]
        elif fn == 8:
            t.name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 9:
            raw = v
        elif fn == 13:
            k = val = ""
            for f2, _, v2 in _fields(buf, *v):
                if f2 == 1:
                    k = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 2:
                    val = bytes(buf[v2[0]:v2[1]]).decode()
            ext[k] = val
        elif fn == 14:
            location = v
    t.dims = tuple(dims)
    npdt = _NP.get(t.data_type)
    if npdt is None:
        raise ValueError(f"tensor {t.name!r}: unsupported ONNX data type {t.data_type}")
    count = int(np.prod(dims)) if dims else 1
    if location == 1 or ext:
        t.external = ext
        if base_dir is None:
            raise ValueError(f"tensor {t.name!r} uses external data but the model was parsed from bytes without a directory")
        path = os.path.join(base_dir, ext["location"])
        off = int(ext.get("offset", 0))
        m = mapped.view(path)
        t.array = np.frombuffer(m, dtype=npdt, count=count, offset=off).reshape(dims)
    elif raw is not None:
        t.array = np.frombuffer(buf, dtype=npdt, count=count, offset=raw[0]).reshape(dims)
    elif f32:
        t.array = np.asarray(f32, dtype=np.float32).reshape(dims)
    elif i64:
        t.array = np.asarray(i64, dtype=np.int64).reshape(dims)
    elif i32:
        if t.data_type in (FLOAT16, BFLOAT16):
            t.array = np.asarray(i32, dtype=np.uint16).reshape(dims).view(npdt)
        else:
            t.array = np.asarray(i32).astype(npdt).reshape(dims)
    else:
        t.array = np.zeros(dims, dtype=npdt)
    return t


def _decode_attr(buf, span, base_dir, mapped):
    name, val = "", None
    floats, ints, strs = [], [], []
    for fn, wt, v in _fields(buf, *span):
        if fn == 1:
            name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 2:
            val = struct.unpack("<f", struct.pack("<I", v))[0]
        elif fn == 3:
            val = _signed(v)
        elif fn == 4:
            val = bytes(buf[v[0]:v[1]])
        elif fn == 5:
            val = _decode_tensor(buf, v, base_dir, mapped)
        elif fn == 6:                      # a subgraph (If / Loop / Scan bodies)
            val = _decode_graph(buf, v, base_dir, mapped)
        elif fn == 7:
            floats += list(np.frombuffer(buf[v[0]:v[1]], dtype="<f4")) if wt == 2 else [struct.unpack("<f", struct.pack("<I", v))[0]]
        elif fn == 8:
            ints += _packed_ints(buf, v) if wt == 2 else [_signed(v)]
        elif fn == 9:
            strs.append(bytes(buf[v[0]:v[1]]))
    if val is None:
        val = floats or ints or strs or 0
    if isinstance(val, bytes):
        try:
            val = val.decode()
        except UnicodeDecodeError:
            pass
    return name, val


def _decode_value_info(buf, span) -> ValueInfo:
    vi = ValueInfo("")
    for fn, wt, v in _fields(buf, *span):
        if fn == 1:
            vi.name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 2:
            for f2, _, v2 in _fields(buf, *v):
                if f2 == 1:  # tensor_type
                    for f3, _, v3 in _fields(buf, *v2):
                        if f3 == 1:
                            vi.elem_type = v3
                        elif f3 == 2:
                            dims = []
                            for f4, _, v4 in _fields(buf, *v3):
                                if f4 == 1:
                                    d = None
                                    for f5, w5, v5 in _fields(buf, *v4):
                                        if f5 == 1:
                                            d = _signed(v5)
                                        elif f5 == 2:
                                            d = bytes(buf[v5[0]:v5[1]]).decode()
                                    dims.append(d)
                            vi.shape = tuple(dims)
    return vi


def _decode_node(buf, span, base_dir, mapped) -> Node:
    n = Node("", [], [])
    for fn, wt, v in _fields(buf, *span):
        if fn == 1:
            n.inputs.append(bytes(buf[v[0]:v[1]]).decode())
        elif fn == 2:
            n.outputs.append(bytes(buf[v[0]:v[1]]).decode())
        elif fn == 3:
            n.name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 4:
            n.op_type = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 5:
            k, val = _decode_attr(buf, v, base_dir, mapped)
            n.attrs[k] = val
        elif fn == 7:
            n.domain = bytes(buf[v[0]:v[1]]).decode()
    return n


def _decode_graph(buf, span, base_dir, mapped) -> Graph:
    g = Graph()
    for fn, wt, v in _fields(buf, *span):
        if fn == 1:
            g.nodes.append(_decode_node(buf, v, base_dir, mapped))
        elif fn == 2:
            g.name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 5:
            t = _decode_tensor(buf, v, base_dir, mapped)
            g.initializers[t.name] = t
        elif fn == 11:
            g.inputs.append(_decode_value_info(buf, v))
        elif fn == 12:
            g.outputs.append(_decode_value_info(buf, v))
    return g


def load_model(path: str) -> Model:
    """Parse ``path`` (memory-mapped); initializers view the file or its external-data files."""
    mapped = _Mapped()
    buf = mapped.view(path)
    model = parse_model(buf, os.path.dirname(os.path.abspath(path)), mapped)
    model._mapped = mapped  # keep maps alive
    return model


def parse_model(buf, base_dir=None, mapped=None) -> Model:
    mapped = mapped or _Mapped()
    m = Model(opsets={})
    for fn, wt, v in _fields(buf):
        if fn == 1:
            m.ir_version = v
        elif fn == 2:
            m.producer_name = bytes(buf[v[0]:v[1]]).decode()
        elif fn == 7:
            m.graph = _decode_graph(buf, v, base_dir, mapped)
        elif fn == 8:
            dom, ver = "", 0
            for f2, _, v2 in _fields(buf, *v):
                if f2 == 1:
                    dom = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 2:
                    ver = v2
            m.opsets[dom] = ver
        elif fn == 14:
            k = val = ""
            for f2, _, v2 in _fields(buf, *v):
                if f2 == 1:
                    k = bytes(buf[v2[0]:v2[1]]).decode()
                elif f2 == 2:
                    val = bytes(buf[v2[0]:v2[1]]).decode()
            m.metadata[k] = val
    return m


# ---------------------------------------------------------------------------------------------
# encoding
# ---------------------------------------------------------------------------------------------
def _enc_tensor(t: Tensor, ext_file=None, ext_name=None, threshold=1024) -> bytes:
    out = bytearray()
    for d in t.dims:
        out += _int(1, d)
    out += _int(2, t.data_type)
    out += _str(8, t.name)
    raw = np.ascontiguousarray(t.array).tobytes()
    if ext_file is not None and len(raw) >= threshold:
        pad = (-ext_file.tell()) % 64
        ext_file.write(b"\0" * pad)
        off = ext_file.tell()
        ext_file.write(raw)
        for k, v in (("location", ext_name), ("offset", str(off)), ("length", str(len(raw)))):
            out += _ld(13, _str(1, k) + _str(2, v))
        out += _int(14, 1)
    else:
        out += _ld(9, raw)
    return bytes(out)


def _enc_attr(name, val) -> bytes:
    out = bytearray(_str(1, name))
    if isinstance(val, bool):
        val = int(val)
    if isinstance(val, float):
        out += _key(2, 5) + struct.pack("<f", val) + _int(20, 1)
    elif isinstance(val, int):
        out += _int(3, val) + _int(20, 2)
    elif isinstance(val, str):
        out += _ld(4, val.encode()) + _int(20, 3)
    elif isinstance(val, Tensor):
        out += _ld(5, _enc_tensor(val)) + _int(20, 4)
    elif isinstance(val, Graph):
        out += _ld(6, _enc_graph(val)) + _int(20, 5)
    elif isinstance(val, (list, tuple)) and val and isinstance(val[0], float):
        for f in val:
            out += _key(7, 5) + struct.pack("<f", f)
        out += _int(20, 6)
    elif isinstance(val, (list, tuple)):
        for i in val:
            out += _int(8, i)
        out += _int(20, 7)
    else:
        raise TypeError(f"attribute {name!r}: unsupported value {type(val)}")
    return bytes(out)


def _enc_value_info(vi: ValueInfo) -> bytes:
    dims = bytearray()
    for d in vi.shape:
        dims += _ld(1, _str(2, d) if isinstance(d, str) else _int(1, d))
    ttype = _int(1, vi.elem_type) + _ld(2, bytes(dims))
    return _str(1, vi.name) + _ld(2, _ld(1, ttype))


def _enc_node(n: Node) -> bytes:
    out = bytearray()
    for i in n.inputs:
        out += _str(1, i)
    for o in n.outputs:
        out += _str(2, o)
    if n.name:
        out += _str(3, n.name)
    out += _str(4, n.op_type)
    for k, v in n.attrs.items():
        out += _ld(5, _enc_attr(k, v))
    if n.domain:
        out += _str(7, n.domain)
    return bytes(out)


def _enc_graph(g: Graph) -> bytes:
    """A subgraph, tensors inline (bodies of control-flow operators are small)."""
    gb = bytearray()
    for n in g.nodes:
        gb += _ld(1, _enc_node(n))
    gb += _str(2, g.name)
    for t in g.initializers.values():
        gb += _ld(5, _enc_tensor(t))
    for vi in g.inputs:
        gb += _ld(11, _enc_value_info(vi))
    for vi in g.outputs:
        gb += _ld(12, _enc_value_info(vi))
    return bytes(gb)


def save_model(model: Model, path: str, external_data: bool = True) -> None:
    """Write ``path``; tensors of 1 KiB or more go to ``<path>.data`` when ``external_data``."""
    ext_name = os.path.basename(path) + ".data"
    ext_file = open(os.path.join(os.path.dirname(os.path.abspath(path)), ext_name), "wb") if external_data else None
    g = model.graph
    gb = bytearray()
    for n in g.nodes:
        gb += _ld(1, _enc_node(n))
    gb += _str(2, g.name)
    for t in g.initializers.values():
        gb += _ld(5, _enc_tensor(t, ext_file, ext_name))
    for vi in g.inputs:
        gb += _ld(11, _enc_value_info(vi))
    for vi in g.outputs:
        gb += _ld(12, _enc_value_info(vi))
    out = bytearray(_int(1, model.ir_version) + _str(2, model.producer_name))
    out += _ld(7, bytes(gb))
    for dom, ver in model.opsets.items():
        out += _ld(8, _str(1, dom) + _int(2, ver))
    for k, v in model.metadata.items():
        out += _ld(14, _str(1, k) + _str(2, v))
    with open(path, "wb") as f:
        f.write(out)
    if ext_file is not None:
        ext_file.close()
