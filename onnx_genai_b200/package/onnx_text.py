"""ONNX models in protobuf text format (``.onnx.textproto`` / ``.textproto`` / ``.pbtxt``) -> :class:`onnx_pb.Model`.

Tiny fixture models are easier to review as text than as binary, and the reference commits all of its workflow and
tiny-LLM fixtures that way (tests/fixtures/**/model.onnx.textproto; its ``onnx-std`` crate reads and writes the text
form).  This is a small recursive-descent reader of the protobuf text syntax -- ``field: scalar``, ``field { ... }``,
repeated fields by repetition or ``[a, b]`` lists, ``#`` comments, C-style string escapes including octal bytes --
followed by a mapping of the ONNX message tree onto the same dataclasses the binary reader produces, so everything
downstream (decoder lowering, the graph executor) is format-agnostic.
"""
from __future__ import annotations

import re

import numpy as np

from . import onnx_pb as pb

_TOKEN = re.compile(r"""\s*(?:(\#[^\n]*)|([{}\[\]<>:,;])|("(?:[^"\\]|\\.)*"|'(?:[^'\\]|\\.)*')|([^\s{}\[\]<>:,;"'\#]+))""", re.S)
_DTYPES = {"UNDEFINED": 0, "FLOAT": pb.FLOAT, "UINT8": pb.UINT8, "INT8": pb.INT8, "UINT16": pb.UINT16, "INT16": pb.INT16, "INT32": pb.INT32,
           "INT64": pb.INT64, "STRING": pb.STRING, "BOOL": pb.BOOL, "FLOAT16": pb.FLOAT16, "DOUBLE": pb.DOUBLE, "UINT32": pb.UINT32,
           "UINT64": pb.UINT64, "BFLOAT16": pb.BFLOAT16, "FLOAT8E4M3FN": pb.FLOAT8E4M3FN}
_SIMPLE = {"n": b"\n", "t": b"\t", "r": b"\r", "\\": b"\\", '"': b'"', "'": b"'", "a": b"\a", "b": b"\b", "f": b"\f", "v": b"\v", "?": b"?"}


class TextFormatError(ValueError):
    pass


def _unescape(lit: str) -> bytes:
    body, out, i = lit[1:-1], bytearray(), 0
    while i < len(body):
        c = body[i]
        if c != "\\":
            out += c.encode("utf-8")
            i += 1
            continue
        n = body[i + 1]
        if n in _SIMPLE:
            out += _SIMPLE[n]
            i += 2
        elif n in "xX":
            j = i + 2
            while j < len(body) and j < i + 4 and body[j] in "0123456789abcdefABCDEF":
                j += 1
            out.append(int(body[i + 2:j], 16))
            i = j
        elif n in "01234567":
            j = i + 1
            while j < len(body) and j < i + 4 and body[j] in "01234567":
                j += 1
            out.append(int(body[i + 1:j], 8) & 0xFF)
            i = j
        else:
            raise TextFormatError(f"unknown escape \\{n} in a string literal")
    return bytes(out)


def _tokens(text: str):
    pos, out = 0, []
    while True:
        m = _TOKEN.match(text, pos)
        if not m:
            if text[pos:].strip():
                raise TextFormatError(f"cannot read the text format at offset {pos}: {text[pos:pos + 30]!r}")
            return out
        pos = m.end()
        if m.group(1) is not None:
            continue
        if m.group(2) is not None:
            out.append(("p", m.group(2)))
        elif m.group(3) is not None:
            out.append(("s", _unescape(m.group(3))))
        else:
            out.append(("w", m.group(4)))


def _scalar(kind, val):
    if kind == "s":
        return val
    low = val.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("inf", "infinity", "+inf"):
        return float("inf")
    if low in ("-inf", "-infinity"):
        return float("-inf")
    if low == "nan":
        return float("nan")
    try:
        return int(val, 0) if not re.fullmatch(r"-?0\d+", val) else int(val, 8)
    except ValueError:
        pass
    try:
        return float(val[:-1] if low.endswith("f") else val)
    except ValueError:
        return val                          # an enum name


def parse_text(text: str) -> dict:
    """Protobuf text -> ``{field: [values]}`` where a value is a scalar, bytes, or a nested dict of the same form."""
    toks = _tokens(text)
    pos = 0

    def message(closer):
        nonlocal pos
        msg: dict = {}
        while pos < len(toks):
            kind, val = toks[pos]
            if kind == "p" and val == closer:
                pos += 1
                return msg
            if kind == "p" and val in ",;":
                pos += 1
                continue
            if kind != "w":
                raise TextFormatError(f"expected a field name, found {val!r}")
            name = val
            pos += 1
            if pos < len(toks) and toks[pos] == ("p", ":"):
                pos += 1
            kind, val = toks[pos]
            if kind == "p" and val in "{<":
                pos += 1
                msg.setdefault(name, []).append(message("}" if val == "{" else ">"))
            elif kind == "p" and val == "[":
                pos += 1
                while toks[pos] != ("p", "]"):
                    k2, v2 = toks[pos]
                    pos += 1
                    if k2 == "p" and v2 == ",":
                        continue
                    if k2 == "p" and v2 in "{<":
                        msg.setdefault(name, []).append(message("}" if v2 == "{" else ">"))
                    else:
                        msg.setdefault(name, []).append(_scalar(k2, v2))
                pos += 1
            else:
                pos += 1
                v = _scalar(kind, val)
                while kind == "s" and pos < len(toks) and toks[pos][0] == "s":       # adjacent string literals concatenate
                    v += toks[pos][1]
                    pos += 1
                msg.setdefault(name, []).append(v)
        if closer is not None:
            raise TextFormatError("the text ends inside a message: a closing brace is missing")
        return msg

    return message(None)


def _one(msg, key, default=None):
    v = msg.get(key)
    return v[0] if v else default


def _str(v) -> str:
    return v.decode("utf-8", errors="replace") if isinstance(v, (bytes, bytearray)) else ("" if v is None else str(v))


def _dtype(v) -> int:
    if isinstance(v, int):
        return v
    if v is None:
        return pb.FLOAT
    if _str(v) not in _DTYPES:
        raise TextFormatError(f"unknown tensor data type {v!r}")
    return _DTYPES[_str(v)]


def _tensor(msg, base_dir=None) -> pb.Tensor:
    t = pb.Tensor(name=_str(_one(msg, "name", b"")), dims=tuple(int(d) for d in msg.get("dims", [])), data_type=_dtype(_one(msg, "data_type")))
    npdt = pb._NP.get(t.data_type)
    if npdt is None:
        raise TextFormatError(f"tensor {t.name!r}: unsupported ONNX data type {t.data_type}")
    count = int(np.prod(t.dims)) if t.dims else 1
    raw = _one(msg, "raw_data")
    if "external_data" in msg:
        import os

        ext = {_str(_one(e, "key", b"")): _str(_one(e, "value", b"")) for e in msg["external_data"]}
        if base_dir is None:
            raise TextFormatError(f"tensor {t.name!r} is stored as external data ({ext.get('location')}), but the text was parsed "
                                  "without a directory to resolve it against; use load_model_text(path)")
        path = os.path.join(base_dir, ext["location"])
        if not os.path.exists(path):
            raise TextFormatError(f"tensor {t.name!r}: external data file {path} does not exist")
        t.external = ext
        t.array = np.fromfile(path, dtype=npdt, count=count, offset=int(ext.get("offset", 0) or 0)).reshape(t.dims)
    elif raw is not None:
        t.array = np.frombuffer(bytes(raw), dtype=npdt, count=count).reshape(t.dims)
    elif "float_data" in msg:
        t.array = np.asarray(msg["float_data"], dtype=np.float32).reshape(t.dims)
    elif "double_data" in msg:
        t.array = np.asarray(msg["double_data"], dtype=np.float64).reshape(t.dims)
    elif "int64_data" in msg:
        t.array = np.asarray(msg["int64_data"], dtype=np.int64).reshape(t.dims)
    elif "uint64_data" in msg:
        t.array = np.asarray(msg["uint64_data"], dtype=np.uint64).astype(npdt).reshape(t.dims)
    elif "int32_data" in msg:
        vals = np.asarray(msg["int32_data"], dtype=np.int64)
        t.array = vals.astype(np.uint16).view(npdt).reshape(t.dims) if t.data_type in (pb.FLOAT16, pb.BFLOAT16) else vals.astype(npdt).reshape(t.dims)
    else:
        t.array = np.zeros(t.dims, dtype=npdt)
    return t


def _attr(msg, base_dir=None):
    name = _str(_one(msg, "name", b""))
    if "t" in msg:
        return name, _tensor(msg["t"][0], base_dir)
    if "g" in msg:
        return name, _graph(msg["g"][0], base_dir)
    kind = _str(_one(msg, "type", b""))
    if "floats" in msg or kind == "FLOATS":
        return name, [float(v) for v in msg.get("floats", [])]
    if "ints" in msg or kind == "INTS":
        return name, [int(v) for v in msg.get("ints", [])]
    if "strings" in msg or kind == "STRINGS":
        return name, [_str(v) for v in msg.get("strings", [])]
    if "f" in msg:
        return name, float(msg["f"][0])
    if "i" in msg:
        return name, int(msg["i"][0])
    if "s" in msg:
        return name, _str(msg["s"][0])
    return name, {"FLOAT": 0.0, "INT": 0, "STRING": ""}.get(kind, 0)       # proto3 omits zero values


def _value_info(msg) -> pb.ValueInfo:
    tt = _one(_one(msg, "type", {}) or {}, "tensor_type", {}) or {}
    shape = []
    for d in (_one(tt, "shape", {}) or {}).get("dim", []):
        shape.append(int(d["dim_value"][0]) if "dim_value" in d else _str(_one(d, "dim_param", b"?")))
    return pb.ValueInfo(_str(_one(msg, "name", b"")), _dtype(_one(tt, "elem_type")) if tt else pb.FLOAT, tuple(shape))


def _graph(msg, base_dir=None) -> pb.Graph:
    g = pb.Graph(name=_str(_one(msg, "name", b"graph")))
    for n in msg.get("node", []):
        g.nodes.append(pb.Node(op_type=_str(_one(n, "op_type", b"")), inputs=[_str(v) for v in n.get("input", [])],
                               outputs=[_str(v) for v in n.get("output", [])], name=_str(_one(n, "name", b"")),
                               domain=_str(_one(n, "domain", b"")), attrs=dict(_attr(a, base_dir) for a in n.get("attribute", []))))
    for t in msg.get("initializer", []):
        tensor = _tensor(t, base_dir)
        g.initializers[tensor.name] = tensor
    g.inputs = [_value_info(v) for v in msg.get("input", [])]
    g.outputs = [_value_info(v) for v in msg.get("output", [])]
    return g


def parse_model_text(text: str, base_dir: str | None = None) -> pb.Model:
    root = parse_text(text)
    if "graph" not in root:
        raise TextFormatError("the text holds no `graph { ... }`: this is not an ONNX ModelProto in text format")
    m = pb.Model(graph=_graph(root["graph"][0], base_dir), ir_version=int(_one(root, "ir_version", 10)), producer_name=_str(_one(root, "producer_name", b"")))
    opsets = {_str(_one(o, "domain", b"")): int(_one(o, "version", 1)) for o in root.get("opset_import", [])}
    if opsets:
        m.opsets = opsets
    m.metadata = {_str(_one(p, "key", b"")): _str(_one(p, "value", b"")) for p in root.get("metadata_props", [])}
    return m


def load_model_text(path: str) -> pb.Model:
    import os

    with open(path, encoding="utf-8") as f:
        return parse_model_text(f.read(), os.path.dirname(os.path.abspath(path)))


def load_any(path: str) -> pb.Model:
    """Binary or text, by file name."""
    if path.endswith((".textproto", ".pbtxt", ".prototxt", ".txt")):
        return load_model_text(path)
    return pb.load_model(path)
