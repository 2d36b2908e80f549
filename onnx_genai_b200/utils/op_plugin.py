"""Third-party operator kernels behind the operator plugin ABI (``csrc/abi/ogb_kernel_abi.h``).

``OpPlugin(path)`` loads a plugin through the C++ host loader (``csrc/runtime/op_plugin_host.cpp``), which does the
version and capability handshake and checks the plugin's vtables.  ``register()`` enters every kernel the plugin lists
into the graph executor's operator table under ``domain::op`` (a domain-qualified entry wins over a built-in one; a
default-domain kernel replaces the built-in operator), so any graph run through ``GraphExecutor`` -- workflow components
included -- reaches the plugin.  Per node the plugin sees the attributes once (``create_kernel``); per call it infers
the output shapes, the host allocates torch tensors, and ``compute`` fills them.  Tensors are host tensors: a plugin is
used on the CPU path.  Counterpart of the reference's native EP plugin host (crates/onnx-runtime-ep-nxrt-abi).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_double, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p

import numpy as np
import torch

from ..package import onnx_pb as pb

MAX_RANK = 8
CODES = {0: "ok", 1: "invalid argument", 2: "unsupported", 3: "version mismatch", 4: "internal error"}
ATTR_INT, ATTR_FLOAT, ATTR_STRING, ATTR_INTS, ATTR_FLOATS = 1, 2, 3, 4, 5

_TORCH = {pb.FLOAT: torch.float32, pb.UINT8: torch.uint8, pb.INT8: torch.int8, pb.INT16: torch.int16, pb.INT32: torch.int32,
          pb.INT64: torch.int64, pb.BOOL: torch.bool, pb.FLOAT16: torch.float16, pb.DOUBLE: torch.float64, pb.BFLOAT16: torch.bfloat16}
_ONNX = {v: k for k, v in _TORCH.items()}


class OpPluginError(RuntimeError):
    def __init__(self, message, code=None):
        super().__init__(message)
        self.code = code


class _Tensor(Structure):
    _fields_ = [("struct_size", c_uint32), ("dtype", c_int32), ("rank", c_int32), ("reserved", c_int32), ("dims", c_int64 * MAX_RANK),
                ("data", c_void_p), ("byte_size", c_uint64)]


class _Attr(Structure):
    _fields_ = [("struct_size", c_uint32), ("kind", c_uint32), ("name", c_char_p), ("count", c_uint64), ("ints", POINTER(c_int64)),
                ("floats", POINTER(c_double)), ("string", c_char_p)]


class _Node(Structure):
    _fields_ = [("struct_size", c_uint32), ("num_attrs", c_uint32), ("domain", c_char_p), ("op_type", c_char_p), ("name", c_char_p),
                ("attrs", POINTER(_Attr)), ("num_inputs", c_uint32), ("num_outputs", c_uint32)]


def _lib():
    from ..engine.core import load_runtime

    lib = load_runtime()
    if not getattr(lib, "_ophost_bound", False):
        lib.ogb_ophost_load.argtypes, lib.ogb_ophost_load.restype = [c_char_p, c_char_p, c_int], c_void_p
        lib.ogb_ophost_name.argtypes, lib.ogb_ophost_name.restype = [c_void_p], c_char_p
        lib.ogb_ophost_kernel_count.argtypes, lib.ogb_ophost_kernel_count.restype = [c_void_p], c_int
        lib.ogb_ophost_capabilities.argtypes, lib.ogb_ophost_capabilities.restype = [c_void_p], c_int
        lib.ogb_ophost_kernel_desc.argtypes, lib.ogb_ophost_kernel_desc.restype = [c_void_p, c_int, c_char_p, c_int], c_int
        lib.ogb_ophost_create_kernel.argtypes = [c_void_p, c_int, POINTER(_Node), c_char_p, c_int]
        lib.ogb_ophost_create_kernel.restype = c_void_p
        lib.ogb_ophost_run.argtypes = [c_void_p, c_int, POINTER(_Tensor), c_int, POINTER(_Tensor), c_int, c_char_p, c_int]
        lib.ogb_ophost_run.restype = c_int
        lib.ogb_ophost_release_kernel.argtypes, lib.ogb_ophost_release_kernel.restype = [c_void_p], None
        lib.ogb_ophost_unload.argtypes, lib.ogb_ophost_unload.restype = [c_void_p, c_char_p, c_int], c_int
        lib._ophost_bound = True
    return lib


def _pack_attrs(attrs: dict):
    """Node attributes as an array of ABI attribute records, plus the Python objects that own their memory."""
    keep, recs = [], []
    for name, val in attrs.items():
        a = _Attr(struct_size=ctypes.sizeof(_Attr), name=name.encode(), count=1)
        if isinstance(val, bool) or isinstance(val, (int, np.integer)):
            buf = (c_int64 * 1)(int(val))
            a.kind, a.ints = ATTR_INT, buf
        elif isinstance(val, (float, np.floating)):
            buf = (c_double * 1)(float(val))
            a.kind, a.floats = ATTR_FLOAT, buf
        elif isinstance(val, (bytes, str)):
            buf = val.encode() if isinstance(val, str) else bytes(val)
            a.kind, a.string, a.count = ATTR_STRING, buf, len(buf)
        elif isinstance(val, (list, tuple)) and val and all(isinstance(v, (int, np.integer)) for v in val):
            buf = (c_int64 * len(val))(*[int(v) for v in val])
            a.kind, a.ints, a.count = ATTR_INTS, buf, len(val)
        elif isinstance(val, (list, tuple)) and val and all(isinstance(v, (int, float, np.floating, np.integer)) for v in val):
            buf = (c_double * len(val))(*[float(v) for v in val])
            a.kind, a.floats, a.count = ATTR_FLOATS, buf, len(val)
        else:
            continue                      # tensors and subgraphs do not cross this ABI
        keep.append(buf)
        recs.append(a)
    arr = (_Attr * max(1, len(recs)))(*recs)
    keep.append(arr)
    return arr, len(recs), keep


def _describe(t: torch.Tensor, with_data: bool) -> _Tensor:
    if t.dim() > MAX_RANK:
        raise OpPluginError(f"a tensor of rank {t.dim()} does not fit the plugin ABI (at most {MAX_RANK} axes)")
    if t.dtype not in _ONNX:
        raise OpPluginError(f"element type {t.dtype} does not cross the plugin ABI")
    d = _Tensor(struct_size=ctypes.sizeof(_Tensor), dtype=_ONNX[t.dtype], rank=t.dim())
    for i, s in enumerate(t.shape):
        d.dims[i] = int(s)
    d.byte_size = t.numel() * t.element_size()
    d.data = t.data_ptr() if with_data and t.numel() else None
    return d


class PluginKernel:
    """One node's kernel: created from the node's attributes, callable like an entry of the executor's operator table."""

    def __init__(self, plugin: "OpPlugin", index: int, domain: str, op_type: str, attrs: dict, num_inputs: int, num_outputs: int):
        self.plugin, self.lib = plugin, plugin.lib
        arr, n, keep = _pack_attrs(attrs)
        node = _Node(struct_size=ctypes.sizeof(_Node), num_attrs=n, domain=domain.encode(), op_type=op_type.encode(), name=b"",
                     attrs=arr, num_inputs=num_inputs, num_outputs=num_outputs)
        err = ctypes.create_string_buffer(256)
        self.handle = self.lib.ogb_ophost_create_kernel(plugin.handle, index, ctypes.byref(node), err, len(err))
        del keep
        if not self.handle:
            raise OpPluginError(f"{plugin.name}: cannot create a kernel for {domain}::{op_type}: {err.value.decode(errors='replace')}")
        self.num_outputs = num_outputs

    def __call__(self, inputs):
        ins = [t.detach().contiguous().cpu() for t in inputs if t is not None]
        in_arr = (_Tensor * max(1, len(ins)))(*[_describe(t, True) for t in ins])
        out_arr = (_Tensor * max(1, self.num_outputs))()
        for o in out_arr:
            o.struct_size = ctypes.sizeof(_Tensor)
        err = ctypes.create_string_buffer(256)
        rc = self.lib.ogb_ophost_run(self.handle, 0, in_arr, len(ins), out_arr, self.num_outputs, err, len(err))
        if rc != 0:
            raise OpPluginError(f"{self.plugin.name}: shape inference failed ({CODES.get(rc, rc)}): {err.value.decode(errors='replace')}", rc)
        outs = []
        for i in range(self.num_outputs):
            o = out_arr[i]
            if o.dtype not in _TORCH:
                raise OpPluginError(f"{self.plugin.name}: output {i} has element type {o.dtype}, which this host cannot allocate")
            t = torch.empty([int(o.dims[d]) for d in range(o.rank)], dtype=_TORCH[o.dtype])
            o.data = t.data_ptr() if t.numel() else None
            o.byte_size = t.numel() * t.element_size()
            outs.append(t)
        rc = self.lib.ogb_ophost_run(self.handle, 1, in_arr, len(ins), out_arr, self.num_outputs, err, len(err))
        if rc != 0:
            raise OpPluginError(f"{self.plugin.name}: kernel failed ({CODES.get(rc, rc)}): {err.value.decode(errors='replace')}", rc)
        return outs[0] if self.num_outputs == 1 else outs

    def close(self):
        if self.handle:
            self.lib.ogb_ophost_release_kernel(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class OpPlugin:
    def __init__(self, path: str):
        self.lib = _lib()
        err = ctypes.create_string_buffer(512)
        self.handle = self.lib.ogb_ophost_load(str(path).encode(), err, len(err))
        if not self.handle:
            raise OpPluginError(err.value.decode(errors="replace") or f"cannot load operator plugin {path}")
        self.path = str(path)
        self.name = (self.lib.ogb_ophost_name(self.handle) or b"").decode()
        self.kernels = []                   # (index, domain, op_type, since_version)
        buf = ctypes.create_string_buffer(512)
        for i in range(self.lib.ogb_ophost_kernel_count(self.handle)):
            since = self.lib.ogb_ophost_kernel_desc(self.handle, i, buf, len(buf))
            domain, op = buf.raw.split(b"\0")[:2]
            self.kernels.append((i, domain.decode(), op.decode(), since))
        self._registered: dict = {}         # table key -> previous entry (or None)
        self._live: list = []

    @property
    def capabilities(self) -> int:
        return int(self.lib.ogb_ophost_capabilities(self.handle))

    def kernel(self, domain: str, op_type: str, attrs: dict | None = None, num_inputs: int = 1, num_outputs: int = 1) -> PluginKernel:
        for i, d, o, _ in self.kernels:
            if d == domain and o == op_type:
                k = PluginKernel(self, i, domain, op_type, attrs or {}, num_inputs, num_outputs)
                self._live.append(k)
                return k
        raise OpPluginError(f"{self.name} has no kernel for {domain}::{op_type}")

    def register(self, table: dict | None = None) -> list:
        """Enter the plugin's kernels into the graph executor's operator table (``OPS`` by default).  A kernel object is
        created per distinct attribute set the first time a node with those attributes runs."""
        if table is None:
            from ..package.graph_executor import OPS as table
        names = []
        for i, domain, op, _ in self.kernels:
            key = f"{domain}::{op}" if domain else op
            cache: dict = {}

            def run(ins, attrs, _d=domain, _o=op, _cache=cache):
                sig = (len(ins), repr(sorted((k, repr(v)) for k, v in attrs.items())))
                k = _cache.get(sig)
                if k is None:
                    k = _cache[sig] = self.kernel(_d, _o, attrs, num_inputs=len(ins), num_outputs=1)
                return k(ins)

            self._registered[key] = table.get(key)
            table[key] = run
            names.append(key)
        self._table = table
        return names

    def unregister(self):
        for key, old in self._registered.items():
            if old is None:
                self._table.pop(key, None)
            else:
                self._table[key] = old
        self._registered.clear()

    def close(self):
        self.unregister()
        for k in self._live:
            k.close()
        self._live.clear()
        if self.handle:
            err = ctypes.create_string_buffer(256)
            rc = self.lib.ogb_ophost_unload(self.handle, err, len(err))
            if rc != 0:
                raise OpPluginError(err.value.decode(errors="replace"), rc)
            self.handle = None
