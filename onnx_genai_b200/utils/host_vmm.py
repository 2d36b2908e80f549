"""Growable host buffers with a stable address (``csrc/runtime/host_vmm.cpp``): reserve, commit on demand, decommit.

The host twin of :mod:`onnx_genai_b200.utils.vmm`.  ``view`` returns a torch CPU tensor over the committed front; views
taken before a ``grow`` stay valid.  Nothing may touch what a ``shrink`` gave back (it faults, by design)."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint64, c_void_p

import torch


class HostVmmError(RuntimeError):
    pass


def _lib():
    from ..engine.core import load_runtime

    lib = load_runtime()
    if not getattr(lib, "_hostvmm_bound", False):
        lib.ogb_hostvmm_reserve.argtypes, lib.ogb_hostvmm_reserve.restype = [c_uint64], c_void_p
        lib.ogb_hostvmm_commit.argtypes, lib.ogb_hostvmm_commit.restype = [c_void_p, c_uint64], c_int
        lib.ogb_hostvmm_decommit.argtypes, lib.ogb_hostvmm_decommit.restype = [c_void_p, c_uint64], c_int
        for name in ("base", "committed", "reserved", "page"):
            fn = getattr(lib, "ogb_hostvmm_" + name)
            fn.argtypes, fn.restype = [c_void_p], c_uint64
        lib.ogb_hostvmm_release.argtypes, lib.ogb_hostvmm_release.restype = [c_void_p], None
        lib._hostvmm_bound = True
    return lib


class HostGrowableBuffer:
    def __init__(self, reserve_bytes: int, initial_bytes: int = 0):
        self.lib = _lib()
        self.handle = self.lib.ogb_hostvmm_reserve(int(reserve_bytes))
        if not self.handle:
            raise HostVmmError(f"cannot reserve {reserve_bytes / 2**30:.2f} GiB of address space")
        if initial_bytes:
            self.grow(initial_bytes)

    ptr = property(lambda self: int(self.lib.ogb_hostvmm_base(self.handle)))
    committed = property(lambda self: int(self.lib.ogb_hostvmm_committed(self.handle)))
    reserved = property(lambda self: int(self.lib.ogb_hostvmm_reserved(self.handle)))
    page = property(lambda self: int(self.lib.ogb_hostvmm_page(self.handle)))

    def grow(self, nbytes: int) -> int:
        rc = self.lib.ogb_hostvmm_commit(self.handle, int(nbytes))
        if rc == -1:
            raise HostVmmError(f"cannot grow to {nbytes} bytes: only {self.reserved} bytes of address space were reserved")
        if rc != 0:
            raise HostVmmError(f"commit of {nbytes} bytes failed (errno {rc})")
        return self.committed

    def shrink(self, keep_bytes: int) -> int:
        rc = self.lib.ogb_hostvmm_decommit(self.handle, int(keep_bytes))
        if rc != 0:
            raise HostVmmError(f"decommit failed (errno {rc})")
        return self.committed

    def view(self, dtype=torch.uint8, shape=None, offset_bytes: int = 0) -> torch.Tensor:
        item = torch.empty(0, dtype=dtype).element_size()
        avail = self.committed - offset_bytes
        if shape is None:
            shape = (avail // item,)
        count = 1
        for s in shape:
            count *= int(s)
        if offset_bytes < 0 or count * item > avail:
            raise HostVmmError(f"a view of {count * item} bytes at offset {offset_bytes} exceeds the {self.committed} committed bytes; grow first")
        buf = (ctypes.c_uint8 * (count * item)).from_address(self.ptr + offset_bytes)
        return torch.frombuffer(buf, dtype=torch.uint8, count=count * item).view(dtype).reshape(tuple(shape))

    def close(self) -> None:
        if self.handle:
            self.lib.ogb_hostvmm_release(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
