"""Growable device buffers: one reserved address range, physical memory mapped behind its front on demand.

Python face of ``csrc/kernels/vmm_pool.cu`` (CUDA virtual memory management; the reference's ``CudaVmmAllocator``,
crates/onnx-runtime-cuda-memory/src/vmm_allocator.rs).  A :class:`GrowableBuffer` keeps its base address for life, so
tensors viewing it, captured CUDA graphs and cached TMA descriptors stay valid while it grows; ``shrink`` returns
physical memory to the device without giving up the address range.

``view(dtype, shape)`` hands out a torch tensor over the *mapped* front of the range; views taken before a ``grow`` stay
valid (same addresses), a larger view is taken afterwards.  Views must not outlive the buffer, and nothing may touch
the part that a ``shrink`` gives back.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint64, c_void_p

import torch

from ..ops import _native

for _name, _args, _res in (("ogb_vmm_available", [c_int], c_int), ("ogb_vmm_create", [c_int, c_uint64, ctypes.POINTER(c_void_p)], c_int),
                           ("ogb_vmm_grow", [c_void_p, c_uint64], c_int), ("ogb_vmm_shrink", [c_void_p, c_uint64], c_int),
                           ("ogb_vmm_ptr", [c_void_p], c_uint64), ("ogb_vmm_mapped", [c_void_p], c_uint64),
                           ("ogb_vmm_reserved", [c_void_p], c_uint64), ("ogb_vmm_granularity", [c_void_p], c_uint64),
                           ("ogb_vmm_chunks", [c_void_p], c_int), ("ogb_vmm_destroy", [c_void_p], c_int)):
    _native.register(_name, _args, _res)


class VmmError(RuntimeError):
    pass


def available(device: int = 0) -> bool:
    return torch.cuda.is_available() and bool(_native.load().ogb_vmm_available(int(device)))


class _Span:
    """Exposes a device address range through ``__cuda_array_interface__`` so torch can view it without copying."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class GrowableBuffer:
    def __init__(self, reserve_bytes: int, device: int = 0, initial_bytes: int = 0):
        self.lib = _native.load()
        self.device = int(device)
        handle = c_void_p()
        rc = self.lib.ogb_vmm_create(self.device, int(reserve_bytes), ctypes.byref(handle))
        if rc != 0:
            raise VmmError(f"cannot reserve {reserve_bytes / 2**30:.2f} GiB of device address space on cuda:{device} "
                           f"({'virtual memory management is not available' if rc == -2 else f'code {rc}'})")
        self.handle = handle
        if initial_bytes:
            self.grow(initial_bytes)

    @property
    def ptr(self) -> int:
        return int(self.lib.ogb_vmm_ptr(self.handle))

    @property
    def mapped(self) -> int:
        return int(self.lib.ogb_vmm_mapped(self.handle))

    @property
    def reserved(self) -> int:
        return int(self.lib.ogb_vmm_reserved(self.handle))

    @property
    def granularity(self) -> int:
        return int(self.lib.ogb_vmm_granularity(self.handle))

    @property
    def chunks(self) -> int:
        return int(self.lib.ogb_vmm_chunks(self.handle))

    def grow(self, nbytes: int) -> int:
        """Back at least ``nbytes`` from the start of the range; returns the mapped size.  The base address does not move."""
        rc = self.lib.ogb_vmm_grow(self.handle, int(nbytes))
        if rc == -4:
            raise VmmError(f"cannot grow to {nbytes / 2**30:.2f} GiB: only {self.reserved / 2**30:.2f} GiB of address space was reserved")
        if rc != 0:
            raise VmmError(f"cannot grow to {nbytes / 2**30:.2f} GiB ({'out of device memory' if rc == 2 else f'code {rc}'}); "
                           f"{self.mapped / 2**30:.2f} GiB stay mapped")
        return self.mapped

    def shrink(self, keep_bytes: int) -> int:
        """Release whole chunks beyond ``keep_bytes`` (synchronises the device first); returns the mapped size."""
        torch.cuda.synchronize(self.device)
        rc = self.lib.ogb_vmm_shrink(self.handle, int(keep_bytes))
        if rc != 0:
            raise VmmError(f"shrink failed (code {rc})")
        return self.mapped

    def view(self, dtype=torch.uint8, shape=None, offset_bytes: int = 0) -> torch.Tensor:
        """A tensor over the mapped part starting at ``offset_bytes`` (all of it, or ``shape`` elements of ``dtype``)."""
        item = torch.empty(0, dtype=dtype).element_size()
        avail = self.mapped - offset_bytes
        if shape is None:
            shape = (avail // item,)
        count = 1
        for s in shape:
            count *= int(s)
        if count * item > avail or offset_bytes < 0:
            raise VmmError(f"a view of {count * item} bytes at offset {offset_bytes} exceeds the {self.mapped} mapped bytes; grow first")
        if count == 0:
            return torch.empty(shape, dtype=dtype, device=f"cuda:{self.device}")
        flat = torch.as_tensor(_Span(self.ptr + offset_bytes, count * item, self), device=f"cuda:{self.device}")
        return flat.view(dtype).view(*shape)

    def span(self, dtype, shape) -> torch.Tensor:
        """A tensor over the *reserved* range, backed or not, for buffers that are indexed by a unit (a page) and grow in
        place.  The caller must only touch units inside the mapped part; whole-tensor operations are out."""
        item = torch.empty(0, dtype=dtype).element_size()
        count = 1
        for s in shape:
            count *= int(s)
        if count * item > self.reserved:
            raise VmmError(f"a span of {count * item} bytes exceeds the {self.reserved} reserved bytes")
        flat = torch.as_tensor(_Span(self.ptr, count * item, self), device=f"cuda:{self.device}")
        return flat.view(dtype).view(*shape)

    def close(self) -> None:
        if self.handle:
            torch.cuda.synchronize(self.device)
            self.lib.ogb_vmm_destroy(self.handle)
            self.handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
