"""Third-party host allocators behind the memory plugin ABI (``csrc/abi/ogb_memory_abi.h``).

``PluginAllocator(path)`` loads a plugin through the C++ host loader (``csrc/runtime/mem_plugin_host.cpp``), which does
the version negotiation and the prefix-rule reading of the plugin's vtable.  ``tensor(shape, dtype)`` hands out a torch
tensor over plugin memory; the memory goes back to the plugin when the tensor's owner is dropped or ``free`` is called.
The engine uses it for its host swap space when ``EngineConfig.host_allocator_plugin`` names a plugin.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_uint64, c_void_p

import numpy as np
import torch

CODES = {0: "ok", 1: "out of memory", 2: "invalid argument", 3: "unsupported", 4: "version mismatch", 5: "internal error"}


class MemPluginError(RuntimeError):
    def __init__(self, message, code=None):
        super().__init__(message)
        self.code = code


def _lib():
    from ..engine.core import load_runtime

    lib = load_runtime()
    if not getattr(lib, "_memhost_bound", False):
        lib.ogb_memhost_load.argtypes = [c_char_p, c_uint64, c_char_p, c_char_p, c_int]
        lib.ogb_memhost_load.restype = c_void_p
        lib.ogb_memhost_level.argtypes, lib.ogb_memhost_level.restype = [c_void_p], c_int
        lib.ogb_memhost_name.argtypes, lib.ogb_memhost_name.restype = [c_void_p], c_char_p
        lib.ogb_memhost_alloc.argtypes = [c_void_p, c_uint64, c_uint64, ctypes.POINTER(c_void_p), c_char_p, c_int]
        lib.ogb_memhost_free.argtypes = [c_void_p, c_void_p, c_char_p, c_int]
        lib.ogb_memhost_stats.argtypes = [c_void_p, ctypes.POINTER(c_uint64), c_char_p, c_int]
        lib.ogb_memhost_trim.argtypes = [c_void_p, ctypes.POINTER(c_uint64), c_char_p, c_int]
        lib.ogb_memhost_unload.argtypes = [c_void_p, c_char_p, c_int]
        lib._memhost_bound = True
    return lib


class PluginAllocator:
    def __init__(self, path: str, byte_limit: int = 0, purpose: str = ""):
        self.lib = _lib()
        err = ctypes.create_string_buffer(512)
        self.handle = self.lib.ogb_memhost_load(str(path).encode(), int(byte_limit), purpose.encode() or None, err, len(err))
        if not self.handle:
            raise MemPluginError(err.value.decode(errors="replace") or f"cannot load memory plugin {path}")
        self.path = str(path)
        self.live: dict = {}             # address -> bytes

    @property
    def level(self) -> int:
        return int(self.lib.ogb_memhost_level(self.handle))

    @property
    def name(self) -> str:
        return (self.lib.ogb_memhost_name(self.handle) or b"").decode()

    def allocate(self, nbytes: int, alignment: int = 64) -> int:
        out, err = c_void_p(), ctypes.create_string_buffer(256)
        rc = self.lib.ogb_memhost_alloc(self.handle, int(nbytes), int(alignment), ctypes.byref(out), err, len(err))
        if rc != 0:
            raise MemPluginError(f"plugin '{self.name}' could not allocate {nbytes} bytes: {CODES.get(rc, rc)} ({err.value.decode(errors='replace')})", rc)
        self.live[out.value] = int(nbytes)
        return out.value

    def free(self, address: int) -> None:
        if address not in self.live:
            raise MemPluginError(f"address {address:#x} was not allocated through this plugin (or was freed already)")
        err = ctypes.create_string_buffer(256)
        rc = self.lib.ogb_memhost_free(self.handle, c_void_p(address), err, len(err))
        if rc != 0:
            raise MemPluginError(f"plugin '{self.name}' failed to free {address:#x}: {err.value.decode(errors='replace')}", rc)
        del self.live[address]

    def tensor(self, shape, dtype=torch.float32) -> torch.Tensor:
        """A zero-filled CPU tensor over plugin memory.  Call ``free_tensor`` (or ``close``) when done with it."""
        count = int(np.prod(shape)) if len(shape) else 1
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = max(1, count * item)
        address = self.allocate(nbytes)
        buf = (ctypes.c_uint8 * nbytes).from_address(address)
        t = torch.frombuffer(buf, dtype=torch.uint8, count=count * item).view(dtype).reshape(tuple(shape))
        t.zero_()
        return t

    def free_tensor(self, t: torch.Tensor) -> None:
        self.free(t.data_ptr())

    def stats(self) -> dict:
        out, err = (c_uint64 * 4)(), ctypes.create_string_buffer(256)
        rc = self.lib.ogb_memhost_stats(self.handle, out, err, len(err))
        if rc != 0:
            raise MemPluginError(f"plugin '{self.name}': {err.value.decode(errors='replace')}", rc)
        return {"bytes_in_use": int(out[0]), "bytes_peak": int(out[1]), "allocations_live": int(out[2]), "allocations_total": int(out[3])}

    def trim(self) -> int:
        out, err = c_uint64(), ctypes.create_string_buffer(256)
        rc = self.lib.ogb_memhost_trim(self.handle, ctypes.byref(out), err, len(err))
        if rc != 0:
            raise MemPluginError(f"plugin '{self.name}': {err.value.decode(errors='replace')}", rc)
        return int(out.value)

    def close(self) -> None:
        if not self.handle:
            return
        for address in list(self.live):
            self.free(address)
        err = ctypes.create_string_buffer(256)
        rc = self.lib.ogb_memhost_unload(self.handle, err, len(err))
        if rc != 0:
            raise MemPluginError(f"cannot unload plugin '{self.name}': {err.value.decode(errors='replace')}", rc)
        self.handle = None
