"""Allocator interface of the engine: who hands out the bytes behind KV pools, swap space and scratch, what optional
capabilities an allocator has, and when a released allocation's memory may really go back.

* :class:`Allocator` -- the minimum contract: ``allocate(nbytes, role, tag)`` returns an :class:`Allocation` (a flat byte
  tensor plus its identity and the ledger lease that charged it), ``release`` hands it back.  ``tensor(shape, dtype,
  role, tag)`` is the typed convenience the engine uses.
* capabilities -- ``virtual_backing`` (reserve an address range, back a prefix, grow in place: the CUDA VMM pool) and
  ``device_addressable_host`` (pinned host memory the swap kernels may read and write in place).  Callers ask; an
  allocator that lacks one says so instead of emulating it.
* :class:`DeferredReleaseQueue` -- a release requested while GPU work that may still touch the bytes is in flight is
  parked behind a CUDA event recorded at that moment; ``drain()`` completes the releases whose event has passed.  A
  release that fails is quarantined (kept, counted, never retried blindly) rather than lost.

The reference splits the same ground into its memory-API crate (crates/onnx-runtime-memory-api/src/allocator.rs,
capability.rs, deferred.rs); identity generations there guard against reuse under a live binding, here an allocation's
``generation`` does, checked by :meth:`Allocation.check`.
"""
from __future__ import annotations

import dataclasses
import itertools
import threading

import numpy as np
import torch

from .memory import MemoryLedger

_IDS = itertools.count(1)


class AllocatorError(RuntimeError):
    pass


@dataclasses.dataclass
class Allocation:
    ident: int
    generation: int
    nbytes: int
    role: str
    tier: str
    tag: str
    data: torch.Tensor | None                    # flat uint8 view of the bytes
    lease: object | None = None
    owner: object | None = None                  # the allocator that must release it
    handle: object | None = None                 # allocator-private (a growable buffer, a plugin block)
    released: bool = False

    def check(self) -> "Allocation":
        """Raises when the allocation was released: a stale handle must not reach a kernel."""
        if self.released or self.data is None:
            raise AllocatorError(f"allocation {self.ident} ({self.role}: {self.tag}) was released (generation {self.generation})")
        return self

    def view(self, shape, dtype) -> torch.Tensor:
        self.check()
        n = int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()
        if n > self.nbytes:
            raise AllocatorError(f"view of {n} bytes over an allocation of {self.nbytes}")
        return self.data[:n].view(dtype).reshape(tuple(shape))


class Allocator:
    """Base class: accounting against a ledger, identity, the release bookkeeping.  Subclasses provide the bytes."""

    tier = "host"
    virtual_backing = False
    device_addressable_host = False

    def __init__(self, ledger: MemoryLedger | None = None):
        self.ledger = ledger
        self.live: dict = {}
        self.allocated_bytes = 0
        self.peak_bytes = 0
        self.lock = threading.Lock()

    # -- to implement ---------------------------------------------------------------------------------
    def _obtain(self, nbytes: int, role: str, tag: str):
        raise NotImplementedError

    def _dispose(self, alloc: Allocation) -> None:
        alloc.data = None
        alloc.handle = None

    # -- contract -------------------------------------------------------------------------------------
    def allocate(self, nbytes: int, role: str = "workspace", tag: str = "") -> Allocation:
        nbytes = int(nbytes)
        if nbytes < 0:
            raise AllocatorError(f"negative size {nbytes}")
        lease = self.ledger.lease(role, self.tier, nbytes, tag) if self.ledger is not None else None
        try:
            data, handle = self._obtain(nbytes, role, tag)
        except Exception:
            if lease is not None:
                lease.release()
            raise
        a = Allocation(next(_IDS), 1, nbytes, role, self.tier, tag, data, lease, self, handle)
        with self.lock:
            self.live[a.ident] = a
            self.allocated_bytes += nbytes
            self.peak_bytes = max(self.peak_bytes, self.allocated_bytes)
        return a

    def tensor(self, shape, dtype, role: str = "workspace", tag: str = "") -> torch.Tensor:
        """A zero-filled typed tensor; the allocation rides on it as ``tensor.ogb_allocation``."""
        n = int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()
        a = self.allocate(n, role, tag)
        t = a.view(shape, dtype)
        t.zero_()
        t.ogb_allocation = a
        return t

    def release(self, alloc: Allocation) -> None:
        if alloc.owner is not self:
            raise AllocatorError(f"allocation {alloc.ident} belongs to another allocator")
        with self.lock:
            if alloc.released:
                raise AllocatorError(f"allocation {alloc.ident} ({alloc.tag}) released twice")
            alloc.released = True
            alloc.generation += 1
            self.live.pop(alloc.ident, None)
            self.allocated_bytes -= alloc.nbytes
        try:
            self._dispose(alloc)
        finally:
            if alloc.lease is not None:
                alloc.lease.release()

    def stats(self) -> dict:
        return {"kind": type(self).__name__, "tier": self.tier, "live": len(self.live), "allocated_bytes": self.allocated_bytes,
                "peak_bytes": self.peak_bytes, "virtual_backing": self.virtual_backing,
                "device_addressable_host": self.device_addressable_host}


class TorchAllocator(Allocator):
    """Bytes from torch's caching allocator on ``device`` (or plain host memory for the CPU device)."""

    def __init__(self, device, ledger=None):
        super().__init__(ledger)
        self.device = torch.device(device)
        self.tier = "vram" if self.device.type == "cuda" else "host"

    def _obtain(self, nbytes, role, tag):
        return torch.empty(nbytes, dtype=torch.uint8, device=self.device), None


class PinnedHostAllocator(Allocator):
    """Page-locked host memory: the device reads and writes it in place (swap space, weight packs)."""

    tier = "host"

    def __init__(self, ledger=None, pin: bool | None = None):
        super().__init__(ledger)
        self.pin = torch.cuda.is_available() if pin is None else bool(pin)
        self.device_addressable_host = self.pin

    def _obtain(self, nbytes, role, tag):
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.pin), None


class VmmAllocator(Allocator):
    """CUDA virtual-memory pool: ``allocate`` reserves ``reserve_factor`` times the request as address space and backs the
    request; :meth:`grow` backs more of the range in place (addresses never move)."""

    tier = "vram"
    virtual_backing = True

    def __init__(self, device, ledger=None, reserve_factor: float = 4.0):
        super().__init__(ledger)
        self.device = torch.device(device)
        self.reserve_factor = float(reserve_factor)

    def _obtain(self, nbytes, role, tag):
        from ..utils.vmm import GrowableBuffer

        buf = GrowableBuffer(int(nbytes * self.reserve_factor), self.device.index or 0, nbytes)
        return buf.view(torch.uint8)[:nbytes], buf

    def grow(self, alloc: Allocation, nbytes: int) -> Allocation:
        alloc.check()
        if nbytes <= alloc.nbytes:
            return alloc
        if alloc.lease is not None:
            self.ledger.resize(alloc.lease, nbytes)      # refuses before any page is mapped
        alloc.handle.grow(nbytes)
        with self.lock:
            self.allocated_bytes += nbytes - alloc.nbytes
            self.peak_bytes = max(self.peak_bytes, self.allocated_bytes)
        alloc.nbytes = nbytes
        alloc.data = alloc.handle.view(torch.uint8)[:nbytes]
        return alloc

    def _dispose(self, alloc):
        buf = alloc.handle
        super()._dispose(alloc)
        if buf is not None and hasattr(buf, "close"):
            buf.close()


@dataclasses.dataclass
class _Pending:
    alloc: Allocation
    event: object | None
    reason: str


class DeferredReleaseQueue:
    """Releases that must wait for the GPU.  ``enqueue`` records an event on ``stream`` (the work submitted so far may
    still read or write the bytes) and parks the allocation; ``drain`` releases those whose event has completed;
    ``flush`` waits for all of them.  An allocation whose release raises is quarantined: it stays accounted for under
    ``quarantined`` with the error, so the bytes are visible instead of silently leaked or double-freed."""

    def __init__(self):
        self.pending: list = []
        self.quarantined: list = []
        self.released = 0
        self.lock = threading.Lock()

    def enqueue(self, alloc: Allocation, stream=None, reason: str = "") -> None:
        alloc.check()
        event = None
        if alloc.tier == "vram" or (stream is not None):
            if torch.cuda.is_available():
                event = torch.cuda.Event()
                event.record(stream if stream is not None else torch.cuda.current_stream())
        with self.lock:
            if any(p.alloc is alloc for p in self.pending):
                raise AllocatorError(f"allocation {alloc.ident} ({alloc.tag}) is already waiting for release")
            self.pending.append(_Pending(alloc, event, reason))

    @property
    def pending_bytes(self) -> int:
        return sum(p.alloc.nbytes for p in self.pending)

    def _finish(self, p: _Pending) -> None:
        try:
            p.alloc.owner.release(p.alloc)
            self.released += 1
        except Exception as exc:                        # keep the evidence; do not retry blindly
            self.quarantined.append((p.alloc, repr(exc)))

    def drain(self) -> int:
        """Release what the GPU is done with; returns how many allocations went back."""
        with self.lock:
            ready = [p for p in self.pending if p.event is None or p.event.query()]
            self.pending = [p for p in self.pending if p not in ready]
        for p in ready:
            self._finish(p)
        return len(ready)

    def flush(self) -> int:
        with self.lock:
            todo, self.pending = self.pending, []
        for p in todo:
            if p.event is not None:
                p.event.synchronize()
            self._finish(p)
        return len(todo)

    def stats(self) -> dict:
        return {"pending": len(self.pending), "pending_bytes": self.pending_bytes, "released": self.released,
                "quarantined": len(self.quarantined), "quarantined_bytes": sum(a.nbytes for a, _ in self.quarantined)}
