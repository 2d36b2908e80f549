"""Memory ledger: who holds how many bytes in which tier, and what the limits leave for the KV pool.

The reference keeps a process-wide governor with leases per role (weights, KV, activations, ...) and per tier (VRAM,
host, disk) so that capacity decisions -- how large the KV pool may be, whether a model may be loaded, what an
overload error should say -- come from one set of numbers (crates/onnx-runtime-memory-governor/src/lib.rs,
manager.rs; the serving limits `--vram-limit 8GiB|0.9|auto` and `--host-ram-limit`,
crates/onnx-genai-server/src/runtime_args.rs:32-74).  This is that ledger for the engine here: bytes are
authoritative (taken from the tensors that were actually allocated), leases are released when their owner goes away,
and a limit that cannot be met is an error that names the shortfall.
"""
from __future__ import annotations

import re
import threading
from dataclasses import dataclass, field

TIERS = ("vram", "host", "disk")
ROLES = ("weights", "kv", "activations", "workspace", "comm", "kv_offload")
_UNITS = {"": 1, "b": 1, "k": 1 << 10, "kb": 1 << 10, "kib": 1 << 10, "m": 1 << 20, "mb": 1 << 20, "mib": 1 << 20,
          "g": 1 << 30, "gb": 1 << 30, "gib": 1 << 30, "t": 1 << 40, "tb": 1 << 40, "tib": 1 << 40}


class MemoryLimitError(RuntimeError):
    pass


def parse_limit(text, total_bytes: int | None = None) -> int | None:
    """``"auto"`` / ``None`` -> no explicit limit; ``"0.9"`` -> that fraction of ``total_bytes``; ``"8GiB"``,
    ``"512MB"``, ``"1073741824"`` -> bytes."""
    if text is None:
        return None
    t = str(text).strip().lower()
    if t in ("", "auto", "none"):
        return None
    m = re.fullmatch(r"([0-9]*\.?[0-9]+)\s*([a-z]*)", t)
    if not m or m.group(2) not in _UNITS:
        raise ValueError(f"cannot read memory limit {text!r}; use a fraction (0.9), bytes, or a size such as 8GiB")
    value, unit = float(m.group(1)), m.group(2)
    if unit == "" and value <= 1.0:
        if total_bytes is None:
            raise ValueError(f"memory limit {text!r} is a fraction but the tier's total size is unknown; give bytes")
        return int(value * total_bytes)
    return int(value * _UNITS[unit])


@dataclass
class Lease:
    ledger: "MemoryLedger"
    role: str
    tier: str
    nbytes: int
    tag: str = ""
    released: bool = False

    def release(self) -> None:
        self.ledger.release(self)

    def resize(self, nbytes: int) -> None:
        self.ledger.resize(self, nbytes)


@dataclass
class MemoryLedger:
    limits: dict = field(default_factory=dict)          # tier -> bytes | None
    leases: list = field(default_factory=list)
    lock: threading.Lock = field(default_factory=threading.Lock)
    peak: dict = field(default_factory=dict)

    def used(self, tier: str, role: str | None = None) -> int:
        return sum(l.nbytes for l in self.leases if l.tier == tier and (role is None or l.role == role))

    def available(self, tier: str) -> int | None:
        limit = self.limits.get(tier)
        return None if limit is None else max(0, limit - self.used(tier))

    def lease(self, role: str, tier: str, nbytes: int, tag: str = "") -> Lease:
        if role not in ROLES or tier not in TIERS:
            raise ValueError(f"unknown role/tier {role!r}/{tier!r}; roles: {ROLES}, tiers: {TIERS}")
        with self.lock:
            limit = self.limits.get(tier)
            if limit is not None and self.used(tier) + nbytes > limit:
                raise MemoryLimitError(
                    f"{role} ({tag or 'untagged'}) needs {nbytes / 2**30:.2f} GiB of {tier} but only "
                    f"{max(0, limit - self.used(tier)) / 2**30:.2f} GiB remain under the {limit / 2**30:.2f} GiB limit "
                    f"(in use: " + ", ".join(f"{r} {self.used(tier, r) / 2**30:.2f}" for r in ROLES if self.used(tier, r)) +
                    "); raise the limit, shrink the KV pool or unload a model")
            l = Lease(self, role, tier, int(nbytes), tag)
            self.leases.append(l)
            self.peak[tier] = max(self.peak.get(tier, 0), self.used(tier))
            return l

    def release(self, lease: Lease) -> None:
        with self.lock:
            if not lease.released:
                lease.released = True
                self.leases.remove(lease)

    def resize(self, lease: Lease, nbytes: int) -> None:
        with self.lock:
            limit = self.limits.get(lease.tier)
            others = self.used(lease.tier) - lease.nbytes
            if limit is not None and others + nbytes > limit:
                raise MemoryLimitError(f"{lease.role} ({lease.tag}) cannot grow to {nbytes / 2**30:.2f} GiB: the {lease.tier} limit of "
                                       f"{limit / 2**30:.2f} GiB leaves {max(0, limit - others) / 2**30:.2f} GiB")
            lease.nbytes = int(nbytes)
            self.peak[lease.tier] = max(self.peak.get(lease.tier, 0), self.used(lease.tier))

    def kv_budget(self, tier: str = "vram", reserve: int = 0) -> int | None:
        """Bytes the KV pool may take: what the limit leaves after everything already leased and ``reserve``."""
        avail = self.available(tier)
        return None if avail is None else max(0, avail - reserve)

    def snapshot(self) -> dict:
        out = {}
        for tier in TIERS:
            roles = {r: self.used(tier, r) for r in ROLES if self.used(tier, r)}
            if roles or self.limits.get(tier) is not None:
                out[tier] = {"limit_bytes": self.limits.get(tier), "used_bytes": self.used(tier), "peak_bytes": self.peak.get(tier, 0),
                             "by_role": roles}
        return out


def tensor_bytes(obj) -> int:
    """Bytes of every distinct tensor storage reachable from a (nested) object's attributes, lists and dicts."""
    import torch

    seen, total, stack = set(), 0, [obj]
    visited = set()
    while stack:
        o = stack.pop()
        if id(o) in visited:
            continue
        visited.add(id(o))
        if isinstance(o, torch.Tensor):
            key = o.untyped_storage().data_ptr()
            if key not in seen:
                seen.add(key)
                total += o.untyped_storage().nbytes()
        elif isinstance(o, (list, tuple)):
            stack.extend(o)
        elif isinstance(o, dict):
            stack.extend(o.values())
        elif hasattr(o, "__dict__") and not isinstance(o, type):
            stack.extend(vars(o).values())
    return total


# ---------------------------------------------------------------------------------------------
# ticketed, non-blocking pressure protocol for a shared tier (host memory)
# ---------------------------------------------------------------------------------------------
class PressureTicket:
    """A request for bytes that could not be granted at once.  ``poll()`` never blocks and holds no ledger lock;
    ``wait(timeout)`` sleeps on the ticket's own event.  A grant is published only after the bytes have been charged to
    the ticket's lease, so nobody can take them in between.  Dropping or cancelling a ticket gives back whatever it held."""

    PENDING, GRANTED, CANCELLED, EXPIRED = "pending", "granted", "cancelled", "expired"

    def __init__(self, queue: "PressureQueue", role: str, nbytes: int, tag: str, deadline: float | None):
        self.queue, self.role, self.nbytes, self.tag, self.deadline = queue, role, int(nbytes), tag, deadline
        self.state = self.PENDING
        self.lease: Lease | None = None
        self._event = threading.Event()
        self.id = -1

    def poll(self) -> str:
        self.queue._expire()
        return self.state

    def wait(self, timeout: float | None = None) -> str:
        import time

        end = None if timeout is None else time.monotonic() + timeout
        while self.poll() == self.PENDING:
            remaining = None if end is None else end - time.monotonic()
            if remaining is not None and remaining <= 0:
                break
            step = 0.05 if remaining is None else min(0.05, remaining)
            self._event.wait(step)                 # woken by a grant or a cancellation; the short step notices deadlines
        return self.state

    def cancel(self) -> None:
        self.queue.cancel(self)

    def __del__(self):
        try:
            if self.state == self.PENDING:
                self.queue.cancel(self)
        except Exception:
            pass


class PressureQueue:
    """First-come, first-served admission to one tier of a :class:`MemoryLedger` under pressure.

    ``request`` charges the bytes at once when they fit and nobody is waiting ahead; otherwise it files a ticket.  Every
    ``release`` (or cancellation, or expiry) re-examines the queue head: while the head fits it is charged and then
    woken.  A large request at the head is not overtaken by smaller later ones, so it cannot starve.  No method waits
    while holding the lock.  Same contract as the reference's host-memory pressure protocol (charge before wake, waits
    hold no governor lock, cancellation is lossless; crates/onnx-genai-scheduler/src/pressure.rs:1-30)."""

    def __init__(self, ledger: MemoryLedger, tier: str = "host", reclaim=None):
        """``reclaim(nbytes) -> bytes freed``: optional callback asked to give memory back (evict a cache) before a request
        has to queue; called without the queue lock held."""
        if tier not in TIERS:
            raise ValueError(f"unknown tier {tier!r}")
        self.ledger, self.tier, self.reclaim = ledger, tier, reclaim
        self.lock = threading.Lock()
        self.waiting: list = []
        self.next_id = 0
        self.events: list = []          # (sequence, kind, ticket id, bytes): a replayable trace of the linearisation points

    def _log(self, kind, ticket):
        self.events.append((len(self.events), kind, ticket.id, ticket.nbytes))

    def _try_charge(self, ticket) -> bool:
        try:
            ticket.lease = self.ledger.lease(ticket.role, self.tier, ticket.nbytes, ticket.tag)
        except MemoryLimitError:
            return False
        return True

    def request(self, role: str, nbytes: int, tag: str = "", timeout: float | None = None) -> PressureTicket:
        import time

        ticket = PressureTicket(self, role, nbytes, tag, None if timeout is None else time.monotonic() + timeout)
        limit = self.ledger.limits.get(self.tier)
        if limit is not None and nbytes > limit:
            raise MemoryLimitError(f"{role} ({tag or 'untagged'}) asks for {nbytes / 2**30:.2f} GiB of {self.tier}, more than the whole "
                                   f"{limit / 2**30:.2f} GiB limit: it could never be granted")
        if self.reclaim is not None:
            avail = self.ledger.available(self.tier)
            if avail is not None and avail < nbytes:
                self.reclaim(nbytes - avail)
        with self.lock:
            ticket.id = self.next_id
            self.next_id += 1
            self._log("request", ticket)
            if not self.waiting and self._try_charge(ticket):
                ticket.state = PressureTicket.GRANTED
                self._log("grant", ticket)
                ticket._event.set()
            else:
                self.waiting.append(ticket)
        return ticket

    def _pump(self) -> None:
        woken = []
        with self.lock:
            while self.waiting and self._try_charge(self.waiting[0]):
                t = self.waiting.pop(0)
                t.state = PressureTicket.GRANTED          # charged first, published second, woken last
                self._log("grant", t)
                woken.append(t)
        for t in woken:
            t._event.set()

    def release(self, ticket_or_lease) -> None:
        """Give back a granted ticket's (or any lease's) bytes and serve the queue."""
        lease = ticket_or_lease.lease if isinstance(ticket_or_lease, PressureTicket) else ticket_or_lease
        if lease is not None:
            lease.release()
        self._pump()

    def cancel(self, ticket: PressureTicket) -> None:
        with self.lock:
            if ticket.state == PressureTicket.PENDING:
                ticket.state = PressureTicket.CANCELLED
                if ticket in self.waiting:
                    self.waiting.remove(ticket)
                self._log("cancel", ticket)
            elif ticket.state == PressureTicket.GRANTED and ticket.lease is not None and not ticket.lease.released:
                pass                                   # a granted ticket is given back with release(), not cancel()
        ticket._event.set()
        self._pump()                                   # the head may have been what blocked the others

    def _expire(self) -> None:
        import time

        now, expired = time.monotonic(), []
        with self.lock:
            for t in list(self.waiting):
                if t.deadline is not None and now >= t.deadline:
                    t.state = PressureTicket.EXPIRED
                    self.waiting.remove(t)
                    self._log("expire", t)
                    expired.append(t)
        for t in expired:
            t._event.set()
        if expired:
            self._pump()
