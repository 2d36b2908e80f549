"""CPU oracle communicator: ranks are threads of one process sharing host memory.

Counterpart of the reference's `InProcessCommunicator`, `CollectiveSequencer` and
`OwnershipRegistry` (crates/onnx-runtime-comm/src/inprocess.rs:133-1160, ordering.rs:60-445,
registry.rs): the oracle every device backend is checked against, and the vehicle for the
failure tests that must not touch a GPU.

* Reductions run in fixed rank order with per-step rounding to the tensor's dtype
  (reduction.rs:7-143), so results are bit-exact and independent of thread timing.
* Every collective carries a `(execution, sequence)` instance id; the sequencer admits an
  instance only when every rank presents the same op, dtype, element count and membership hash
  (FNV-1a) for the same slot, otherwise the group aborts with a description of the mismatch.
* `abort(cause)` is idempotent, wakes every waiter with a terminal error and closes the epoch;
  waits carry a timeout so a rank that never arrives ends the collective instead of hanging.
* Buffers handed to a collective are leased (read or write) until the instance is terminal; a
  second conflicting lease is an error.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass

import torch


class CommAborted(RuntimeError):
    pass


class CollectiveMismatch(RuntimeError):
    pass


class LeaseConflict(RuntimeError):
    pass


def membership_hash(members) -> int:
    h = 0xCBF29CE484222325
    for m in members:
        for b in int(m).to_bytes(8, "little"):
            h ^= b
            h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


@dataclass(frozen=True)
class CommInstanceId:
    execution: int
    sequence: int


class OwnershipRegistry:
    """Read / write leases on buffers (by storage address) held until a collective instance is terminal."""

    def __init__(self):
        self.lock = threading.Lock()
        self.leases: dict = {}   # key -> (mode, set(instance))

    def acquire(self, key, mode: str, instance):
        with self.lock:
            cur = self.leases.get(key)
            if cur is None:
                self.leases[key] = (mode, {instance})
            elif cur[0] == "read" and mode == "read":
                cur[1].add(instance)
            elif instance in cur[1] and cur[0] == mode:
                pass
            else:
                raise LeaseConflict(f"buffer {key:#x} is leased for {cur[0]} by {sorted(map(str, cur[1]))}; "
                                    f"cannot lease it for {mode} to {instance} until those instances finish")

    def release(self, key, instance):
        with self.lock:
            cur = self.leases.get(key)
            if cur is not None:
                cur[1].discard(instance)
                if not cur[1]:
                    del self.leases[key]


class _Group:
    def __init__(self, world, timeout):
        self.world, self.timeout = world, timeout
        self.cv = threading.Condition()
        self.slots: dict = {}       # instance -> {"desc":..., "bufs": {rank: tensor}, "done": int, "result": ...}
        self.aborted: str | None = None
        self.epoch = 0
        self.log: list = []         # canonical slot log (instance, op) in admission order
        self.registry = OwnershipRegistry()
        self.members = tuple(range(world))
        self.hash = membership_hash(self.members)
        self.mail: dict = {}        # (src, dst) -> list of tensors in send order (point-to-point)
        self.split_lists: dict = {} # sequence number -> {rank: send counts} of a variable-size exchange in flight


class InProcessCommunicator:
    backend_name = "inprocess"

    def __init__(self, group: _Group, rank: int):
        self.g, self.rank, self.world = group, rank, group.world
        self._seq = 0
        self.execution = 0

    @staticmethod
    def create_group(world: int, timeout: float = 5.0):
        g = _Group(world, timeout)
        return [InProcessCommunicator(g, r) for r in range(world)]

    # -- failure handling -------------------------------------------------------------------
    def abort(self, cause: str):
        with self.g.cv:
            if self.g.aborted is None:
                self.g.aborted = cause
            self.g.cv.notify_all()

    def restart(self):
        """Whole-group restart into a new topology epoch (all ranks must call it)."""
        with self.g.cv:
            self.g.aborted = None
            self.g.slots.clear()
            self.g.epoch += 1
        self._seq = 0

    def _next_instance(self):
        self._seq += 1
        return CommInstanceId(self.execution, self._seq)

    def _rendezvous(self, op, tensor, extra, compute):
        inst = self._next_instance()
        g = self.g
        # variable-size exchanges agree on everything but the element count, which each rank states in its split list
        desc = (op, str(tensor.dtype), -1 if op == "all_to_all_v" else tensor.numel(), g.hash, None if op == "all_to_all_v" else extra)
        key = tensor.untyped_storage().data_ptr() + tensor.storage_offset() * tensor.element_size()
        with g.cv:
            if g.aborted is not None:
                raise CommAborted(f"communicator aborted: {g.aborted}")
            slot = g.slots.get(inst)
            if slot is None:
                slot = {"desc": desc, "bufs": {}, "done": 0, "result": None, "first": self.rank}
                g.slots[inst] = slot
                g.log.append((inst, op))
            elif slot["desc"] != desc:
                g.aborted = (f"collective mismatch at {inst}: rank {slot['first']} issued {slot['desc'][:3]} but rank "
                             f"{self.rank} issued {desc[:3]}; every rank must issue the same collective in the same slot")
                g.cv.notify_all()
                raise CollectiveMismatch(g.aborted)
            g.registry.acquire(key, "write", (inst, self.rank))
            slot["bufs"][self.rank] = tensor
            if len(slot["bufs"]) == g.world:
                slot["result"] = compute(slot["bufs"])
                g.cv.notify_all()
            else:
                ok = g.cv.wait_for(lambda: slot["result"] is not None or g.aborted is not None, timeout=g.timeout)
                if g.aborted is not None:
                    g.registry.release(key, (inst, self.rank))
                    raise CommAborted(f"communicator aborted: {g.aborted}")
                if not ok:
                    g.aborted = (f"{op} at {inst} timed out after {g.timeout}s: ranks "
                                 f"{sorted(set(range(g.world)) - set(slot['bufs']))} never joined")
                    g.cv.notify_all()
                    g.registry.release(key, (inst, self.rank))
                    raise CommAborted(g.aborted)
            res = slot["result"]
            slot["done"] += 1
            if slot["done"] == g.world:
                del g.slots[inst]
            g.registry.release(key, (inst, self.rank))
        return res

    # -- collectives ------------------------------------------------------------------------
    @staticmethod
    def _reduce(bufs, op="sum"):
        ranks = sorted(bufs)
        acc = bufs[ranks[0]].clone()
        for r in ranks[1:]:             # fixed rank order, rounding to dtype after every step
            if op == "sum":
                acc = (acc.float() + bufs[r].float()).to(acc.dtype) if acc.dtype in (torch.bfloat16, torch.float16) else acc + bufs[r]
            elif op == "max":
                acc = torch.maximum(acc, bufs[r])
            elif op == "min":
                acc = torch.minimum(acc, bufs[r])
            elif op == "product":
                acc = acc * bufs[r]
        return acc

    def all_reduce(self, t, op="sum"):
        res = self._rendezvous("all_reduce", t, op, lambda bufs: self._reduce(bufs, op))
        t.copy_(res)
        return t

    def reduce_scatter(self, out, t, op="sum"):
        res = self._rendezvous("reduce_scatter", t, op, lambda bufs: self._reduce(bufs, op))
        out.copy_(res.reshape(self.world, -1)[self.rank].view_as(out))
        return out

    def all_gather(self, out, t):
        res = self._rendezvous("all_gather", t, None, lambda bufs: torch.cat([bufs[r].reshape(-1) for r in sorted(bufs)]))
        out.copy_(res.view_as(out))
        return out

    def broadcast(self, t, src=0):
        res = self._rendezvous("broadcast", t, src, lambda bufs: bufs[src].clone())
        t.copy_(res)
        return t

    def all_to_all(self, out, t):
        def compute(bufs):
            parts = {r: bufs[r].reshape(self.world, -1) for r in bufs}
            return {dst: torch.cat([parts[src][dst] for src in sorted(parts)]) for dst in range(self.world)}

        res = self._rendezvous("all_to_all", t, None, compute)
        out.copy_(res[self.rank].view_as(out))
        return out

    def all_to_all_v(self, t, send_counts, recv_counts=None):
        """Variable-size exchange of rows: the first ``send_counts[0]`` rows of ``t`` go to rank 0, the next
        ``send_counts[1]`` to rank 1, ...  Returns the rows received, ordered by source rank.  ``recv_counts`` (from
        :meth:`exchange_counts`) is checked when given."""
        send_counts = [int(c) for c in send_counts]
        if len(send_counts) != self.world or sum(send_counts) != t.shape[0]:
            raise ValueError(f"send_counts {send_counts} must have one entry per rank and sum to the {t.shape[0]} rows sent")
        width = tuple(t.shape[1:])

        def compute(bufs):
            counts = bufs["counts"]
            out = {}
            for dst in range(self.world):
                parts = []
                for src in sorted(r for r in bufs if r != "counts"):
                    lo = sum(counts[src][:dst])
                    parts.append(bufs[src][lo:lo + counts[src][dst]])
                out[dst] = torch.cat(parts) if parts else t.new_zeros((0,) + width)
            return out

        g, seq = self.g, self._seq + 1
        with g.cv:                                   # every rank files its split list before it joins the rendezvous
            g.split_lists.setdefault(seq, {})[self.rank] = send_counts

        def wrapped(bufs):
            merged = dict(bufs)
            merged["counts"] = g.split_lists.pop(seq)
            return compute(merged)

        res = self._rendezvous("all_to_all_v", t, width, wrapped)[self.rank].clone()
        if recv_counts is not None and sum(int(c) for c in recv_counts) != res.shape[0]:
            raise ValueError(f"received {res.shape[0]} rows but recv_counts {list(recv_counts)} announce {sum(recv_counts)}")
        return res

    def send(self, t, dst: int):
        """Point-to-point: hand a copy of ``t`` to rank ``dst`` (matched with its ``recv`` in order)."""
        g = self.g
        with g.cv:
            if g.aborted is not None:
                raise CommAborted(f"communicator aborted: {g.aborted}")
            g.mail.setdefault((self.rank, int(dst)), []).append(t.detach().clone())
            g.cv.notify_all()

    def recv(self, t, src: int):
        g = self.g
        key = (int(src), self.rank)
        with g.cv:
            ok = g.cv.wait_for(lambda: g.mail.get(key) or g.aborted is not None, timeout=g.timeout)
            if g.aborted is not None:
                raise CommAborted(f"communicator aborted: {g.aborted}")
            if not ok:
                g.aborted = f"recv on rank {self.rank} from rank {src} timed out after {g.timeout}s: nothing was sent"
                g.cv.notify_all()
                raise CommAborted(g.aborted)
            msg = g.mail[key].pop(0)
        if msg.shape != t.shape or msg.dtype != t.dtype:
            raise CollectiveMismatch(f"rank {src} sent {tuple(msg.shape)} {msg.dtype} but rank {self.rank} expected {tuple(t.shape)} {t.dtype}")
        t.copy_(msg)
        return t

    def exchange_counts(self, counts):
        """counts[dst] = rows this rank sends to dst; returns rows received from each source."""
        t = torch.as_tensor(counts, dtype=torch.int64)
        out = torch.empty_like(t)
        return self.all_to_all(out, t).tolist()

    def barrier(self):
        self._rendezvous("barrier", torch.zeros(1), None, lambda bufs: torch.zeros(1))

    def min_int(self, v):
        t = torch.tensor([v], dtype=torch.int64)
        return int(self.all_reduce(t, "min").item())

    def max_float(self, v):
        t = torch.tensor([v], dtype=torch.float64)
        return float(self.all_reduce(t, "max").item())
