"""Communicator used by the tensor/expert-parallel executor.

API shape follows the reference's `Communicator` trait (crates/onnx-runtime-comm/src/
communicator.rs:32-160: all_reduce, all_gather, reduce_scatter, broadcast, all_to_all, barrier,
abort; identity rank/world/backend_name).  Backends:

* :class:`NcclComm`   -- torch.distributed over NCCL.  This is the labelled *baseline* path.
* :class:`FusedComm`  -- (parallel/fused.py) peer-memory kernels that overlap the collective with
                         the GEMM; falls back to NCCL for ops it does not cover.
* :class:`LocalComm`  -- world of one; every collective is the identity.
* the CPU oracle lives in parallel/oracle.py (threads in one process, bit-exact reductions).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


class LocalComm:
    backend_name = "local"
    rank, world = 0, 1

    def all_reduce(self, t):
        return t

    def broadcast(self, t, src=0):
        return t

    def all_gather(self, out, t):
        out.copy_(t.view_as(out))
        return out

    def reduce_scatter(self, out, t):
        out.copy_(t.view_as(out))
        return out

    def all_to_all(self, out, t, out_splits=None, in_splits=None):
        out.copy_(t.view_as(out))
        return out

    def exchange_counts(self, counts):
        return [int(c) for c in counts]

    def all_to_all_v(self, t, send_counts, recv_counts=None):
        return t.clone()

    def send(self, t, dst: int):
        raise RuntimeError("a world of one has no peer to send to")

    def recv(self, t, src: int):
        raise RuntimeError("a world of one has no peer to receive from")

    def abort(self, cause: str):
        pass

    def barrier(self):
        pass

    def min_int(self, v: int) -> int:
        return v

    def max_float(self, v: float) -> float:
        return v


class NcclComm:
    """Plain library collectives (the baseline the fused kernels are measured against)."""

    backend_name = "nccl"

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.calls = 0
        # the same class drives gloo ranks on CPU, which is how the multi-rank host logic (sharding, replica
        # scheduling, row-split sampling) is tested without GPUs
        self.backend_name = dist.get_backend(group)
        self._scalar_device = "cuda" if self.backend_name == "nccl" else "cpu"

    def all_reduce(self, t):
        from .. import ops

        with ops.timed_region("nccl_all_reduce"):
            dist.all_reduce(t, group=self.group)
        self.calls += 1
        return t

    def broadcast(self, t, src=0):
        """``src`` is a rank of this communicator's group (not a global rank)."""
        dist.broadcast(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
        return t

    def all_gather(self, out, t):
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out

    def reduce_scatter(self, out, t):
        dist.reduce_scatter_tensor(out, t, group=self.group)
        return out

    def all_to_all(self, out, t, out_splits=None, in_splits=None):
        dist.all_to_all_single(out, t, out_splits, in_splits, group=self.group)
        return out

    def exchange_counts(self, counts):
        """counts[dst] = rows this rank sends to dst; returns the rows each source sends here."""
        t = torch.tensor([int(c) for c in counts], dtype=torch.int64, device=self._scalar_device)
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t, group=self.group)
        return out.tolist()

    def all_to_all_v(self, t, send_counts, recv_counts=None):
        """Variable-size row exchange (expert-parallel dispatch and combine): rows of ``t`` are grouped by destination
        rank in rank order; returns the rows received, grouped by source rank."""
        send_counts = [int(c) for c in send_counts]
        if recv_counts is None:
            recv_counts = self.exchange_counts(send_counts)
        recv_counts = [int(c) for c in recv_counts]
        out = t.new_empty((sum(recv_counts),) + tuple(t.shape[1:]))
        dist.all_to_all_single(out, t.contiguous(), recv_counts, send_counts, group=self.group)
        return out

    def send(self, t, dst: int):
        dist.send(t, dst=dist.get_global_rank(self.group, dst) if self.group is not None else dst, group=self.group)

    def recv(self, t, src: int):
        dist.recv(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
        return t

    def abort(self, cause: str):
        """End the group's outstanding and future collectives with an error on this rank (peers reach their timeout)."""
        self.aborted = cause
        try:
            backend = self.group._get_backend(torch.device(self._scalar_device)) if self.group is not None else \
                dist.distributed_c10d._get_default_group()._get_backend(torch.device(self._scalar_device))
            if hasattr(backend, "abort"):
                backend.abort()
        except Exception:
            pass

    def barrier(self):
        dist.barrier(group=self.group)

    def min_int(self, v: int) -> int:
        t = torch.tensor([v], dtype=torch.int64, device=self._scalar_device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return int(t.item())

    def max_float(self, v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=self._scalar_device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())


def init_distributed(backend: str | None = None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (torchrun); returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        return 0, 1, 0
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, world, local_rank
