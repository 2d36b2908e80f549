"""Serving one model over a tensor-parallel group through the public API.

Every rank of the group owns an :class:`LLMEngine` over its shard of the weights and runs the same deterministic
scheduler, so the ranks stay in step only if they see the same requests in the same order.  Rank 0 (the *leader*) is the
one a user talks to -- ``Engine.generate``, the HTTP server, the CLI -- and the other ranks *follow*: before each step
the leader broadcasts the commands that changed the scheduler's state since the last one (requests admitted, cancelled,
released) and then every rank steps.  Followers block in the broadcast while the leader is idle, so an idle server costs
no GPU time.

    torchrun --nproc-per-node 4 -m onnx_genai_b200 serve model_dir        # rank 0 serves, ranks 1-3 follow

What a request may use under tensor parallelism is what the device sampler covers (temperature, top-k / top-p / min-p,
stop ids, token budgets): samplers that run on the host, log-probabilities, embeddings and speculative proposers keep
per-rank state the followers do not have, and are refused by the leader with that reason.

(The reference has no multi-GPU path; this is the serving side of the tensor-parallel design in its
docs/research/tensor-parallelism-feasibility.md: one control rank, SPMD workers.)
"""
from __future__ import annotations

import os

import numpy as np
import torch


def bootstrap(device=None):
    """Join the process group the launcher described (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*) and return
    ``(rank, world, device, comm)``: NCCL on GPUs with the fused peer-memory communicator when it can be formed, gloo on
    the CPU (tests).  ``world`` == 1: no group, ``comm`` is None."""
    from ..parallel import comm as comm_mod

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1, torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu")), None
    on_cpu = str(device or "").startswith("cpu") or not torch.cuda.is_available()
    rank, world, local_rank = comm_mod.init_distributed("gloo" if on_cpu else None)
    dev = torch.device("cpu") if on_cpu else torch.device("cuda", local_rank)
    if not on_cpu:
        torch.cuda.set_device(dev)
    comm = comm_mod.NcclComm()
    if not on_cpu and os.environ.get("OGB_TP_FUSED", "1") != "0":
        try:
            from ..parallel.fused import FusedComm

            comm = FusedComm(comm, dev)
        except Exception as exc:            # the NCCL path serves; say why the peer-memory one does not
            if rank == 0:
                import sys

                print(f"fused tensor-parallel communicator unavailable ({exc}); using NCCL", file=sys.stderr)
    return rank, world, dev, comm


class TpControl:
    """Keeps the schedulers of a tensor-parallel group in step (see the module docstring)."""

    def __init__(self, llm, rank: int, world: int, group=None):
        self.llm, self.rank, self.world, self.group = llm, int(rank), int(world), group
        self.pending: list = []
        self.steps = 0
        self.stopped = False

    # -- wire ---------------------------------------------------------------------------------------
    def _exchange(self, cmds):
        import torch.distributed as dist

        box = [cmds if self.rank == 0 else None]
        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    # -- leader -------------------------------------------------------------------------------------
    def install(self) -> None:
        """Rank 0: record what changes the scheduler, and send it ahead of every step."""
        llm, core = self.llm, self.llm.core
        add, step, cancel, release = llm.add_request, llm.step, core.cancel, core.release

        def add_request(prompt_ids, max_new_tokens=256, **kw):
            self.pending.append(("add", np.asarray(prompt_ids, dtype=np.int32).tolist(), int(max_new_tokens), dict(kw)))
            return add(prompt_ids, max_new_tokens, **kw)

        def cancel_(sid):
            self.pending.append(("cancel", int(sid)))
            return cancel(sid)

        def release_(sid):
            self.pending.append(("release", int(sid)))
            return release(sid)

        def step_():
            if self.stopped:
                raise RuntimeError("the tensor-parallel group was shut down")
            cmds, self.pending = self.pending + [("step",)], []
            self._exchange(cmds)
            self.steps += 1
            return step()

        llm.add_request, llm.step, core.cancel, core.release = add_request, step_, cancel_, release_

    def refuse(self, what: str):
        raise ValueError(f"{what} is not available under tensor parallelism: it keeps state on the rank that serves the request, "
                         "which the other ranks do not have; run the model on one GPU for it")

    def shutdown(self) -> None:
        """Rank 0: release the followers (idempotent)."""
        if self.rank == 0 and not self.stopped and self.world > 1:
            self._exchange(self.pending + [("stop",)])
            self.pending = []
        self.stopped = True

    # -- followers ----------------------------------------------------------------------------------
    def follow(self) -> int:
        """Ranks 1..n-1: apply the leader's commands until it says stop; returns the number of steps taken."""
        llm, core = self.llm, self.llm.core
        while True:
            for cmd in self._exchange(None):
                kind = cmd[0]
                if kind == "add":
                    llm.add_request(np.asarray(cmd[1], dtype=np.int32), cmd[2], **cmd[3])
                elif kind == "cancel":
                    core.cancel(cmd[1])
                elif kind == "release":
                    core.release(cmd[1])
                elif kind == "step":
                    llm.step()
                    self.steps += 1
                elif kind == "stop":
                    self.stopped = True
                    return self.steps
                else:
                    raise RuntimeError(f"unknown command {kind!r} from the leader")
