"""Token-sharded expert parallelism: dispatch tokens to the ranks that own their experts, combine the results back.

Each rank holds a slice of the tokens and a contiguous block of the experts.  For every (token, chosen expert) pair the
token's hidden row travels to the expert's owner, the owner runs its experts on what it received, and the outputs
travel back to be summed with the router weights.  The exchange is the reference's contract for expert parallelism --
``exchange_counts`` then ``all_to_all_v``, with the inverse permutation owned by the routing plan
(crates/onnx-runtime-comm/src/communicator.rs:77-94; docs/quantization/MOE_EXPERT_PARALLELISM.md:60-100) -- over any
communicator of this package: the CPU oracle in tests, ``torch.distributed`` (gloo / NCCL) across processes.

This is the library form.  The serving engine keeps activations replicated across the tensor-parallel group (every
rank already has every token after the attention block's exchange), so its MoE layers need no dispatch and combine over
the fused exchange kernel instead (``models/moe.py``); this module serves deployments that shard tokens (data-parallel
attention with expert-parallel MLPs).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class RoutingPlan:
    order: torch.Tensor        # [T*k] positions of the (token, slot) pairs sorted by (destination rank, expert)
    send_counts: list          # rows to each rank
    recv_counts: list          # rows from each rank
    recv_experts: torch.Tensor # [R] local expert index of every received row
    tokens: int
    top_k: int


class EpDispatcher:
    def __init__(self, comm, num_experts: int):
        self.comm = comm
        self.world, self.rank = comm.world, comm.rank
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not split evenly over {self.world} ranks")
        self.num_experts, self.per_rank = num_experts, num_experts // self.world

    def owner(self, expert_ids: torch.Tensor) -> torch.Tensor:
        return expert_ids // self.per_rank

    def plan(self, expert_ids: torch.Tensor) -> RoutingPlan:
        """``expert_ids`` [T, k] int: the experts chosen for this rank's tokens."""
        t, k = expert_ids.shape
        flat = expert_ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                 # experts are blocked by rank, so this sorts by rank too
        dst = self.owner(flat[order])
        send_counts = torch.bincount(dst, minlength=self.world).tolist()
        recv_counts = self.comm.exchange_counts(send_counts)
        recv_experts = self.comm.all_to_all_v((flat[order] % self.per_rank).to(torch.int64).reshape(-1, 1), send_counts, recv_counts).reshape(-1)
        return RoutingPlan(order=order, send_counts=send_counts, recv_counts=recv_counts, recv_experts=recv_experts, tokens=t, top_k=k)

    def dispatch(self, hidden: torch.Tensor, plan: RoutingPlan) -> torch.Tensor:
        """``hidden`` [T, H] -> rows received by this rank [R, H], aligned with ``plan.recv_experts``."""
        rows = hidden.index_select(0, plan.order // plan.top_k)
        return self.comm.all_to_all_v(rows, plan.send_counts, plan.recv_counts)

    def combine(self, expert_out: torch.Tensor, weights: torch.Tensor, plan: RoutingPlan) -> torch.Tensor:
        """``expert_out`` [R, H] (same order as received) and router ``weights`` [T, k] -> [T, H]."""
        back = self.comm.all_to_all_v(expert_out, plan.recv_counts, plan.send_counts)     # the inverse exchange
        out = torch.zeros(plan.tokens, expert_out.shape[1], dtype=torch.float32, device=expert_out.device)
        w = weights.reshape(-1).float().index_select(0, plan.order)
        out.index_add_(0, plan.order // plan.top_k, back.float() * w[:, None])
        return out.to(expert_out.dtype)

    def run(self, hidden, expert_ids, weights, expert_fn):
        """Dispatch, ``expert_fn(rows [n, H], local expert index) -> [n, H]`` per local expert, combine."""
        plan = self.plan(expert_ids)
        rows = self.dispatch(hidden, plan)
        out = torch.empty_like(rows)
        for e in range(self.per_rank):
            sel = (plan.recv_experts == e).nonzero(as_tuple=True)[0]
            if len(sel):
                out[sel] = expert_fn(rows[sel], e)
        return self.combine(out, weights, plan)
