"""Tensor-parallel sharding arithmetic (Megatron 1-D layout).

The scheme is the one the reference's feasibility study records but never implements
(docs/research/tensor-parallelism-feasibility.md:60-110): q/k/v and gate/up projections are
column-parallel, o_proj and down_proj row-parallel, and KV heads are replicated when there are
fewer of them than ranks.  One addition: when the query heads of a KV group do not divide evenly
over the ranks that share the group (Qwen2.5-7B: 7 query heads per KV head, 2 ranks per KV head at
TP=8) the split is uneven (4 + 3) instead of padding with dummy heads.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class HeadShard:
    q_heads: list[int]     # global query head ids owned by this rank (contiguous inside one or more KV groups)
    kv_heads: list[int]    # global KV head ids held by this rank

    @property
    def group(self) -> int:
        return len(self.q_heads) // max(1, len(self.kv_heads))


def shard_heads(num_heads: int, num_kv_heads: int, tp: int, rank: int) -> HeadShard:
    if tp == 1:
        return HeadShard(list(range(num_heads)), list(range(num_kv_heads)))
    group = num_heads // num_kv_heads
    assert group * num_kv_heads == num_heads, "query heads must be a multiple of KV heads"
    if num_kv_heads >= tp:
        assert num_kv_heads % tp == 0, (num_kv_heads, tp)
        per = num_kv_heads // tp
        kv = list(range(rank * per, (rank + 1) * per))
        q = [h * group + g for h in kv for g in range(group)]
        return HeadShard(q, kv)
    assert tp % num_kv_heads == 0, (num_kv_heads, tp)
    ranks_per_kv = tp // num_kv_heads
    kv_head = rank // ranks_per_kv
    local = rank % ranks_per_kv
    base, extra = divmod(group, ranks_per_kv)
    assert base >= 1, "more ranks per KV head than query heads in the group"
    start = local * base + min(local, extra)
    count = base + (1 if local < extra else 0)
    q = [kv_head * group + start + i for i in range(count)]
    return HeadShard(q, [kv_head])


def shard_range(total: int, tp: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous [begin, end) of a dimension split into ``tp`` near-equal parts of ``multiple`` granularity."""
    units = total // multiple
    assert units * multiple == total, (total, multiple)
    base, extra = divmod(units, tp)
    start = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return start * multiple, (start + count) * multiple
