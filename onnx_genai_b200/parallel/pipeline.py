"""Pipeline parallelism: stage planning, the forward schedule, and a stage runner over point-to-point messages.

Layers are split into contiguous stages, one per rank; a batch is cut into micro-batches that flow through the
stages so that stage s works on micro-batch m while stage s+1 works on m-1.  The reference describes this shape
(stage layer ranges and a send/recv pattern between neighbouring stages, docs/distributed/DISTRIBUTED_RUNTIME.md:892-940)
without implementing it.  Here:

* :func:`plan_stages` -- contiguous layer ranges that minimise the slowest stage, given per-layer costs and the
  extra cost of the embedding (first stage) and of the final norm + LM head (last stage);
* :func:`forward_schedule` -- the fill / steady / drain timetable of an inference (forward-only) pipeline and its
  bubble fraction ``(stages - 1) / (micro_batches + stages - 1)``;
* :class:`PipelineStage` -- runs one rank's part: receive the activation from the previous stage, apply this stage's
  function, send to the next; the last stage collects results.  It works over any communicator of this package with
  ``send`` / ``recv`` (the CPU oracle in tests, ``torch.distributed`` across GPUs).

The serving engine does not use it: a 7B to 30B model fits one B200 several times over and tensor parallelism over
NVLink has the lower latency, so the named configurations never need stages.  It is the seam for models that do.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class StagePlan:
    ranges: list            # [(first layer, one past last layer)] per stage
    costs: list             # cost per stage (including embedding / head extras)

    @property
    def imbalance(self) -> float:
        return max(self.costs) / (sum(self.costs) / len(self.costs)) if self.costs else 1.0


def plan_stages(num_layers: int, stages: int, layer_costs=None, embed_cost: float = 0.0, head_cost: float = 0.0) -> StagePlan:
    """Contiguous partition of ``num_layers`` into ``stages`` parts minimising the largest stage cost (dynamic programme)."""
    if stages < 1 or stages > num_layers:
        raise ValueError(f"{stages} stages for {num_layers} layers: every stage needs at least one layer")
    costs = [1.0] * num_layers if layer_costs is None else [float(c) for c in layer_costs]
    if len(costs) != num_layers:
        raise ValueError(f"{len(costs)} layer costs for {num_layers} layers")
    prefix = [0.0]
    for c in costs:
        prefix.append(prefix[-1] + c)

    def seg(i, j, s):     # cost of layers [i, j) as stage s
        return prefix[j] - prefix[i] + (embed_cost if s == 0 else 0.0) + (head_cost if s == stages - 1 else 0.0)

    inf = float("inf")
    best = [[inf] * (num_layers + 1) for _ in range(stages + 1)]
    cut = [[0] * (num_layers + 1) for _ in range(stages + 1)]
    best[0][0] = 0.0
    for s in range(1, stages + 1):
        for j in range(s, num_layers - (stages - s) + 1):
            for i in range(s - 1, j):
                v = max(best[s - 1][i], seg(i, j, s - 1))
                if v < best[s][j]:
                    best[s][j], cut[s][j] = v, i
    ranges, j = [], num_layers
    for s in range(stages, 0, -1):
        i = cut[s][j]
        ranges.append((i, j))
        j = i
    ranges.reverse()
    return StagePlan(ranges=ranges, costs=[seg(i, j, s) for s, (i, j) in enumerate(ranges)])


def forward_schedule(stages: int, micro_batches: int) -> dict:
    """Timetable of a forward-only pipeline: slot t has stage s working on micro-batch t - s (when that exists)."""
    slots = []
    for t in range(micro_batches + stages - 1):
        slots.append([(s, t - s) for s in range(stages) if 0 <= t - s < micro_batches])
    return {"slots": slots, "num_slots": len(slots), "bubble_fraction": (stages - 1) / (micro_batches + stages - 1)}


class PipelineStage:
    def __init__(self, comm, stage_fn, first: bool | None = None, last: bool | None = None):
        """``stage_fn(x) -> y`` is this rank's layers.  Rank r is stage r; first / last default to the ends of the group."""
        self.comm, self.fn = comm, stage_fn
        self.first = comm.rank == 0 if first is None else first
        self.last = comm.rank == comm.world - 1 if last is None else last

    def run(self, micro_batches=None, shapes=None, dtype=torch.float32, device="cpu"):
        """First stage: ``micro_batches`` is the list of inputs.  Other stages: ``shapes`` lists the activation shape of each
        micro-batch as it arrives.  Returns the outputs on the last stage, None elsewhere."""
        n = len(micro_batches) if self.first else len(shapes)
        outs = []
        for m in range(n):
            if self.first:
                x = micro_batches[m]
            else:
                x = torch.empty(shapes[m], dtype=dtype, device=device)
                self.comm.recv(x, self.comm.rank - 1)
            y = self.fn(x)
            if self.last:
                outs.append(y)
            else:
                self.comm.send(y.contiguous(), self.comm.rank + 1)
        return outs if self.last else None
