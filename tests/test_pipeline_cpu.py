"""Pipeline planning, schedule and a three-stage forward over the CPU oracle."""
import pytest
import torch

from onnx_genai_b200.parallel.pipeline import PipelineStage, forward_schedule, plan_stages
from test_ep_dispatch_cpu import run_ranks


def test_plan_balances_uneven_layers_and_extras():
    p = plan_stages(8, 4)
    assert p.ranges == [(0, 2), (2, 4), (4, 6), (6, 8)] and p.imbalance == 1.0
    p = plan_stages(6, 3, layer_costs=[4, 1, 1, 1, 1, 4])
    assert p.ranges == [(0, 1), (1, 5), (5, 6)] and p.costs == [4.0, 4.0, 4.0]
    # an expensive LM head pulls layers away from the last stage
    p = plan_stages(8, 2, head_cost=2.0)
    assert p.ranges == [(0, 5), (5, 8)] and p.costs == [5.0, 5.0]
    with pytest.raises(ValueError, match="at least one layer"):
        plan_stages(2, 3)


def test_forward_schedule_fill_and_drain():
    s = forward_schedule(3, 4)
    assert s["num_slots"] == 6 and s["slots"][0] == [(0, 0)] and s["slots"][2] == [(0, 2), (1, 1), (2, 0)] and s["slots"][5] == [(2, 3)]
    assert s["bubble_fraction"] == pytest.approx(2 / 6)
    assert forward_schedule(1, 5)["bubble_fraction"] == 0


def test_three_stage_forward_equals_sequential():
    torch.manual_seed(1)
    layers = [torch.randn(8, 8) * 0.4 for _ in range(6)]
    plan = plan_stages(6, 3)
    batches = [torch.randn(n, 8) for n in (3, 5, 2, 4)]

    def fn(c):
        lo, hi = plan.ranges[c.rank]

        def stage(x):
            for w in layers[lo:hi]:
                x = torch.tanh(x @ w)
            return x

        return PipelineStage(c, stage).run(micro_batches=batches if c.rank == 0 else None, shapes=[b.shape for b in batches])

    out, errs = run_ranks(3, fn)
    assert errs == [None] * 3 and out[0] is None and out[1] is None
    for got, x in zip(out[2], batches):
        for w in layers:
            x = torch.tanh(x @ w)
        assert torch.allclose(got, x, atol=1e-6)
