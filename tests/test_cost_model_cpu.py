"""Roofline cost model: ideal times, calibration from a measured breakdown, persistence, planning helpers."""
import json

import pytest

from onnx_genai_b200.models.config import PRESETS
from onnx_genai_b200.parallel.pipeline import plan_stages
from onnx_genai_b200.utils.cost_model import CostModel, HardwareRates, StepShape

Q7 = PRESETS["qwen2.5-7b"]
SHAPE = StepShape(decode_rows=255, prefill_tokens=1025, mean_context=1200, prefill_context=600)
# one measured 1-GPU step of that shape (milliseconds per part)
MEASURED = {"mlp": 10.25, "decode_attention": 3.76, "prefill_attention": 2.10, "qkv": 1.41, "o_proj": 1.02, "sampler": 0.46,
            "rowwise": 1.00, "lm_head": 0.27}


def test_ideal_is_a_lower_bound_close_to_the_measured_gemms():
    cm = CostModel()
    ideal = cm.ideal(Q7, SHAPE)
    assert all(ideal[k] <= MEASURED[k] * 1.05 for k in MEASURED), {k: (ideal[k], MEASURED[k]) for k in MEASURED}
    assert 0.9 < ideal["mlp"] / MEASURED["mlp"] < 1.05            # the big GEMMs run near the sustained library rate
    # compute-bound at this batch, weight-bound at batch 1
    one = cm.ideal(Q7, StepShape(decode_rows=1, mean_context=512))
    weights_ms = Q7.weight_bytes() / (cm.rates.hbm_gbs * 1e9) * 1e3
    assert 0.8 * weights_ms < sum(one[k] for k in ("qkv", "o_proj", "mlp", "lm_head")) < 1.1 * weights_ms


def test_calibration_reproduces_the_measurement_and_persists(tmp_path):
    cm = CostModel()
    eff = cm.calibrate(Q7, SHAPE, MEASURED)
    assert all(e >= 0.95 for e in eff.values()) and eff["sampler"] > 5       # the sampler is far from its byte bound
    est = cm.estimate(Q7, SHAPE)
    assert est["total_ms"] == pytest.approx(sum(MEASURED.values()), rel=1e-6)
    assert est["output_tok_s"] == pytest.approx(255 / sum(MEASURED.values()) * 1e3, rel=1e-6)
    path = str(tmp_path / "cm.json")
    cm.save(path)
    again = CostModel.load(path)
    assert again.estimate(Q7, SHAPE) == est and json.load(open(path))["version"] == 1
    with pytest.raises(KeyError, match="unknown part 'gemm'"):
        cm.calibrate(Q7, SHAPE, {"gemm": 1.0})
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"version": 9}))
    with pytest.raises(ValueError, match="version 9"):
        CostModel.load(str(bad))


def test_planning_helpers(tmp_path):
    cm = CostModel()
    cm.calibrate(Q7, SHAPE, MEASURED)
    pick = cm.pick_tp(Q7, SHAPE)
    t = pick["table"]
    assert t[1] > t[2] > t[4] and pick["tp"] in (4, 8)
    assert t[8] > t[1] / 8 * 1.5                                    # exchanges and replicated work keep scaling sub-linear
    assert cm.pick_tp(Q7, SHAPE, max_step_ms=t[2] + 0.1)["tp"] == 2
    fp8 = cm.estimate(Q7, StepShape(255, 1025, 1200, 600, kv_bytes=1))
    assert fp8["parts_ms"]["decode_attention"] == pytest.approx(cm.estimate(Q7, SHAPE)["parts_ms"]["decode_attention"] / 2)
    costs = cm.layer_costs(Q7, SHAPE)
    plan = plan_stages(Q7.num_layers, 4, [costs["layer"]] * Q7.num_layers, costs["embed"], costs["head"])
    assert plan.ranges[0][0] == 0 and plan.ranges[-1][1] == Q7.num_layers and plan.imbalance < 1.15
    assert plan.ranges[-1][1] - plan.ranges[-1][0] < plan.ranges[-2][1] - plan.ranges[-2][0]      # the head costs about a layer
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"hbm_gbs": 5000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1300.0, "gpu_name": "X"}))
    r = HardwareRates.from_measured(str(peaks))
    assert (r.hbm_gbs, r.bf16_tflops, r.name) == (5000.0, 1300.0, "X")
    moe = cm.estimate(PRESETS["qwen3-30b-a3b"], StepShape(128, 0, 1024), tp=4)
    assert moe["total_ms"] > 0 and moe["parts_ms"]["exchange"] > 0
