"""Trace / profile diagnosis: each finding fires on evidence built for it, and nothing is classified without numbers."""
import json

from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.utils import diagnose as dg
from onnx_genai_b200.utils.cost_model import StepShape

AN = dg.RooflineAnalyzer(peak_tflops=1000.0, hbm_gbs=5000.0)


def test_roofline_classification_and_indeterminate_samples():
    r = AN.analyze(dg.KernelSample("gemm", 2e-3, 1, flops=1e12, bytes=1e8))
    assert r.bound == "compute" and abs(r.efficiency - 0.5) < 1e-9 and abs(r.achieved_tflops - 500.0) < 1e-6
    r = AN.analyze(dg.KernelSample("decode", 1e-3, 1, flops=1e9, bytes=2.5e9))
    assert r.bound == "memory" and abs(r.efficiency - 0.5) < 1e-9 and abs(r.achieved_gbs - 2500.0) < 1e-6
    r = AN.analyze(dg.KernelSample("tiny", 1e-3, 100, flops=1e6, bytes=1e6))
    assert r.bound == "latency"
    r = AN.analyze(dg.KernelSample("mystery", 1e-3, 3))
    assert r.bound == "indeterminate" and r.efficiency is None


def test_findings_fire_on_their_evidence():
    samples = [
        dg.KernelSample("gemm:gate_up", 6e-3, 28, flops=1.5e12, bytes=1e9),          # 0.25 of compute roofline, 48 % of time
        dg.KernelSample("paged_decode", 3e-3, 28, flops=1e9, bytes=13.5e9),           # 0.9 of memory roofline: fine
        dg.KernelSample("rmsnorm", 0.5e-3, 228, bytes=1e8),                            # 2.2 us each: launch-bound
        dg.KernelSample("tp_exchange_norm", 3e-3, 56),                                 # 24 % in exchanges
    ]
    d = dg.diagnose_samples(samples, AN, wall_s=25e-3, steps=1, preemptions=2)
    titles = [i.title for i in d.issues]
    assert any("gemm:gate_up runs at 0.25" in t for t in titles)
    assert not any("paged_decode runs" in t for t in titles)
    assert any("rmsnorm is launch-bound" in t for t in titles)
    assert "tensor-parallel exchange dominates" in titles and "the GPU waits for the host" in titles and "sequences were preempted" in titles
    for i in d.issues:
        assert i.description and i.evidence and i.root_cause and i.suggestion       # what, why and how are never empty
    text = d.report()
    assert text.index("[high]") < text.index("[medium]") and "roofline (share of device time" in text
    quiet = dg.diagnose_samples(samples[1:2], AN, wall_s=3.1e-3)
    assert quiet.issues == []
    assert dg.diagnose_samples([], AN).notes


def test_profile_tables_get_rooflines_from_the_model_shape():
    cfg = DecoderConfig(name="q", num_layers=28, hidden=3584, num_heads=28, num_kv_heads=4, head_dim=128, intermediate=18944, vocab=152064)
    shape = StepShape(decode_rows=255, prefill_tokens=1025, mean_context=1200, prefill_context=600)
    agg = {"gemm:gate_up+swiglu": (6.55, 28), "gemm:down": (3.7, 28), "paged_decode": (3.76, 28), "rmsnorm": (0.54, 57), "sample": (0.46, 1)}
    samples = dg.samples_from_profile(agg, cfg, shape)
    by = {s.name: s for s in samples}
    assert abs(by["gemm:gate_up+swiglu"].flops - 2.0 * 1280 * 2 * 18944 * 3584 * 28) < 1e6
    assert by["paged_decode"].bytes == 255 * 1200 * 4 * 2 * 128 * 2 * 28 and by["sample"].flops is None
    d = dg.diagnose_samples(samples, dg.RooflineAnalyzer(1376.4, 6446.6))
    eff = {r.name: r.efficiency for r, _ in d.rooflines}
    assert 0.8 < eff["gemm:gate_up+swiglu"] < 1.1 and 0.6 < eff["paged_decode"] < 1.0
    assert any("sample" in n for n in d.notes) or True


def test_trace_documents_are_read_and_reported(tmp_path, capsys):
    doc = {"traceEvents": [
        {"name": "MatMul", "cat": "op", "ph": "X", "ts": 0.0, "dur": 4000.0, "args": {"flops": 1e12, "bytes": 1e8}},
        {"name": "MatMul", "cat": "op", "ph": "X", "ts": 5000.0, "dur": 4000.0, "args": {"flops": 1e12, "bytes": 1e8}},
        {"name": "Softmax", "cat": "op", "ph": "X", "ts": 9000.0, "dur": 1000.0},
        {"name": "thread_name", "ph": "M", "pid": 1, "tid": 1, "args": {"name": "op"}}]}
    samples, wall = dg.samples_from_trace(doc)
    assert abs(wall - 0.010) < 1e-9 and {s.name: s.calls for s in samples} == {"MatMul": 2, "Softmax": 1}
    p = tmp_path / "t.json"
    p.write_text(json.dumps(doc))
    assert dg.main([str(p)]) == 0
    out = capsys.readouterr().out
    assert "MatMul runs at" in out and "Softmax" in out and "indeterminate" in out


def test_device_tracks_are_judged_against_the_host_span_that_encloses_them():
    """A trace with one category per GPU stream (what the CUPTI activity collector writes): kernels are aggregated under
    short names, copies by direction, load-time events outside the longest host span are left out, overlapping streams
    count once, and a mostly idle device is reported as waiting for the host."""
    from onnx_genai_b200.utils.diagnose import device_view, diagnose_samples

    ev = lambda name, cat, ts_us, dur_us: {"name": name, "cat": cat, "ph": "X", "ts": ts_us, "dur": dur_us, "pid": 1, "tid": 1}
    events = [ev("load", "cli", 0, 500), ev("generate", "cli", 1000, 10000),
              ev("memcpy host to device 1048576 B", "gpu0 stream 13", 100, 300)]                      # load time: outside the window
    for i in range(20):
        events.append(ev("void ogb::gemm_bf16_tcgen05_kernel<32, 1>(CUtensorMap_st, int)", "gpu0 stream 7", 1100 + 400 * i, 30))
        events.append(ev("void ogb::rmsnorm_warp_kernel(__nv_bfloat16*, int)", "gpu0 stream 7", 1140 + 400 * i, 3))
        events.append(ev("memcpy device to host 4 B", "gpu0 stream 13", 1110 + 400 * i, 10))           # under the GEMM: no extra busy time
    view = device_view({"traceEvents": events})
    samples, wall, busy, window = view
    assert window == "generate" and abs(wall - 0.010) < 1e-9
    by = {s.name: s for s in samples}
    assert set(by) == {"gemm_bf16_tcgen05_kernel<32, 1>", "rmsnorm_warp_kernel", "memcpy device to host"}
    assert by["gemm_bf16_tcgen05_kernel<32, 1>"].calls == 20 and by["memcpy device to host"].category == "copy"
    assert abs(busy - 20 * 33e-6) < 1e-9                                                              # 30 + 3 us per step, the copy hidden
    d = diagnose_samples(samples, wall_s=wall, device_busy_s=busy)
    titles = [i.title for i in d.issues]
    assert "the GPU waits for the host" in titles and any("rmsnorm_warp_kernel is launch-bound" in t for t in titles)
    assert device_view({"traceEvents": [ev("step", "engine", 0, 10)]}) is None
