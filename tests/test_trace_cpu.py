"""Trace spans: the optional NVTX hand-off to external profilers."""
def test_spans_mirror_into_nvtx_ranges_when_asked():
    """With the NVTX hand-off on, every span pushes and pops one range named category:name, nested in order; a push
    that raises turns the hand-off off instead of breaking the span."""
    from onnx_genai_b200.utils.trace import Tracer

    t = Tracer()
    log = []
    assert t.enable_nvtx(push=lambda name: log.append(("push", name)), pop=lambda: log.append(("pop",)))
    with t.span("loop.step"):
        with t.span("gemm", cat="op"):
            pass
    assert log == [("push", "engine:loop.step"), ("push", "op:gemm"), ("pop",), ("pop",)]

    def bad(name):
        raise RuntimeError("no NVTX here")

    t.enable_nvtx(push=bad, pop=lambda: log.append(("pop",)))
    with t.span("x"):
        pass
    assert t.nvtx is None and log[-1] == ("pop",) and len(log) == 4


def test_engine_steps_land_in_the_trace_file_named_by_the_environment(tmp_path):
    """`ONNX_GENAI_TRACE=<path>`: every engine step records loop.step with its schedule / forward / commit parts, and the
    file is written when the process exits."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    trace = str(tmp_path / "engine_trace.json")
    code = """
import numpy as np, torch
from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
cfg = DecoderConfig(name="t", num_layers=1, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=128, vocab=97, max_position=128)
w = random_weights(cfg, "cpu", seed=1, std=0.2, dtype=torch.float32)
eng = LLMEngine(EngineConfig(model=cfg, num_pages=16, max_seqs=2, max_tokens_per_step=32, max_seq_len=64), weights=w, device="cpu")
print(eng.generate([[1, 2, 3, 4]], max_new_tokens=5))
"""
    proc = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, PYTHONPATH=root, ONNX_GENAI_TRACE=trace, CUDA_VISIBLE_DEVICES=""),
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    events = [e for e in json.load(open(trace))["traceEvents"] if e["ph"] == "X"]
    names = [e["name"] for e in events]
    assert names.count("loop.step") >= 5 and names.count("loop.schedule") >= 5 and "loop.forward" in names and "loop.commit" in names
    step = next(e for e in events if e["name"] == "loop.step")
    inner = [e for e in events if e["name"] != "loop.step" and step["ts"] <= e["ts"] and e["ts"] + e["dur"] <= step["ts"] + step["dur"] + 1]
    assert {e["name"] for e in inner} >= {"loop.schedule", "loop.forward", "loop.commit"}
