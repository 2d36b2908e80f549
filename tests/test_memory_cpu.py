"""Memory ledger: limits, leases, the KV budget, and the engine's own registration."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.engine.memory import MemoryLedger, MemoryLimitError, parse_limit, tensor_bytes
from onnx_genai_b200.models.config import DecoderConfig


def test_parse_limit_forms():
    assert parse_limit("auto") is None and parse_limit(None) is None
    assert parse_limit("8GiB") == 8 << 30 and parse_limit("512mb") == 512 << 20 and parse_limit("1073741824") == 1 << 30
    assert parse_limit("0.9", total_bytes=1000) == 900 and parse_limit("1.5g") == int(1.5 * (1 << 30))
    with pytest.raises(ValueError, match="fraction"):
        parse_limit("0.5")
    with pytest.raises(ValueError, match="cannot read"):
        parse_limit("lots")


def test_leases_limits_and_kv_budget():
    led = MemoryLedger(limits={"vram": 1000})
    w = led.lease("weights", "vram", 400, "model")
    a = led.lease("activations", "vram", 100)
    assert led.kv_budget("vram", reserve=50) == 450 and led.available("host") is None
    with pytest.raises(MemoryLimitError, match="kv .* needs .* but only"):
        led.lease("kv", "vram", 600, "pool")
    kv = led.lease("kv", "vram", 450)
    with pytest.raises(MemoryLimitError, match="cannot grow"):
        kv.resize(600)
    a.release()
    kv.resize(550)
    snap = led.snapshot()["vram"]
    assert snap["used_bytes"] == 950 and snap["by_role"] == {"weights": 400, "kv": 550} and snap["peak_bytes"] == 950
    w.release()
    w.release()                                     # idempotent
    assert led.used("vram") == 550
    with pytest.raises(ValueError):
        led.lease("cache", "vram", 1)


def test_engine_registers_what_it_allocated():
    cfg = DecoderConfig(name="m", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=97,
                        rope_theta=1e4, tie_embeddings=True, max_position=256)
    eng = LLMEngine(EngineConfig(model=cfg, num_pages=32, max_seqs=4, max_tokens_per_step=64, max_seq_len=128), device="cpu")
    snap = eng.memory.snapshot()["host"]
    kv_bytes = 2 * 32 * 2 * 2 * 16 * 16 * 4                                    # layers x pages x kv heads x (K,V) x tokens x dim x fp32
    assert snap["by_role"]["kv"] == kv_bytes == tensor_bytes(eng.kv)
    assert snap["by_role"]["weights"] == tensor_bytes(eng.weights) > 0 and snap["by_role"]["activations"] > 0
    shared = torch.zeros(10)
    assert tensor_bytes({"a": shared, "b": [shared, shared[2:]]}) == 40        # one storage counted once
