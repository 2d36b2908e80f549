"""Engine allocator interface: accounting against the ledger, identity after release, capabilities, the deferred-release
queue with its quarantine, and an engine whose KV pools come from a caller's allocator."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.allocator import (Allocator, AllocatorError, DeferredReleaseQueue, PinnedHostAllocator,
                                              TorchAllocator)
from onnx_genai_b200.engine.memory import MemoryLedger, MemoryLimitError


def test_allocations_are_charged_identified_and_refused_over_the_limit():
    ledger = MemoryLedger(limits={"host": 1 << 20})
    alloc = TorchAllocator("cpu", ledger)
    a = alloc.allocate(600 << 10, "kv", "pool")
    assert ledger.used("host", "kv") == 600 << 10 and alloc.stats()["live"] == 1
    with pytest.raises(MemoryLimitError, match="only"):
        alloc.allocate(600 << 10, "workspace", "too much")
    assert alloc.stats()["live"] == 1 and ledger.used("host") == 600 << 10           # the refused request left nothing behind
    t = a.view((10, 4), torch.float32)
    t.fill_(3.0)
    assert float(a.data[:160].view(torch.float32).sum()) == 120.0
    with pytest.raises(AllocatorError, match="view of"):
        a.view((1 << 20,), torch.float32)
    alloc.release(a)
    assert ledger.used("host") == 0 and a.generation == 2
    with pytest.raises(AllocatorError, match="was released"):
        a.check()
    with pytest.raises(AllocatorError, match="released twice"):
        alloc.release(a)
    other = TorchAllocator("cpu")
    with pytest.raises(AllocatorError, match="another allocator"):
        other.release(alloc.allocate(16))
    assert alloc.stats()["peak_bytes"] == 600 << 10
    assert not alloc.virtual_backing and not PinnedHostAllocator(pin=False).device_addressable_host


def test_deferred_releases_complete_on_drain_and_failures_are_quarantined():
    class Flaky(Allocator):
        def _obtain(self, nbytes, role, tag):
            return torch.empty(nbytes, dtype=torch.uint8), None

        def _dispose(self, alloc):
            if alloc.tag == "bad":
                raise OSError("unmap failed")
            super()._dispose(alloc)

    alloc = Flaky()
    q = DeferredReleaseQueue()
    good, bad = alloc.allocate(128, tag="good"), alloc.allocate(64, tag="bad")
    q.enqueue(good, reason="evicted")
    q.enqueue(bad)
    with pytest.raises(AllocatorError, match="already waiting"):
        q.enqueue(good)
    assert q.stats()["pending"] == 2 and q.pending_bytes == 192
    assert q.drain() == 2                                      # no GPU work is pending on the CPU: both are ready
    s = q.stats()
    assert s == {"pending": 0, "pending_bytes": 0, "released": 1, "quarantined": 1, "quarantined_bytes": 64}
    assert good.released and "unmap failed" in q.quarantined[0][1]
    assert q.flush() == 0


def test_engine_takes_its_kv_pools_from_the_callers_allocator_and_returns_them_on_close():
    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import DecoderConfig

    cfg = DecoderConfig(name="a", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=97,
                        rope_theta=1e4, tie_embeddings=True, qkv_bias=True, weight_format="bf16", max_position=256)
    alloc = TorchAllocator("cpu")
    plain = LLMEngine(EngineConfig(model=cfg, num_pages=16, max_seqs=4, max_tokens_per_step=64, max_seq_len=128, seed=3), device="cpu")
    eng = LLMEngine(EngineConfig(model=cfg, num_pages=16, max_seqs=4, max_tokens_per_step=64, max_seq_len=128, seed=3, allocator=alloc),
                    device="cpu")
    assert alloc.stats()["live"] == 2 and alloc.allocated_bytes == eng.kv.mapped_bytes()
    prompt = np.arange(20, dtype=np.int32) % cfg.vocab
    assert eng.generate([prompt], 8) == plain.generate([prompt], 8)
    stats = eng.close()
    assert stats["released"] == 2 and stats["pending"] == 0 and alloc.stats()["live"] == 0 and alloc.allocated_bytes == 0
