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


def test_pressure_queue_grants_in_order_after_charging():
    import threading
    import time

    from onnx_genai_b200.engine.memory import MemoryLedger, MemoryLimitError, PressureQueue, PressureTicket

    ledger = MemoryLedger(limits={"host": 100})
    q = PressureQueue(ledger, "host")
    a = q.request("kv_offload", 60, "a")
    assert a.poll() == PressureTicket.GRANTED and ledger.used("host") == 60
    b = q.request("kv_offload", 70, "b")                     # does not fit: queued
    c = q.request("kv_offload", 10, "c")                     # would fit, but must not overtake b
    assert b.poll() == c.poll() == PressureTicket.PENDING and ledger.used("host") == 60
    seen = []
    waiter = threading.Thread(target=lambda: seen.append(b.wait(5.0)))
    waiter.start()
    time.sleep(0.05)
    q.release(a)                                             # frees 60: b (70) is charged and woken, then c (10) fits too
    waiter.join(5.0)
    assert seen == [PressureTicket.GRANTED] and c.poll() == PressureTicket.GRANTED and ledger.used("host") == 80
    # the trace shows charge-before-wake order and first-come-first-served grants
    grants = [tid for _, kind, tid, _ in q.events if kind == "grant"]
    assert grants == [a.id, b.id, c.id]
    # cancellation of the head unblocks what is behind it; expiry does the same
    d = q.request("kv", 50, "d")
    e = q.request("kv", 15, "e")
    assert d.poll() == e.poll() == PressureTicket.PENDING
    d.cancel()
    assert d.poll() == PressureTicket.CANCELLED and e.poll() == PressureTicket.GRANTED and ledger.used("host") == 95
    f = q.request("kv", 30, "f", timeout=0.05)
    g = q.request("kv", 5, "g")
    time.sleep(0.08)
    assert f.poll() == PressureTicket.EXPIRED and g.poll() == PressureTicket.GRANTED and ledger.used("host") == 100
    with pytest.raises(MemoryLimitError, match="could never be granted"):
        q.request("kv", 101, "too big")
    # a reclaim callback is asked before a request has to queue
    for t in (b, c, e, g):
        q.release(t)
    cache = [ledger.lease("kv_offload", "host", 90, "cache")]
    asked = []

    def reclaim(nbytes):
        asked.append(nbytes)
        cache.pop().release()
        return 90

    q2 = PressureQueue(ledger, "host", reclaim=reclaim)
    assert q2.request("weights", 40, "h").poll() == PressureTicket.GRANTED and asked == [30]


def test_pressure_queue_under_threads_never_exceeds_the_limit():
    import random
    import threading

    from onnx_genai_b200.engine.memory import MemoryLedger, PressureQueue, PressureTicket

    ledger = MemoryLedger(limits={"host": 64})
    q = PressureQueue(ledger, "host")
    peak, errors = [0], []

    def worker(seed):
        rng = random.Random(seed)
        for _ in range(40):
            t = q.request("workspace", rng.randint(1, 32), f"w{seed}")
            if t.wait(5.0) != PressureTicket.GRANTED:
                errors.append("timeout")
                return
            peak[0] = max(peak[0], ledger.used("host"))
            if ledger.used("host") > 64:
                errors.append("over limit")
            q.release(t)

    threads = [threading.Thread(target=worker, args=(s,)) for s in range(6)]
    [t.start() for t in threads]
    [t.join(30) for t in threads]
    assert errors == [] and ledger.used("host") == 0 and 0 < peak[0] <= 64 and not q.waiting


def test_host_growable_buffer_keeps_its_address_and_returns_pages():
    import torch

    from onnx_genai_b200.utils.host_vmm import HostGrowableBuffer, HostVmmError

    buf = HostGrowableBuffer(1 << 30)                      # address space only: nothing is committed
    assert buf.committed == 0 and buf.reserved >= 1 << 30
    base = buf.ptr
    buf.grow(100_000)
    assert buf.committed % buf.page == 0 and buf.committed >= 100_000
    a = buf.view(torch.int32, (1000,))
    a.copy_(torch.arange(1000, dtype=torch.int32))
    first = buf.committed
    buf.grow(8 << 20)
    whole = buf.view(torch.uint8)
    assert buf.ptr == base and whole.data_ptr() == a.data_ptr() and whole.numel() == buf.committed
    assert torch.equal(buf.view(torch.int32, (1000,)), torch.arange(1000, dtype=torch.int32))      # contents survive growth
    whole[first:].fill_(7)
    del whole
    assert buf.shrink(first) == first
    buf.grow(8 << 20)
    assert int(buf.view(torch.uint8)[first:].sum()) == 0   # pages given back come back as fresh zero pages
    with pytest.raises(HostVmmError, match="exceeds the"):
        buf.view(torch.uint8, (buf.committed + 1,))
    with pytest.raises(HostVmmError, match="address space were reserved"):
        buf.grow(2 << 30)
    buf.close()
