"""KV offload connector: chunks leave the device when a request finishes and come back on a later prefix hit."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.api import Engine, GenerateOptions
from onnx_genai_b200.engine.kv_connector import LocalTieredConnector, chunk_keys
from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights

CFG = DecoderConfig(name="kvc", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96,
                    vocab=211, rope_theta=1e4, tie_embeddings=True, qkv_bias=True, weight_format="bf16", max_position=1024)


def _engine(weights, kv_dtype="bf16", num_pages=48):
    llm = LLMEngine(EngineConfig(model=CFG, num_pages=num_pages, max_seqs=4, max_tokens_per_step=256, max_seq_len=768,
                                 enable_prefix_cache=True, kv_dtype=kv_dtype), weights=weights, device="cpu")
    return Engine(llm)


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8", "int8"])
def test_chunks_are_offloaded_and_restored_after_the_device_cache_forgot_them(tmp_path, kv_dtype):
    weights = random_weights(CFG, "cpu", seed=11, std=0.3, dtype=torch.float32)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, CFG.vocab, size=600).tolist()                      # two full 256-token chunks + a tail
    opt = GenerateOptions(max_new_tokens=6, ignore_eos=True)
    eng = _engine(weights, kv_dtype)
    conn = LocalTieredConnector(str(tmp_path / "kv"), max_host_bytes=1)         # everything but one chunk spills to disk
    eng.attach_kv_connector(conn)
    first = eng.generate(prompt, opt)
    assert eng.kv_offload.chunks_stored == 2 and conn.stats["spilled"] >= 1
    for _ in range(3):                                                          # other traffic evicts the cached pages (48-page pool)
        eng.generate(rng.integers(0, CFG.vocab, size=500).tolist(), opt)
    assert len(eng.llm.core.prefix_peek(prompt)) < 32                           # the device no longer serves both chunks
    hits0 = eng.llm.core.prefix_hits
    again = eng.generate(prompt, opt)
    assert eng.kv_offload.tokens_restored >= 256 and eng.llm.core.prefix_hits > hits0
    assert again.token_ids == first.token_ids                                   # restored K/V is the K/V that was computed
    # a second engine process (same weights) picks the chunks up from the directory
    conn.flush()
    other = _engine(weights, kv_dtype)
    other.attach_kv_connector(LocalTieredConnector(str(tmp_path / "kv")))
    fresh = other.generate(prompt, opt)
    assert other.kv_offload.tokens_restored == 512 and other.kv_offload.connector.stats["disk_hits"] == 2
    assert fresh.token_ids == first.token_ids


def test_connector_tiers_keys_and_limits(tmp_path):
    keys = chunk_keys(list(range(600)), "m")
    assert len(keys) == 2 and keys != chunk_keys(list(range(600)), "other-model")
    assert chunk_keys([9] + list(range(1, 600)), "m")[1] != keys[1]             # a key covers the whole prefix
    c = LocalTieredConnector(str(tmp_path / "d"), max_host_bytes=250, max_disk_bytes=250)
    for i in range(5):
        c.store(f"k{i}", bytes([i]) * 100)
    assert c.host_bytes <= 250 and c.disk_bytes <= 250 and c.stats["deleted"] >= 1
    assert c.fetch("k4") == bytes([4]) * 100 and c.stats["host_hits"] == 1
    assert c.fetch("k0") is None                                                # oldest chunk fell off the disk tier
    survivors = [k for k in ("k1", "k2") if c.contains(k)]
    assert survivors and c.fetch(survivors[-1]) is not None and c.stats["disk_hits"] == 1
    c.evict("k4")
    assert not c.contains("k4")
    with pytest.raises(ValueError, match="prefix cache"):
        llm = LLMEngine(EngineConfig(model=CFG, num_pages=16, max_seqs=2, max_tokens_per_step=64, max_seq_len=128,
                                     enable_prefix_cache=False), weights=random_weights(CFG, "cpu", seed=1, dtype=torch.float32), device="cpu")
        Engine(llm).attach_kv_connector(c)


def test_host_tier_is_accounted_and_reclaimed_under_pressure(tmp_path):
    """Offloaded chunks held in host memory show in the ledger; another consumer of host memory that does not fit makes
    the connector spill to disk before anyone waits, and the chunks stay restorable."""
    from onnx_genai_b200.engine.memory import PressureTicket

    weights = random_weights(CFG, "cpu", seed=11, std=0.3, dtype=torch.float32)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, CFG.vocab, size=600).tolist()
    opt = GenerateOptions(max_new_tokens=4, ignore_eos=True)
    eng = _engine(weights)
    conn = LocalTieredConnector(str(tmp_path / "kv"), max_host_bytes=1 << 30)
    eng.attach_kv_connector(conn)
    first = eng.generate(prompt, opt)
    ledger = eng.llm.memory
    held = conn.host_bytes
    assert held > 0 and ledger.used("host", "kv_offload") == held
    ledger.limits["host"] = ledger.used("host") + 1000                         # almost nothing left for anyone else
    ticket = eng.host_pressure.request("workspace", held // 2 + 1000, "pinned staging")
    assert ticket.poll() == PressureTicket.GRANTED                              # the connector gave memory back instead of a wait
    assert conn.host_bytes < held and conn.stats["spilled"] >= 1 and ledger.used("host", "kv_offload") == conn.host_bytes
    assert ledger.used("host") <= ledger.limits["host"]
    for _ in range(3):
        eng.generate(rng.integers(0, CFG.vocab, size=500).tolist(), opt)
    again = eng.generate(prompt, opt)
    assert again.token_ids == first.token_ids and eng.kv_offload.tokens_restored >= 256


def test_restore_into_a_pool_that_runs_out_mid_chunk_leaves_no_unfilled_page_in_the_cache(tmp_path):
    """Adoption publishes pages under their prefix hashes before they are filled.  When the pool cannot hold a whole
    chunk, the pages adopted for the partial chunk must leave the prefix cache again: a later request with that prefix
    must not attach to K/V nobody wrote."""
    weights = random_weights(CFG, "cpu", seed=11, std=0.3, dtype=torch.float32)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, CFG.vocab, size=600).tolist()
    opt = GenerateOptions(max_new_tokens=4, ignore_eos=True)
    big = _engine(weights)
    conn = LocalTieredConnector(str(tmp_path / "kv"))
    big.attach_kv_connector(conn)
    first = big.generate(prompt, opt)
    assert big.kv_offload.chunks_stored == 2
    conn.flush()
    small = _engine(weights, num_pages=24)                 # one chunk is 16 pages: the second cannot be adopted whole
    small.attach_kv_connector(LocalTieredConnector(str(tmp_path / "kv")))
    restored = small.kv_offload.restore(prompt)
    assert restored == 256                                 # the whole first chunk, nothing of the second
    served = small.llm.core.prefix_peek(prompt)
    assert len(served) == 16                               # no page of the partial chunk stays published
    assert small.llm.core.num_free_pages == 24             # and they are free again (cached pages count as free)
    # a wrong-sized blob ends the run before anything is adopted
    other = _engine(weights)
    bad = LocalTieredConnector(str(tmp_path / "bad"))
    for key in chunk_keys(prompt[:512], other.kv_offload.tag if getattr(other, "kv_offload", None) else ""):
        bad.store(key, b"x" * 10)
    other.attach_kv_connector(bad)
    for key in chunk_keys(prompt[:512], other.kv_offload.tag):
        bad.store(key, b"x" * 10)
    assert other.kv_offload.restore(prompt) == 0 and len(other.llm.core.prefix_peek(prompt)) == 0
