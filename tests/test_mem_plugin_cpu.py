"""Memory plugin ABI: the host loader against a well-behaved plugin and against the ways a plugin can be wrong."""
import os
import shutil
import subprocess

import pytest
import torch

from onnx_genai_b200.utils.mem_plugin import MemPluginError, PluginAllocator

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "examples", "plugins", "arena_allocator.c")
pytestmark = pytest.mark.skipif(shutil.which("gcc") is None, reason="building the example plugin needs gcc")


def build(tmp_path, name, *defines):
    out = str(tmp_path / f"lib{name}.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-I", os.path.join(ROOT, "csrc", "abi"), *defines, SRC, "-o", out], check=True)
    return out


def test_current_plugin_allocates_accounts_and_limits(tmp_path):
    alloc = PluginAllocator(build(tmp_path, "arena"), byte_limit=1 << 20, purpose="test")
    assert alloc.name == "arena" and alloc.level == 1
    t = alloc.tensor((64, 128), torch.float32)
    assert t.data_ptr() % 64 == 0 and float(t.abs().sum()) == 0
    t += 3.0
    assert float(t.sum()) == 3.0 * 64 * 128
    st = alloc.stats()
    assert st["bytes_in_use"] == 64 * 128 * 4 and st["allocations_live"] == 1
    with pytest.raises(MemPluginError, match="out of memory") as e:
        alloc.allocate(2 << 20)                                     # beyond the byte limit the host passed down
    assert e.value.code == 1 and "in use" in str(e.value)
    with pytest.raises(MemPluginError, match="no trim capability") as e:
        alloc.trim()                                                # an absent optional slot is "unsupported", not a silent success
    assert e.value.code == 3
    with pytest.raises(MemPluginError, match="was not allocated through this plugin"):
        alloc.free(12345)
    alloc.free_tensor(t)
    assert alloc.stats()["bytes_in_use"] == 0 and alloc.stats()["bytes_peak"] == 64 * 128 * 4
    alloc.close()


def test_baseline_plugin_loads_at_its_own_level(tmp_path):
    alloc = PluginAllocator(build(tmp_path, "old", "-DPLUGIN_MINOR0"))
    assert alloc.level == 0
    a = alloc.allocate(4096, 256)
    assert a % 256 == 0
    with pytest.raises(MemPluginError, match="no stats capability"):
        alloc.stats()                                               # the slot lies beyond the prefix the old plugin wrote
    alloc.close()                                                   # frees what is still live, then unloads


def test_misbehaving_plugins_are_refused_at_load(tmp_path):
    with pytest.raises(MemPluginError, match=r"version negotiation failed: host speaks 1\.1, plugin answers 2\."):
        PluginAllocator(build(tmp_path, "v2", "-DPLUGIN_MAJOR=2"))
    with pytest.raises(MemPluginError, match="claims minor 1, which needs .* contradicts itself"):
        PluginAllocator(build(tmp_path, "liar", "-DPLUGIN_LIES"))
    with pytest.raises(MemPluginError, match="cannot load"):
        PluginAllocator(str(tmp_path / "missing.so"))
    empty = tmp_path / "empty.c"
    empty.write_text("int nothing(void) { return 0; }\n")
    out = str(tmp_path / "libempty.so")
    subprocess.run(["gcc", "-shared", "-fPIC", str(empty), "-o", out], check=True)
    with pytest.raises(MemPluginError, match="does not export OgbMemNegotiate"):
        PluginAllocator(out)
    flaky = PluginAllocator(build(tmp_path, "flaky", "-DPLUGIN_FAIL_AFTER=2"))
    flaky.allocate(64)
    with pytest.raises(MemPluginError, match="injected allocation failure"):
        flaky.allocate(64)
    flaky.close()


def test_engine_swap_space_comes_from_the_plugin(tmp_path):
    """Swap preemption with the host pages held in plugin memory: same tokens as a roomy engine, and the plugin saw the bytes."""
    import numpy as np

    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights

    cfg = DecoderConfig(name="p", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=97,
                        rope_theta=1e4, tie_embeddings=True, max_position=512)
    w = random_weights(cfg, "cpu", seed=3, std=0.3, dtype=torch.float32)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg.vocab, size=30).tolist() for _ in range(6)]
    mk = lambda **kw: LLMEngine(EngineConfig(model=cfg, max_seqs=8, max_tokens_per_step=64, max_seq_len=256, enable_prefix_cache=False, **kw),
                                weights=w, device="cpu")
    tight = mk(num_pages=14, num_host_pages=64, preempt="swap", host_allocator_plugin=build(tmp_path, "arena"))
    got = tight.generate(prompts, 20)
    assert tight.core.num_preemptions > 0 and got == mk(num_pages=128).generate(prompts, 20)
    st = tight.host_allocator.stats()
    want = sum(t.numel() * t.element_size() for t in tight.host_kv)
    assert st["bytes_in_use"] == want and st["allocations_live"] == cfg.num_layers
    assert [l.nbytes for l in tight.memory.leases if l.tag == "swap space"] == [want]
