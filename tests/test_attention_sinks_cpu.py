"""Sliding window with attention sinks: the mask, the C++ CPU kernel, page release in the scheduler core, and generation."""
import numpy as np
import pytest
import torch

from onnx_genai_b200 import metadata as md
from onnx_genai_b200.engine.core import Core, CoreConfig
from onnx_genai_b200.ops import cpu as cpu_ops
from onnx_genai_b200.ops import reference as ref


def _dense(q, k, v, hq, hkv, d, ctx, window, sink):
    """Plain attention of the last rows of a sequence with the window-plus-sinks mask written out by hand."""
    t = q.shape[0]
    g = hq // hkv
    out = torch.zeros(t, hq * d)
    for r in range(t):
        qpos = ctx - t + r
        keep = [j for j in range(qpos + 1) if window <= 0 or j > qpos - window or j < sink]
        for h in range(hq):
            kk, vv = k[h // g, keep], v[h // g, keep]
            p = torch.softmax(kk @ q[r, h * d:(h + 1) * d] / d ** 0.5, dim=0)
            out[r, h * d:(h + 1) * d] = p @ vv
    return out


@pytest.mark.parametrize("window,sink", [(0, 0), (24, 0), (24, 16), (40, 32), (200, 16)])
def test_reference_and_cpu_kernel_apply_window_plus_sinks(window, sink):
    torch.manual_seed(3)
    hq, hkv, d, ctx, t = 4, 2, 16, 90, 5
    n_pages = (ctx + 15) // 16
    pool = torch.randn(n_pages + 2, hkv, 2, 16, d)
    table = torch.randperm(n_pages + 2)[:n_pages].to(torch.int32)[None]
    k = pool[table[0].long(), :, 0].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
    v = pool[table[0].long(), :, 1].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
    q = torch.randn(t, hq * d)
    want = _dense(q, k, v, hq, hkv, d, ctx, window, sink)
    ctx_t, cu = torch.tensor([ctx], dtype=torch.int32), torch.tensor([0, t], dtype=torch.int32)
    got = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, window=window, sink=sink)
    assert torch.allclose(got, want, atol=1e-5)
    # pages wholly between the sinks and the window of the first query row may be gone
    if window > 0:
        holes = table.clone()
        lo, hi = (sink + 15) // 16, max(0, ctx - t - window + 1) // 16
        if hi > lo:
            holes[0, lo:hi] = -1
            assert torch.allclose(ref.paged_attention(q, pool, holes, ctx_t, cu, hq, hkv, d, window=window, sink=sink), want, atol=1e-5)
            table = holes
    if cpu_ops.available():
        got = cpu_ops.paged_attention(q, pool.contiguous(), table, ctx_t, cu, hq, hkv, d, window=window, sink=sink)
        assert torch.allclose(got, want, atol=1e-5)


def test_core_releases_pages_between_sinks_and_window_and_refuses_deep_rewinds():
    core = Core(CoreConfig(num_pages=64, num_host_pages=0, max_seqs=4, max_tokens_per_step=64, max_pages_per_seq=32,
                           prefill_chunk=64, enable_prefix_cache=False))
    core.set_window(32, 4)                                    # 4 sink tokens -> the first page stays
    sid = core.add_request(list(range(1, 41)), max_new_tokens=200, ignore_eos=True)
    plan = np.zeros(core.layout.total_words, dtype=np.int32)
    sampled = np.full(4, 7, dtype=np.int32)
    for _ in range(150):
        assert core.build_step(plan.ctypes.data) >= 1
        core.commit_step(sampled.ctypes.data, 1)
    length = core.seq_len(sid)
    assert length == 40 + 150
    pages = core.seq_pages(sid)
    released = [i for i, p in enumerate(pages) if p < 0]
    assert released and released[0] == 1                      # page 0 holds the sinks
    assert released == list(range(1, released[-1] + 1))
    # the newest released page ends at or below (computed - window - one page of slack)
    assert (released[-1] + 1) * 16 <= (length - 1) - 32 - 16
    assert (released[-1] + 2) * 16 > (length - 1) - 32 - 16 - 16
    assert all(p >= 0 for p in pages[released[-1] + 1:])
    assert core.released_pages(sid) == len(released)
    assert 64 - core.num_free_pages == sum(1 for p in pages if p >= 0)
    # the page table handed to the kernels carries the holes as -1
    core.build_step(plan.ctypes.data)
    L = core.layout
    table = plan[L.page_table:L.page_table + len(pages)]
    assert [int(x) for x in table[:len(pages)]] == [int(x) for x in core.seq_pages(sid)][:len(pages)]
    core.commit_step(sampled.ctypes.data, 1)
    assert not core.rewind(sid, 20)                           # keys 16.. are gone: cannot look at them again
    assert core.rewind(sid, length - 2)
    core.release(sid)
    assert core.num_free_pages == 64


def test_metadata_carries_window_and_sinks():
    doc = {"schema_version": "v1", "model": {"attention": {"type": "group_query_attention", "sliding_window": 4096, "sink_tokens": 4}}}
    m = md.parse(doc)
    assert m.sliding_window == 4096 and m.sink_tokens == 4
    assert md.parse({"model": {"attention": {"sink_tokens": 4}}}).sink_tokens == 0          # no window: sinks mean nothing
    with pytest.raises(md.MetadataError, match="sliding_window"):
        md.parse({"model": {"attention": {"sliding_window": 0}}})


def test_generation_is_the_same_whether_or_not_unseen_pages_are_released():
    """A sliding-window model with sinks, run through the engine: releasing the pages between the sinks and the window
    changes the memory held, not one token -- and differs from what full attention would produce."""
    import dataclasses

    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights

    full = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96,
                         vocab=97, rope_theta=1e4, tie_embeddings=True, weight_format="bf16", max_position=512)
    swa = dataclasses.replace(full, sliding_window=32, attention_sinks=4)
    assert swa.sink_len == 16 and full.sink_len == 0
    w = random_weights(full, "cpu", seed=5, std=0.3, dtype=torch.float32)
    prompts = [list(range(3, 60)), [5, 9, 11]]
    outs = {}
    for name, cfg, release in (("full", full, True), ("keep", swa, False), ("release", swa, True)):
        eng = LLMEngine(EngineConfig(model=cfg, num_pages=64, max_seqs=4, max_tokens_per_step=64, max_seq_len=400,
                                     release_window_pages=release, enable_prefix_cache=False), weights=w, device="cpu")
        sids = [eng.add_request(p, max_new_tokens=150, ignore_eos=True) for p in prompts]
        low = eng.core.num_free_pages
        while eng.core.has_work:
            eng.step()
            low = min(low, eng.core.num_free_pages)
        outs[name] = ([list(eng.core.seq_tokens(s)) for s in sids], 64 - low)
    assert outs["keep"][0] == outs["release"][0]
    assert outs["keep"][0] != outs["full"][0]
    assert outs["release"][1] < outs["keep"][1] - 6          # (57 + 150) / 16 = 13 pages against 1 sink + ~4 window pages
