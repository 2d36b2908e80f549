"""Scheduling policies under pressure, on the CPU engine: priority preemption, a page-pressure stress with
interleaved arrivals, fair share between tenants, and the sampler's draw distribution."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.ops import cpu, reference

CFG = DecoderConfig(name="s", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96,
                    vocab=97, rope_theta=1e4, tie_embeddings=True, qkv_bias=True, weight_format="bf16", max_position=512)


@pytest.fixture(scope="module")
def weights():
    return random_weights(CFG, "cpu", seed=7, std=0.3, dtype=torch.float32)


def _engine(weights, **kw):
    base = dict(model=CFG, num_pages=64, max_seqs=8, max_tokens_per_step=64, max_seq_len=256, enable_prefix_cache=False)
    base.update(kw)
    return LLMEngine(EngineConfig(**base), weights=weights, device="cpu")


def _solo(weights, prompt, n):
    return _engine(weights).generate([prompt], n)[0]


def test_high_priority_request_preempts_and_both_match_their_solo_runs(weights):
    """A long low-priority request owns most of a small KV pool; an urgent one arrives mid-flight, takes its pages,
    finishes first, and the preempted request still produces exactly its solo output."""
    rng = np.random.default_rng(1)
    low_p = rng.integers(0, CFG.vocab, size=90).tolist()
    high_p = rng.integers(0, CFG.vocab, size=80).tolist()
    eng = _engine(weights, num_pages=12, policy="priority", max_seqs=4)          # 192 token slots for 90+40 and 80+10
    low = eng.add_request(np.asarray(low_p, dtype=np.int32), 40, priority=0)
    outs, order = {low: []}, []
    for _ in range(6):
        for sid, tok, fin in eng.step().events:
            outs[sid].append(tok)
    high = eng.add_request(np.asarray(high_p, dtype=np.int32), 10, priority=5)
    outs[high] = []
    while eng.has_work:
        for sid, tok, fin in eng.step().events:
            outs[sid].append(tok)
            if fin is not None:
                order.append(sid)
    assert order == [high, low]
    assert eng.core.num_preemptions > 0
    assert outs[high] == _solo(weights, high_p, 10)
    assert outs[low] == _solo(weights, low_p, 40)


@pytest.mark.parametrize("preempt,host_pages", [("recompute", 0), ("swap", 96)])
def test_page_pressure_stress_with_interleaved_arrivals(weights, preempt, host_pages):
    """Twelve requests arrive two steps apart into a pool that holds about three of them; every one of them must end
    with the tokens of its solo run, whatever was preempted on the way."""
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, CFG.vocab, size=int(n)).tolist() for n in rng.integers(12, 60, size=12)]
    eng = _engine(weights, num_pages=16, num_host_pages=host_pages, preempt=preempt, max_seqs=8)
    outs, ids, pending = {}, [], list(prompts)
    steps = 0
    while pending or eng.has_work:
        if pending and steps % 2 == 0:
            sid = eng.add_request(np.asarray(pending.pop(0), dtype=np.int32), 24)
            ids.append(sid)
            outs[sid] = []
        for sid, tok, fin in eng.step().events:
            outs[sid].append(tok)
        steps += 1
        assert steps < 4000
    assert eng.core.num_preemptions > 0
    for sid, prompt in zip(ids, prompts):
        assert outs[sid] == _solo(weights, prompt, 24), sid


def test_fair_share_serves_tenants_evenly(weights):
    """Tenant 0 floods the queue before tenant 1's requests arrive; under fair share tenant 1 is not starved."""
    rng = np.random.default_rng(3)
    eng = _engine(weights, policy="fair_share", max_seqs=2, num_pages=64)
    fcfs = _engine(weights, policy="fcfs", max_seqs=2, num_pages=64)
    finish = {}
    for e, tag in ((eng, "fair"), (fcfs, "fcfs")):
        owners = {}
        for i in range(6):
            owners[e.add_request(rng.integers(0, CFG.vocab, size=20).astype(np.int32), 8, tenant=0)] = 0
        for i in range(2):
            owners[e.add_request(rng.integers(0, CFG.vocab, size=20).astype(np.int32), 8, tenant=1)] = 1
        done = []
        while e.has_work:
            for sid, tok, fin in e.step().events:
                if fin is not None:
                    done.append(owners[sid])
        finish[tag] = done
    assert finish["fcfs"][-2:] == [1, 1]                       # arrival order: tenant 1 waits for all six
    first_t1 = finish["fair"].index(1)
    assert first_t1 <= 3, finish["fair"]                        # fair share: tenant 1 is served among the first few


@pytest.mark.skipif(not cpu.available(), reason="runtime library not built")
def test_sampler_draws_follow_the_filtered_distribution():
    """100 000 draws from one logits row under temperature 0.7 + top-k 8 + top-p 0.9: empirical frequencies match the
    renormalised filtered distribution (chi-square well under the 0.999 quantile for 7 degrees of freedom), and
    tokens outside the kept set never appear."""
    torch.manual_seed(0)
    vocab, draws = 64, 100_000
    logits = (torch.randn(1, vocab) * 2).expand(draws, vocab).contiguous()
    temp, k, p = 0.7, 8, 0.9
    u = torch.rand(draws, generator=torch.Generator().manual_seed(1))
    toks = cpu.sample(logits, torch.full((draws,), temp), torch.full((draws,), k, dtype=torch.int32), torch.full((draws,), p),
                      torch.zeros(draws), u)
    w = reference.sample_weights(logits[0], temp).double()
    order = torch.argsort(w, descending=True)
    kept = order[:k]
    csum = torch.cumsum(w[kept], 0)
    target = float(csum[-1]) * p
    n_keep = int(torch.searchsorted(csum, torch.tensor(target, dtype=csum.dtype))) + 1
    kept = kept[:n_keep]
    probs = (w[kept] / w[kept].sum()).numpy()
    counts = np.bincount(toks.numpy(), minlength=vocab)
    assert counts.sum() == draws and counts[[i for i in range(vocab) if i not in set(kept.tolist())]].sum() == 0
    chi2 = float((((counts[kept.numpy()] - draws * probs) ** 2) / (draws * probs)).sum())
    assert chi2 < 26.0, (chi2, n_keep)
    same = cpu.sample(logits[:100], torch.full((100,), temp), torch.full((100,), k, dtype=torch.int32), torch.full((100,), p),
                      torch.zeros(100), u[:100])
    assert torch.equal(same, toks[:100])                        # same uniforms -> same tokens


def test_pool_growth_adds_allocatable_pages():
    from onnx_genai_b200.engine.core import Core, CoreConfig

    core = Core(CoreConfig(num_pages=4, max_seqs=2, max_tokens_per_step=64, max_pages_per_seq=16, enable_prefix_cache=False))
    assert core.num_pages == 4 and core.num_free_pages == 4
    core.add_pages(6)
    assert core.num_pages == 10 and core.num_free_pages == 10
    core.add_pages(0)
    assert core.num_pages == 10
