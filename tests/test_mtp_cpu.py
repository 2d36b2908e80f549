"""MTP proposer: head arithmetic, persistence, and the engine's hidden-state hand-off."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.api import GenerateOptions
from onnx_genai_b200.speculative import SpeculativeProposer
from onnx_genai_b200.speculative.mtp import MtpHead, MtpProposer, attach_mtp
from test_api_cpu import CFG, _engine, model_dir  # noqa: F401  (fixture)


def test_head_batches_round_trips_and_checks_shapes(tmp_path):
    torch.manual_seed(0)
    embed = torch.randn(50, 16)
    head = MtpHead.random(embed, embed, inter=24, seed=3, std=0.3)
    h, tok = torch.randn(5, 16), torch.tensor([1, 2, 3, 4, 5])
    together = head.draft(h, tok, 3)
    assert together.shape == (5, 3)
    for i in range(5):
        assert together[i].tolist() == head.draft(h[i:i + 1], tok[i:i + 1], 3)[0].tolist()
    # plain restatement of one head step
    w = head.w
    rms = lambda x: x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6)
    z = np.concatenate([rms(h.numpy()), rms(embed[tok].numpy())], -1) @ w["fuse"].numpy().T
    m = rms(z)
    g = m @ w["gate"].numpy().T
    z = z + ((g / (1 + np.exp(-g))) * (m @ w["up"].numpy().T)) @ w["down"].numpy().T
    assert (rms(z) @ embed.numpy().T).argmax(-1).tolist() == together[:, 0].tolist()
    path = str(tmp_path / "mtp.safetensors")
    head.save(path)
    again = MtpHead.load(path, embed, embed)
    assert again.draft(h, tok, 3).tolist() == together.tolist() and again.inter == 24
    with pytest.raises(ValueError, match="does not match the target's embedding width 32"):
        MtpHead.load(path, torch.randn(50, 32), torch.randn(50, 32))
    with pytest.raises(ValueError, match="missing tensors"):
        MtpHead({"fuse": torch.zeros(16, 32)}, embed, embed)


def test_mtp_speculation_equals_plain_greedy(model_dir):  # noqa: F811
    plain = _engine(model_dir)
    spec = _engine(model_dir, max_draft_tokens=3)
    head = attach_mtp(spec, seed=1)
    assert head.hidden == CFG.hidden
    prompt = [5, 6, 7, 8, 9, 10, 11]
    want = plain.generate(prompt, GenerateOptions(max_new_tokens=20, ignore_eos=True))
    got = spec.generate(prompt, GenerateOptions(max_new_tokens=20, ignore_eos=True, speculative=True))
    assert got.token_ids == want.token_ids
    assert got.speculative.verification_steps > 0 and got.speculative.proposed_tokens >= 3 * (got.speculative.verification_steps - 1)
    for p in (prompt[::-1], prompt * 3):
        assert spec.generate(p, GenerateOptions(max_new_tokens=12, ignore_eos=True, speculative=True)).token_ids == \
            plain.generate(p, GenerateOptions(max_new_tokens=12, ignore_eos=True)).token_ids
    assert spec.llm.proposers == {}
    # sequences that share a head are drafted in one pass
    props = [MtpProposer(head), MtpProposer(head), MtpProposer(head)]
    props[0].observe(torch.randn(CFG.hidden))
    props[2].observe(torch.randn(CFG.hidden))
    drafts = MtpProposer.propose_many(props, [[1, 2], [3], [4, 5]], 3)
    assert [len(d) for d in drafts] == [3, 0, 3] and drafts[0].tolist() == props[0].propose([1, 2], 3).tolist()


def test_engine_hands_over_the_row_of_the_last_committed_token(model_dir):  # noqa: F811
    plain = _engine(model_dir)
    prompt = [21, 22, 23, 24, 25]
    want = plain.generate(prompt, GenerateOptions(max_new_tokens=16, ignore_eos=True)).token_ids
    spec = _engine(model_dir, max_draft_tokens=3)
    lm_head = spec.llm.model.w.lm_head
    seen = []

    class Recording(SpeculativeProposer):
        wants_hidden = True

        def __init__(self):
            self.hidden = None

        def observe(self, hidden):
            self.hidden = hidden

        def propose(self, token_ids, k):
            if self.hidden is not None:
                seen.append((int((lm_head.float() @ self.hidden.float()).argmax()), int(token_ids[-1])))
            done = len(token_ids) - len(prompt)
            # alternate between fully right and half right drafts so that every accepted count occurs
            draft = list(want[done:done + k])
            if done % 2 and len(draft) > 1:
                draft[1] = (draft[1] + 1) % CFG.vocab
            return np.asarray(draft, dtype=np.int32)

    spec.proposer_factory = Recording
    got = spec.generate(prompt, GenerateOptions(max_new_tokens=16, ignore_eos=True, speculative=True))
    assert got.token_ids == want
    assert len(seen) >= 4 and all(a == b for a, b in seen)
    assert 0 < got.speculative.accepted_tokens < got.speculative.proposed_tokens


def test_a_package_with_an_mtp_head_uses_it(model_dir, tmp_path):  # noqa: F811
    import os
    import shutil

    pkg = str(tmp_path / "pkg")
    shutil.copytree(model_dir, pkg)
    probe = _engine(pkg)
    MtpHead.random(probe.llm.model.w.embed, probe.llm.model.w.lm_head, seed=2).save(os.path.join(pkg, "mtp_head.safetensors"))
    eng = _engine(pkg, max_draft_tokens=2)
    assert isinstance(eng.proposer_factory(), MtpProposer)
    assert _engine(pkg).proposer_factory is None          # no drafting configured: the head is not loaded
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    assert eng.generate(prompt, GenerateOptions(max_new_tokens=10, ignore_eos=True, speculative=True)).token_ids == \
        probe.generate(prompt, GenerateOptions(max_new_tokens=10, ignore_eos=True)).token_ids


def test_eagle3_head_reads_three_layer_taps_and_keeps_greedy_output(model_dir):  # noqa: F811
    from onnx_genai_b200.speculative.mtp import Eagle3Head, Eagle3Proposer, attach_eagle3

    big = CFG.replace(num_layers=6)
    from onnx_genai_b200.models.decoder import random_weights
    from onnx_genai_b200.package.export import export_package
    import tempfile

    w = random_weights(big, "cpu", seed=9, std=0.3, dtype=torch.float32)
    with tempfile.TemporaryDirectory() as tmp:
        d = export_package(big, w, tmp)
        plain = _engine(d)
        spec = _engine(d, max_draft_tokens=3)
        head = attach_eagle3(spec, seed=4)
        assert head.tap_layers == [1, 3, 5] and spec.llm.model.tap_layers == [1, 3, 5]
        assert isinstance(spec.proposer_factory(), Eagle3Proposer)
        prompt = [9, 8, 7, 6, 5, 4, 3, 2, 1]
        want = plain.generate(prompt, GenerateOptions(max_new_tokens=14, ignore_eos=True))
        got = spec.generate(prompt, GenerateOptions(max_new_tokens=14, ignore_eos=True, speculative=True))
        assert got.token_ids == want.token_ids and got.speculative.proposed_tokens > 0
        # the taps are the residual stream entering those layers: a model cut after l layers ends with exactly that state
        import dataclasses

        from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine

        def last_prompt_state(cfg, weights, taps=()):
            eng = LLMEngine(EngineConfig(model=cfg, num_pages=32, max_seqs=2, max_tokens_per_step=64, max_seq_len=128), weights=weights,
                            device="cpu")
            eng.model.set_hidden_taps(taps)
            eng.add_request(np.asarray(prompt, dtype=np.int32), 1)
            eng.step()
            return eng.model

        full = last_prompt_state(big, w, head.tap_layers)
        for l in head.tap_layers:
            cut = last_prompt_state(big.replace(num_layers=l), dataclasses.replace(w, layers=w.layers[:l]))
            assert torch.allclose(full.taps[l][0], cut.x_last[0], atol=1e-5), l
    with pytest.raises(ValueError, match="three layers"):
        Eagle3Head.random(torch.randn(10, 8), torch.randn(10, 8), [1, 2])
    with pytest.raises(ValueError, match="must lie in"):
        spec.llm.model.set_hidden_taps([6])


def test_shared_kv_head_attends_over_the_targets_pages(model_dir):  # noqa: F811
    from onnx_genai_b200.ops import reference
    from onnx_genai_b200.speculative.mtp import SharedKvHead, SharedKvProposer, attach_shared_kv

    plain = _engine(model_dir)
    spec = _engine(model_dir, max_draft_tokens=2)
    head = attach_shared_kv(spec, seed=6)
    assert isinstance(spec.proposer_factory(), SharedKvProposer) and head.layer == -1
    prompt = list(range(40, 75))                                   # 35 tokens: more than two pages of context
    want = plain.generate(prompt, GenerateOptions(max_new_tokens=10, ignore_eos=True))
    got = spec.generate(prompt, GenerateOptions(max_new_tokens=10, ignore_eos=True, speculative=True))
    assert got.token_ids == want.token_ids and got.speculative.proposed_tokens > 0
    # the attention read is the target's own: drafting from a dense restatement over the gathered pages gives the same tokens
    llm = spec.llm
    sid = llm.add_request(np.asarray(prompt, dtype=np.int32), 4, temperature=0.0, ignore_eos=True)
    prop = llm.proposers[sid] = SharedKvProposer(head)
    llm.step()                                                     # prefill: one token sampled, 35 tokens cached
    toks = llm.core.seq_tokens(sid)
    prop.bind(llm, sid)
    drafts = SharedKvProposer.propose_many([prop], [toks], 2)[0]
    ctx = len(toks) - 1
    pages = llm.core.seq_pages(sid)[: -(-ctx // 16)]
    k_all, v_all = reference._gather_kv(llm.kv.pools[-1], torch.from_numpy(pages), ctx)
    w, m = head.w, llm.model
    rms = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    h, tok, mine = prop.hidden[None].float(), int(toks[-1]), []
    for j in range(2):
        z = torch.cat([rms(h), rms(m.w.embed[tok][None].float())], -1) @ w["fuse"].T
        q = reference.apply_rope((rms(z) @ w["q_proj"].T).view(1, m.hq, m.d), torch.tensor([ctx + j]), m.cos_sin, m.rotary_dim)[0]
        g = m.hq // m.hkv
        o = torch.cat([torch.softmax((q[hh] @ k_all[hh // g].T) * m.scale, -1) @ v_all[hh // g] for hh in range(m.hq)])
        z = z + o[None] @ w["o_proj"].T
        mm = rms(z)
        z = z + (torch.nn.functional.silu(mm @ w["gate"].T) * (mm @ w["up"].T)) @ w["down"].T
        tok = int((rms(z) @ m.w.lm_head.T.float()).argmax())
        mine.append(tok)
        h = z
    assert drafts.tolist() == mine
    llm.core.release(sid)
    llm.proposers.pop(sid, None)
    with pytest.raises(ValueError, match="q_proj is"):
        SharedKvHead.random(torch.randn(10, 8), torch.randn(10, 8), 2, 4).__class__(
            {**{n: torch.zeros(1) for n in SharedKvHead.NAMES}, "fuse": torch.zeros(8, 16), "gate": torch.zeros(4, 8),
             "q_proj": torch.zeros(3, 8)}, torch.randn(10, 8), torch.randn(10, 8), 2, 4)
