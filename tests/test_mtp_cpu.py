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
