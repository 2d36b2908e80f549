"""Public Engine API on CPU: package loading, device vs host sampling paths, seams, sessions, speculation."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.engine import processors as procs
from onnx_genai_b200.engine.api import Engine, GenerateOptions
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package
from onnx_genai_b200.speculative import NgramProposer, SpeculativeProposer

CFG = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                    rope_theta=1e4, tie_embeddings=True, qkv_bias=False, max_position=512)


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    w = random_weights(CFG, "cpu", seed=5, std=0.3, dtype=torch.float32)
    return export_package(CFG, w, str(tmp_path_factory.mktemp("pkg")))


def _engine(model_dir, **kw):
    return Engine.from_dir(model_dir, device="cpu", num_pages=128, max_seqs=8, max_tokens_per_step=128, **kw)


def test_from_dir_generate_text_and_ids(model_dir):
    eng = _engine(model_dir)
    ids = eng.tokenize("hello world")
    assert eng.detokenize(ids) == "hello world"
    res = eng.generate("hello world", GenerateOptions(max_new_tokens=8, ignore_eos=True))
    assert res.completion_tokens == 8 and res.finish_reason == "length" and res.prompt_tokens == len(ids)
    again = eng.generate(ids, GenerateOptions(max_new_tokens=8, ignore_eos=True))
    assert again.token_ids == res.token_ids
    streamed = [t for t, _, _ in eng.generate_stream(ids, GenerateOptions(max_new_tokens=8, ignore_eos=True))]
    assert streamed == res.token_ids


def test_host_path_matches_device_path_for_greedy(model_dir):
    eng = _engine(model_dir)
    base = eng.generate([5, 6, 7, 8], GenerateOptions(max_new_tokens=10, ignore_eos=True))
    # logprobs force the host path; greedy choice must be identical
    lp = eng.generate([5, 6, 7, 8], GenerateOptions(max_new_tokens=10, ignore_eos=True, logprobs=3))
    assert lp.token_ids == base.token_ids and len(lp.logprobs) == 10 and len(lp.logprobs[0][1]) == 3
    assert all(lp.logprobs[i][0] <= 0 for i in range(10))


def test_repetition_penalty_changes_output_and_custom_seams(model_dir):
    eng = _engine(model_dir)
    prompt = [9, 9, 9, 9, 9, 9]
    base = eng.generate(prompt, GenerateOptions(max_new_tokens=12, ignore_eos=True))
    pen = eng.generate(prompt, GenerateOptions(max_new_tokens=12, ignore_eos=True, repetition_penalty=5.0))
    assert pen.token_ids != base.token_ids

    class AlwaysSeven(procs.Sampler):
        def sample(self, logits, u):
            return 7

    forced = eng.generate(prompt, GenerateOptions(max_new_tokens=4, ignore_eos=True), sampler=AlwaysSeven())
    assert forced.token_ids == [7, 7, 7, 7]

    class Ban(procs.LogitProcessor):
        def process(self, token_ids, logits):
            logits[base.token_ids[0]] = -np.inf
            return logits

    banned = eng.generate(prompt, GenerateOptions(max_new_tokens=1, ignore_eos=True), processors=[Ban()])
    assert banned.token_ids[0] != base.token_ids[0]


def test_sampling_plan_predicate():
    chain = procs.build_processor_chain(GenerateOptions(greedy=False, temperature=0.7, top_p=0.9, top_k=50, min_p=0.05), 4)
    assert [type(p).__name__ for p in chain.processors] == ["Temperature", "TopKTopP", "MinP"]
    assert procs.device_sampling_plan(chain, GenerateOptions(greedy=False), False) == "sampled"
    assert procs.device_sampling_plan(chain, GenerateOptions(greedy=False), True) == "host"
    chain2 = procs.build_processor_chain(GenerateOptions(greedy=False, temperature=0.7, typical_p=0.5), 4)
    assert procs.device_sampling_plan(chain2, GenerateOptions(greedy=False), False) == "host"
    g = procs.build_processor_chain(GenerateOptions(greedy=True, temperature=0.7, top_p=0.5), 4)
    assert g.processors == [] and procs.device_sampling_plan(g, GenerateOptions(greedy=True), False) == "greedy"
    order = procs.build_processor_chain(GenerateOptions(greedy=False, repetition_penalty=1.1, frequency_penalty=0.1,
                                                        dry_multiplier=0.5, temperature=0.5, top_k=5, min_p=0.1, top_a=0.1,
                                                        typical_p=0.9, mirostat=True, xtc_probability=0.5), 0)
    assert [type(p).__name__ for p in order.processors] == ["RepetitionPenalty", "FrequencyPresencePenalty", "DryPenalty",
                                                            "Temperature", "TopKTopP", "MinP", "TopA", "TypicalP", "Mirostat", "Xtc"]


def test_stop_string_and_batch(model_dir):
    eng = _engine(model_dir)
    full = eng.generate("abc", GenerateOptions(max_new_tokens=12, ignore_eos=True))
    if len(full.text) >= 4:
        stop = full.text[2:4]
        cut = eng.generate("abc", GenerateOptions(max_new_tokens=12, ignore_eos=True, stop=(stop,)))
        assert cut.finish_reason == "stop" and stop not in cut.text and full.text.startswith(cut.text)
    outs = eng.generate_batch(["abc", "hello there", [1, 2, 3]], GenerateOptions(max_new_tokens=6, ignore_eos=True))
    assert [r.completion_tokens for r in outs] == [6, 6, 6]
    assert outs[0].token_ids == full.token_ids[:6]


def test_sessions_reuse_prefix_pages_and_rewind(model_dir):
    eng = _engine(model_dir)
    s = eng.create_session()
    first = eng.generate_in_session(s, list(range(10, 60)), GenerateOptions(max_new_tokens=6, ignore_eos=True))
    hits0 = eng.llm.core.prefix_hits
    cp = eng.checkpoint_session(s)
    second = eng.generate_in_session(s, [3, 4, 5], GenerateOptions(max_new_tokens=6, ignore_eos=True))
    assert eng.llm.core.prefix_hits > hits0                       # the first turn's pages were found again
    assert eng.session_len(s) == 50 + 6 + 3 + 6
    child = eng.fork_session(s)
    eng.restore_session(cp)
    assert eng.session_len(s) == 56 and eng.session_len(child) == 65
    redo = eng.generate_in_session(s, [3, 4, 5], GenerateOptions(max_new_tokens=6, ignore_eos=True))
    assert redo.token_ids == second.token_ids                      # same history -> same continuation
    eng.close_session(s)
    with pytest.raises(KeyError):
        eng.session_len(s)


def test_speculative_ngram_equals_plain_greedy(model_dir):
    plain = _engine(model_dir)
    spec = _engine(model_dir, max_draft_tokens=4)
    prompt = [11, 12, 13, 14] * 6
    want = plain.generate(prompt, GenerateOptions(max_new_tokens=24, ignore_eos=True))
    got = spec.generate(prompt, GenerateOptions(max_new_tokens=24, ignore_eos=True, speculative=True))
    assert got.token_ids == want.token_ids
    assert got.speculative.verification_steps > 0 and got.speculative.proposed_tokens > 0

    class Oracle(SpeculativeProposer):          # proposes the true continuation: everything is accepted
        def propose(self, token_ids, k):
            done = len(token_ids) - len(prompt)
            return np.asarray(want.token_ids[done:done + k], dtype=np.int32)

    spec.proposer_factory = Oracle
    fast = spec.generate(prompt, GenerateOptions(max_new_tokens=24, ignore_eos=True, speculative=True))
    assert fast.token_ids == want.token_ids
    assert fast.speculative.accepted_tokens == fast.speculative.proposed_tokens > 0
    assert fast.speculative.accepted_per_step > 2

    class Wrong(SpeculativeProposer):           # always wrong: every draft is rewound, output unchanged
        def propose(self, token_ids, k):
            return np.full(k, 299, dtype=np.int32)

    spec.proposer_factory = Wrong
    slow = spec.generate(prompt, GenerateOptions(max_new_tokens=24, ignore_eos=True, speculative=True))
    assert slow.token_ids == want.token_ids and slow.speculative.accepted_tokens == 0


def test_ngram_proposer():
    p = NgramProposer(max_ngram=3)
    assert p.propose([1, 2, 3, 9, 9, 1, 2, 3], 2).tolist() == [9, 9]
    assert p.propose([1, 2, 3], 4).tolist() == []


def test_draft_model_proposer_keeps_its_sequence_aligned_without_resubmitting(model_dir):
    """A draft engine with the target's own weights proposes the true continuation, so every draft is accepted; the
    proposer re-aligns its sequence after each verification by rewind + append (never by re-submitting the prompt)."""
    from onnx_genai_b200.speculative import DraftModelProposer

    plain = _engine(model_dir)
    spec = _engine(model_dir, max_draft_tokens=3)
    draft = _engine(model_dir)
    prompt = list(range(40, 75))
    want = plain.generate(prompt, GenerateOptions(max_new_tokens=20, ignore_eos=True))
    admitted = []
    real_add = draft.llm.add_request
    draft.llm.add_request = lambda *a, **k: (admitted.append(1), real_add(*a, **k))[1]
    spec.proposer_factory = lambda: DraftModelProposer(draft.llm)
    got = spec.generate(prompt, GenerateOptions(max_new_tokens=20, ignore_eos=True, speculative=True))
    assert got.token_ids == want.token_ids
    # everything is accepted except drafts that fall beyond the 20-token budget in the last step
    assert got.speculative.proposed_tokens - 3 <= got.speculative.accepted_tokens <= got.speculative.proposed_tokens
    assert got.speculative.accepted_per_step > 2
    assert len(admitted) == 1                     # one submission for the whole generation

    class HalfWrong(DraftModelProposer):          # corrupt the second draft token: rewind + append of the correction
        def propose(self, token_ids, k):
            out = super().propose(token_ids, k).copy()
            if len(out) > 1:
                out[1] = (int(out[1]) + 1) % 1000
            return out

    admitted.clear()
    spec.proposer_factory = lambda: HalfWrong(draft.llm)
    mixed = spec.generate(prompt, GenerateOptions(max_new_tokens=20, ignore_eos=True, speculative=True))
    assert mixed.token_ids == want.token_ids and 0 < mixed.speculative.accepted_tokens < mixed.speculative.proposed_tokens
    assert len(admitted) == 1


def test_draft_model_proposals_are_batched_across_sequences(model_dir):
    """Two requests decoded together share one draft engine: their drafts come from batched draft steps."""
    from onnx_genai_b200.speculative import DraftModelProposer

    plain = _engine(model_dir)
    spec = _engine(model_dir, max_draft_tokens=3)
    draft = _engine(model_dir)
    prompts = [list(range(40, 75)), list(range(100, 118))]
    opt = GenerateOptions(max_new_tokens=16, ignore_eos=True)
    want = plain.generate_batch(prompts, opt)
    spec.proposer_factory = lambda: DraftModelProposer(draft.llm)
    steps0 = draft.llm.steps
    got = spec.generate_batch(prompts, GenerateOptions(max_new_tokens=16, ignore_eos=True, speculative=True))
    assert [g.token_ids for g in got] == [w.token_ids for w in want]
    verify_steps = spec.llm.core.spec_steps
    # with per-sequence proposals the draft would need about 3 steps per sequence per verification step
    assert draft.llm.steps - steps0 < 3 * verify_steps


def test_fill_in_the_middle_prompt_uses_the_models_sentinels(model_dir):
    eng = _engine(model_dir)
    prompt = eng.fim_prompt("def add(a, b):\n    return ", "\n\nprint(add(1, 2))")
    assert prompt.startswith("<|fim_prefix|>def add") and "<|fim_suffix|>\n\nprint" in prompt and prompt.endswith("<|fim_middle|>")
    ids = eng.tokenize(prompt)
    tok = eng.tokenizer
    assert ids[0] == tok.token_to_id("<|fim_prefix|>") and ids[-1] == tok.token_to_id("<|fim_middle|>")   # sentinels are single tokens
    res = eng.generate_fim("x = ", " + 1", GenerateOptions(max_new_tokens=5, ignore_eos=True))
    assert res.completion_tokens == 5
