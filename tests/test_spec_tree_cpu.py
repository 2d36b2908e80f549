"""Tree speculation core: structure, masks, acceptance, KV retention and greedy equivalence."""
import numpy as np
import pytest

from onnx_genai_b200.speculative.tree import (PathScorer, SpecTree, ancestor_attention_mask, greedy_decode_with_trees,
                                              kv_retention_plan, relative_position_ids, verify_tree)

V = 11


def toy_logits(ctx):
    """Deterministic next-token function with some structure (depends on the last two tokens)."""
    a, b = (ctx[-1], ctx[-2]) if len(ctx) > 1 else (ctx[-1], 0)
    out = np.zeros(V, np.float32)
    out[(3 * a + b + 1) % V] = 2.0
    out[(a + 5) % V] = 1.0
    return out


def greedy(prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(toy_logits(toks))))
    return toks[len(prompt):]


def test_structure_mask_and_positions():
    t = SpecTree.from_paths([[1, 2, 3], [1, 2, 4], [5]])
    assert [(n.token, n.parent, n.depth) for n in t.nodes] == [(1, -1, 0), (2, 0, 1), (3, 1, 2), (4, 1, 2), (5, -1, 0)]
    assert t.leaves() == [2, 3, 4] and t.path_to(3) == [0, 1, 3] and t.children(1) == [2, 3]
    m = ancestor_attention_mask(t)
    assert m.tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [1, 1, 1, 0, 0], [1, 1, 0, 1, 0], [0, 0, 0, 0, 1]]
    assert np.array_equal(m, np.tril(m))
    assert relative_position_ids(t, 10).tolist() == [10, 11, 12, 12, 10]
    with pytest.raises(ValueError, match="after its parent"):
        SpecTree().add(1, parent=0)
    cat = SpecTree.from_topk([[7, 8], [9, 1, 2], [3]], max_nodes=5)
    assert [(n.token, n.parent) for n in cat.nodes] == [(7, -1), (8, -1), (9, 0), (1, 0), (2, 0)]


def test_accept_walk_and_retention_plan():
    t = SpecTree.from_paths([[1, 2, 3], [1, 2, 4], [5]])
    # the target says: after ctx -> 1; after [1] -> 2; after [1,2] -> 4; after [1,2,4] -> 9
    acc = t.accept(1, [2, 4, 0, 9, 0])
    assert acc.path == [0, 1, 3] and acc.tokens.tolist() == [1, 2, 4, 9] and acc.accepted == 3
    plan = kv_retention_plan(t, acc, context_len=20)
    assert plan.keep == [0, 1, 3] and plan.moves == [(3, 2)] and plan.new_length == 23
    # nothing matches: only the target's own token is committed
    acc = t.accept(6, [0] * 5)
    assert acc.path == [] and acc.tokens.tolist() == [6]
    # the second root child can win too
    acc = t.accept(5, [0, 0, 0, 0, 7])
    assert acc.path == [4] and acc.tokens.tolist() == [5, 7]
    assert kv_retention_plan(t, acc, 3).moves == [(4, 0)]


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_tree_speculation_equals_plain_greedy(seed):
    rng = np.random.default_rng(seed)
    prompt = [int(x) for x in rng.integers(0, V, 4)]
    want = greedy(prompt, 24)

    def propose(toks):
        # a noisy oracle: the right continuation with a wrong sibling at each depth, sometimes a wrong spine
        truth = greedy(toks, 3)
        spine = [truth[0], truth[1] if rng.random() < 0.7 else (truth[1] + 1) % V, truth[2]]
        return SpecTree.from_paths([spine, [int(rng.integers(0, V))], [truth[0], int(rng.integers(0, V))]])

    got, passes = greedy_decode_with_trees(toy_logits, prompt, 24, propose)
    assert got == want
    assert passes < 24                      # some drafts were accepted, so fewer passes than tokens
    # an adversarial proposer never changes the output either
    got2, passes2 = greedy_decode_with_trees(toy_logits, prompt, 24, lambda toks: SpecTree.from_paths([[(toks[-1] + 7) % V]]))
    assert got2 == want and passes2 >= 12


def test_verify_tree_scores_every_node_with_its_own_path():
    ctx = [1, 2, 3]
    truth = greedy(ctx, 3)
    t = SpecTree.from_paths([[truth[0], truth[1], (truth[2] + 1) % V], [(truth[0] + 1) % V, 0]])
    scorer = PathScorer(toy_logits)
    acc, plan = verify_tree(ctx, t, scorer)
    assert acc.tokens.tolist() == truth and acc.path == [0, 1] and plan.new_length == 5 and scorer.calls == 1 + len(t)


def test_engine_verifies_a_tree_as_forked_branches_and_keeps_the_winner():
    """A proposer whose first path goes wrong after one token and whose second path is right: the forked branch wins,
    its state continues under the request's id, the output equals plain greedy decoding, fewer steps are taken, and
    every page returns to the pool."""
    import torch

    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights

    cfg = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=97,
                        rope_theta=1e4, tie_embeddings=True, qkv_bias=True, weight_format="bf16", max_position=512)
    w = random_weights(cfg, "cpu", seed=5, std=0.3, dtype=torch.float32)
    mk = lambda **kw: LLMEngine(EngineConfig(model=cfg, num_pages=48, max_seqs=8, max_tokens_per_step=128, max_seq_len=256,
                                             enable_prefix_cache=False, **kw), weights=w, device="cpu")
    prompts = [np.random.default_rng(i).integers(0, cfg.vocab, size=n).astype(np.int32) for i, n in enumerate((37, 21))]
    plain = mk()
    want = plain.generate([p for p in prompts], 24)
    plain_steps = plain.steps

    class OracleTree:
        """Knows the continuation; hides it on the second path of the tree."""
        def __init__(self, full):
            self.full = list(full)

        def propose_tree(self, toks, k):
            done = len(toks)
            nxt = self.full[done:done + k]
            if len(nxt) < 2:
                return SpecTree()
            wrong = lambda t: (int(t) + 1) % cfg.vocab
            return SpecTree.from_paths([[nxt[0], wrong(nxt[1])] + [wrong(t) for t in nxt[2:]], list(nxt), [wrong(nxt[0])]])

    eng = mk(max_draft_tokens=4)
    free0 = eng.core.num_free_pages
    ids = []
    for p, out in zip(prompts, want):
        sid = eng.add_request(p, 24)
        eng.proposers[sid] = OracleTree(list(p) + list(out))
        ids.append(sid)
    got = {i: [] for i in ids}
    while eng.has_work:
        for sid, tok, fin in eng.step().events:
            assert sid in got                                  # fork ids never surface
            got[sid].append(tok)
    for sid in ids:
        eng.core.release(sid)
    assert [got[i] for i in ids] == want
    assert eng.tree_branch_wins > 0 and eng.tree_branches >= 2 * eng.tree_branch_wins
    assert eng.steps < plain_steps
    assert eng.core.num_free_pages == free0 and not eng.tree_groups
