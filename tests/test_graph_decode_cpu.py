"""Decode through the generic graph executor: the oracle for the fast path, and the route for unrecognised graphs."""
import os

import numpy as np
import pytest
import torch

from onnx_genai_b200.engine.api import Engine, GenerateOptions
from onnx_genai_b200.engine.graph_decode import GraphDecodeSession
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


@pytest.mark.parametrize("int4, bias", [(False, True), (True, False)])
def test_same_package_two_executors_same_greedy_tokens(tmp_path, int4, bias):
    cfg = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                        rope_theta=1e4, tie_embeddings=not int4, qkv_bias=bias, max_position=128,
                        weight_format="int4" if int4 else "bf16")
    w = random_weights(cfg, "cpu", seed=11, std=0.3, dtype=torch.float32)
    d = export_package(cfg, w, str(tmp_path / "pkg"))
    eng = Engine.from_dir(d, device="cpu", num_pages=32, max_seqs=2, max_tokens_per_step=64)
    prompt = [5, 17, 200, 42, 42, 7, 99, 1, 250, 13, 8, 77, 3, 150, 21, 64, 33, 2]            # crosses a 16-token page
    want = eng.generate(prompt, GenerateOptions(max_new_tokens=12, ignore_eos=True)).token_ids
    sess = GraphDecodeSession.from_dir(d)
    assert sess.generate(prompt, 12) == want
    # KV threading: feeding token by token, all at once, or after a rewind gives the same logits
    a = GraphDecodeSession.from_dir(d)
    whole = a.feed(prompt)
    b = GraphDecodeSession.from_dir(d)
    step = torch.stack([b.feed([t])[0] for t in prompt])
    assert torch.allclose(whole, step, atol=2e-4)
    b.rewind(10)
    assert b.length == 10 and torch.allclose(b.feed(prompt[10:]), whole[10:], atol=2e-4)
    with pytest.raises(ValueError, match="cannot rewind to 99"):
        b.rewind(99)


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "fixtures", "tiny-llm", "model.onnx.textproto")),
                    reason="the upstream tiny-llm fixture is not available on this machine")
def test_upstream_gpt2_style_fixture_decodes_with_consistent_kv():
    """A decoder the pattern matcher does not lower (LayerNorm, learned positions, fused Attention op, text-format ONNX)."""
    d = os.path.join(REF, "tests", "fixtures", "tiny-llm")
    sess = GraphDecodeSession.from_dir(d)
    assert sess.pos_in == "position_ids" and sess.kv_in == ["past_key_values.0.key", "past_key_values.0.value"]
    prompt = [3, 9, 27, 1, 14]
    toks = sess.generate(prompt, 6)
    assert len(toks) == 6 and all(0 <= t < 32 for t in toks)
    full = GraphDecodeSession.from_dir(d)
    logits = full.feed(prompt + toks[:-1])                      # one pass over everything
    assert [int(torch.argmax(logits[len(prompt) - 1 + i])) for i in range(6)] == toks


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-native-scalar-gqa")),
                    reason="the upstream tiny decoder fixtures are not available on this machine")
def test_upstream_tiny_decoders_reproduce_their_pinned_tokens():
    """Greedy tokens that the upstream project pins in its own tests (crates/onnx-genai-engine/tests/native_engine.rs:38,341)."""
    fixtures = os.path.join(REF, "tests", "fixtures")
    assert GraphDecodeSession.from_dir(os.path.join(fixtures, "tiny-native-scalar-gqa")).generate([0], 4) == [1, 1, 1, 1]
    assert GraphDecodeSession.from_dir(os.path.join(fixtures, "tiny-native-engine")).generate([0], 3) == [1, 1, 1]
    # packed q|k|v GroupQueryAttention with in-op rotary embedding: cached steps equal one full pass
    d = os.path.join(fixtures, "tiny-llm-sharedbuffer")
    toks = GraphDecodeSession.from_dir(d).generate([3, 9, 27], 5)
    logits = GraphDecodeSession.from_dir(d).feed([3, 9, 27] + toks[:-1])
    assert [int(torch.argmax(logits[2 + i])) for i in range(5)] == toks


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "fixtures", "tiny-llm-scatter", "model.onnx.textproto")),
                    reason="the upstream static-cache fixture is not available on this machine")
def test_static_cache_decoder_steps_equal_one_full_pass():
    """Fixed-size caches written by TensorScatter at ``write_indices``, attention bounded by ``nonpad_kv_seqlen``."""
    from onnx_genai_b200.engine.graph_decode import StaticCacheDecodeSession
    from onnx_genai_b200.package.onnx_text import load_any

    path = os.path.join(REF, "tests", "fixtures", "tiny-llm-scatter", "model.onnx.textproto")
    sess = StaticCacheDecodeSession(load_any(path))
    toks = sess.generate([3, 9, 27], 5)
    assert sess.capacity == 16 and len(sess.tokens) == 7
    full = StaticCacheDecodeSession(load_any(path))
    logits = full.feed([3, 9, 27] + toks[:-1])
    assert [int(torch.argmax(logits[2 + i])) for i in range(5)] == toks
    assert all(tuple(v.shape) == (1, 16, 16) for v in full.cache.values())        # shapes never change
    with pytest.raises(ValueError, match="exceed the cache length 16"):
        full.feed(list(range(12)))
    with pytest.raises(ValueError, match="not a static-cache decoder"):
        StaticCacheDecodeSession(load_any(os.path.join(REF, "tests", "fixtures", "tiny-llm", "model.onnx.textproto")))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-mtp-full", "mtp")),
                    reason="the upstream target + MTP head fixture is not available on this machine")
@pytest.mark.parametrize("k", [1, 3])
def test_onnx_mtp_head_speculation_equals_plain_greedy(k):
    from onnx_genai_b200.engine.graph_decode import GraphMtpSpeculator

    d = os.path.join(REF, "tests", "fixtures", "tiny-mtp-full")
    for prompt in ([3, 9, 27], [1], [5, 5, 5, 5, 5, 5]):
        want = GraphDecodeSession.from_dir(d).generate(prompt, 8)
        spec = GraphMtpSpeculator.from_dir(d, draft_tokens=k)
        assert spec.generate(prompt, 8) == want
        st = spec.stats
        assert st["proposed"] > 0 and 0 <= st["accepted"] <= st["proposed"] and st["target_passes"] <= 9
        assert spec.target.length == len(prompt) + 8 - 1 or spec.target.length == len(prompt) + 8   # the cache holds no rejected draft


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-deepseek-v2-qmoe-attention")),
                    reason="the upstream QMoE fixture is not available on this machine")
def test_upstream_qmoe_decoder_reproduces_its_pinned_tokens():
    """Integer-quantised mixture of experts (fused interleaved SwiGLU) as a graph operator; tokens pinned upstream in
    crates/onnx-genai-engine/tests/deepseek_v2_tiny_qmoe_native_e2e.rs:16-17."""
    d = os.path.join(REF, "tests", "fixtures", "tiny-deepseek-v2-qmoe-attention")
    assert GraphDecodeSession.from_dir(d).generate([3], 8) == [11] * 8


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-llm-scatter")),
                    reason="the upstream tiny decoder fixtures are not available on this machine")
def test_one_model_exported_four_ways_gives_the_same_tokens():
    """The upstream tiny LLM exists with a fused Attention operator, with explicit IO names, with packed-QKV
    GroupQueryAttention over shared buffers, and with a reasoning template: every export decodes to the same tokens."""
    from onnx_genai_b200.engine.graph_decode import StaticCacheDecodeSession, open_decode_session

    fixtures = os.path.join(REF, "tests", "fixtures")
    runs = {}
    for name in ("tiny-llm", "tiny-llm-explicit-io", "tiny-llm-sharedbuffer", "tiny-reasoning"):
        sess = open_decode_session(os.path.join(fixtures, name))
        runs[name] = sess.generate([3, 9, 27], 6)
    assert isinstance(open_decode_session(os.path.join(fixtures, "tiny-llm-scatter")), StaticCacheDecodeSession)
    assert len({tuple(v) for v in runs.values()}) == 1, runs


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-native-sub4-engine")),
                    reason="the upstream sub-4-bit fixture is not available on this machine")
def test_upstream_block_quantised_decoder_with_batchless_logits():
    """A decoder whose logits come from ``pkg.nxrt::BlockQuantizedMatMul`` (mxfp4) and have no batch axis: the all-zero
    weight leaves the bias, so every step picks token 1 (crates/onnx-genai-engine/tests/native_engine.rs uses this fixture)."""
    from onnx_genai_b200.engine.graph_decode import open_decode_session

    sess = open_decode_session(os.path.join(REF, "tests", "fixtures", "tiny-native-sub4-engine"))
    assert sess.generate([0], 4) == [1, 1, 1, 1]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-glm52-qmoe-indexshare")),
                    reason="the upstream sparse-attention fixture is not available on this machine")
def test_upstream_sparse_attention_decoder_reproduces_its_manifest_tokens():
    """A GLM-style decoder with a learned top-8 indexer feeding ``pkg.nxrt::IndexShare`` and QMoE layers: prompt and
    expected tokens come from the manifest beside the graph.  Past eight cached tokens the selection decides the result,
    and the indexer's ReLU-gated scores tie at zero, so TopK's lower-index tie rule is part of what this pins."""
    import json

    from onnx_genai_b200.engine.graph_decode import open_decode_session

    d = os.path.join(REF, "tests", "fixtures", "tiny-glm52-qmoe-indexshare")
    with open(os.path.join(d, "manifest.json")) as f:
        manifest = json.load(f)
    want = manifest["expected_tokens"]
    assert len(want) > 8
    assert open_decode_session(d).generate(manifest["prompt_ids"], len(want)) == want


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-multiaxis-state-decoder")),
                    reason="the upstream stateful decoder fixture is not available on this machine")
def test_hybrid_decoder_with_recurrent_state_and_three_axis_positions():
    """The upstream fixture's logits are a one-hot at (sum of the three position axes + sum of both recurrent states), its
    states grow by 1 and 2 per call, and its KV layers are numbered 3 and 11: the chosen token shows whether positions,
    state and cache were threaded right, and that a rewind recomputes the state instead of keeping a stale one."""
    from onnx_genai_b200.package.onnx_text import load_any

    model = load_any(os.path.join(REF, "tests", "fixtures", "tiny-multiaxis-state-decoder", "decoder.onnx.textproto"))
    with pytest.raises(ValueError, match="routed_sequence"):
        GraphDecodeSession(model)
    routed = lambda past, n: torch.zeros(1, n, 1)
    io = {"kv_inputs": ["past.3.key", "past.3.value", "past.11.key", "past.11.value"],
          "kv_outputs": ["present.3.key", "present.3.value", "present.11.key", "present.11.value"],
          "state_pairs": [{"input": "state_a.in", "output": "state_a.out"}, {"input": "state_b.in", "output": "state_b.out"}]}
    for spec in (io, None):                                       # declared, and found by the .in / .out naming
        s = GraphDecodeSession(model, io=spec, extra_feeds={"routed_sequence": routed})
        assert s.state_in == ["state_a.in", "state_b.in"] and len(s.kv_in) == 4
        assert s.feed([5, 6, 7]).argmax(-1).tolist() == [0, 3, 6]                  # 3 axes x position, zero state
        assert s.feed([9]).argmax(-1).tolist() == [3 * 3 + 2 + 4]                  # one call later: states (1, 1) and (2, 2)
        assert s.past["past.11.value"].reshape(-1).tolist() == [16.0, 17.0, 18.0, 20.0]
        s.rewind(2)                                                                # state cannot be cut: tokens re-fed from zero
        assert s.length == 2 and s.state["state_a.in"].tolist() == [[1.0, 1.0]]
        assert s.feed([1]).argmax(-1).tolist() == [3 * 2 + 2 + 4]
        assert s.past["past.3.key"].reshape(-1).tolist() == [5.0, 6.0, 1.0]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-eagle3")),
                    reason="the upstream drafter fixtures are not available on this machine")
@pytest.mark.parametrize("name, hidden_inputs, outputs", [
    ("tiny-eagle3", {"inputs_embeds": 16, "fused_hidden": 48, "recycled_hidden": 16}, ["draft_logits", "next_hidden"]),
    ("tiny-qwen35-mtp", {"inputs_embeds": 16, "hidden_states": 16}, ["mtp_hidden"]),
])
def test_upstream_drafter_heads_run_and_are_causal(name, hidden_inputs, outputs):
    """The EAGLE-3 and MTP drafter graphs take hidden-state inputs and a KV cache of their own.  Both were exported with
    mask-building constants that only hold for an empty cache, so they are exercised from an empty cache: every output
    has one row per position, and a position's row does not change when later positions are appended."""
    from onnx_genai_b200.package.graph_executor import GraphExecutor
    from onnx_genai_b200.package.onnx_text import load_any

    ex = GraphExecutor(load_any(os.path.join(REF, "tests", "fixtures", name, "model.onnx.textproto")), "cpu")
    g = torch.Generator().manual_seed(3)
    full = {k: torch.randn(1, 3, w, generator=g) for k, w in hidden_inputs.items()}
    empty = torch.zeros(1, 1, 0, 8)

    def call(n):
        feeds = {k: v[:, :n] for k, v in full.items()}
        feeds.update({"attention_mask": torch.ones(1, n, dtype=torch.int64), "position_ids": torch.arange(n)[None],
                      "past_key_values.0.key": empty, "past_key_values.0.value": empty})
        return ex.run(feeds)

    three, two, one = call(3), call(2), call(1)
    for o in outputs:
        assert three[o].shape[:2] == (1, 3) and bool(torch.isfinite(three[o]).all())
        assert torch.allclose(three[o][:, :2], two[o], atol=1e-5) and torch.allclose(two[o][:, :1], one[o], atol=1e-5), o
        assert not torch.allclose(three[o][:, 2], three[o][:, 1])
    assert three["present.0.key"].shape == (1, 1, 3, 8) and torch.allclose(three["present.0.key"][:, :, :2], two["present.0.key"], atol=1e-6)


def test_recurrent_decoder_steps_like_it_prefills():
    """A decoder with no attention cache at all -- a causal short convolution and gated-delta linear attention, both
    carrying state through ``X.in`` / ``X.out`` ports: token-by-token decoding gives the logits of one prefill call."""
    from onnx_genai_b200.package import onnx_pb as pb

    rng = np.random.default_rng(4)
    vocab, hidden, heads, dk, dv, taps = 20, 16, 2, 4, 8, 4
    f = lambda *shape: (rng.standard_normal(shape) * 0.4).astype(np.float32)
    inits = {"embed": f(vocab, hidden), "conv_w": f(hidden, 1, taps), "conv_b": f(hidden), "wq": f(hidden, heads * dk), "wk": f(hidden, heads * dk),
             "wv": f(hidden, heads * dv), "wd": f(hidden, heads), "wb": f(hidden, heads), "head": f(heads * dv, vocab)}
    N = lambda op, ins, outs, domain="", **attrs: pb.Node(op_type=op, inputs=ins, outputs=outs, name=outs[0], domain=domain, attrs=attrs)
    nodes = [N("Gather", ["embed", "input_ids"], ["x"]), N("Transpose", ["x"], ["x_cf"], perm=[0, 2, 1]),
             N("CausalConvWithState", ["x_cf", "conv_w", "conv_b", "conv.in"], ["y_cf", "conv.out"], "com.microsoft", activation="silu"),
             N("Transpose", ["y_cf"], ["y"], perm=[0, 2, 1]), N("MatMul", ["y", "wq"], ["q"]), N("MatMul", ["y", "wk"], ["k_raw"]),
             N("LpNormalization", ["k_raw"], ["k"], axis=-1, p=2),          # one key head group per row is enough for the test's purpose
             N("MatMul", ["y", "wv"], ["v"]), N("MatMul", ["y", "wd"], ["d_raw"]), N("Softplus", ["d_raw"], ["d_pos"]), N("Neg", ["d_pos"], ["decay"]),
             N("MatMul", ["y", "wb"], ["b_raw"]), N("Sigmoid", ["b_raw"], ["beta"]),
             N("LinearAttention", ["q", "k", "v", "mem.in", "decay", "beta"], ["o", "mem.out"], "com.microsoft", q_num_heads=heads, kv_num_heads=heads,
               update_rule="gated_delta"),
             N("MatMul", ["o", "head"], ["logits"])]
    vi = lambda name, dt, shape: pb.ValueInfo(name, dt, shape)
    graph = pb.Graph(name="recurrent", nodes=nodes,
                     initializers={k: pb.Tensor(name=k, dims=tuple(v.shape), data_type=pb.FLOAT, array=v) for k, v in inits.items()},
                     inputs=[vi("input_ids", pb.INT64, (1, "seq")), vi("conv.in", pb.FLOAT, (1, hidden, taps - 1)), vi("mem.in", pb.FLOAT, (1, heads, dk, dv))],
                     outputs=[vi("logits", pb.FLOAT, (1, "seq", vocab)), vi("conv.out", pb.FLOAT, (1, hidden, taps - 1)), vi("mem.out", pb.FLOAT, (1, heads, dk, dv))])
    model = pb.Model(graph=graph)
    model.opsets = {"": 21, "com.microsoft": 1}
    tokens = [3, 17, 5, 5, 9, 0, 12, 8]
    whole = GraphDecodeSession(model)
    assert whole.state_in == ["conv.in", "mem.in"] and whole.kv_in == []
    full = whole.feed(tokens)
    stepped = GraphDecodeSession(model)
    rows = torch.cat([stepped.feed(tokens[:3])] + [stepped.feed([t]) for t in tokens[3:]])
    assert torch.allclose(rows, full, atol=1e-5) and float(full.abs().max()) > 1e-3
    assert torch.allclose(stepped.state["mem.in"], whole.state["mem.in"], atol=1e-5)
    stepped.rewind(5)                                            # recomputed from the start, then continued
    assert torch.allclose(stepped.feed(tokens[5:]), full[5:], atol=1e-5)
    assert GraphDecodeSession(model).generate(tokens[:2], 4) == GraphDecodeSession(model).generate(tokens[:2], 4)
