"""Workflow executor: loops with carried state, branches, emits, session state, errors."""
import copy
import os

import numpy as np
import pytest

from onnx_genai_b200.engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession, run_workflow
from onnx_genai_b200.package.comfyui import import_comfyui
from test_comfyui_cpu import GRAPH
from test_workflow_cpu import DOC


def _diffusion_components(calls):
    sig = np.linspace(1.0, 0.0, 21)

    def denoiser(p):
        calls.append(("denoiser", int(p["step"][0])))
        return {"noise_pred": p["sample"] * 0.5 + p["encoder_hidden_states"].mean()}

    return {
        "schedule": lambda p: {"schedule": sig},
        "text_encoder": lambda p: {"encoder_hidden_states": p["input_ids"].astype(np.float32) / 10.0},
        "denoiser": denoiser,
        "guidance": lambda p: {"guided": p["unconditional"] + float(p["scale"][0]) * (p["conditional"] - p["unconditional"])},
        "solver_step": lambda p: {"next_state": p["sample"] + (p["schedule"][int(p["step"][0]) + 1] - p["schedule"][int(p["step"][0])]) * p["derivative"]},
        "continue_predicate": lambda p: {"continue": ~np.asarray(p["done"])},
        "vae_decoder": lambda p: {"image": np.repeat(np.repeat(p["latent"][:, :3], 8, axis=2), 8, axis=3)},
    }


def test_imported_diffusion_graph_runs_and_matches_a_plain_loop():
    doc = import_comfyui(GRAPH)
    calls = []
    comps = _diffusion_components(calls)
    rng = np.random.default_rng(0)
    noise = rng.standard_normal((2, 4, 64, 96)).astype(np.float32)
    pos, neg = np.array([[1, 2, 3]]), np.array([[4, 5, 6]])
    out = run_workflow(doc, comps, {"request.positive_ids": pos, "request.negative_ids": neg, "request.noise": noise})
    sig, x = np.linspace(1.0, 0.0, 21), noise.copy()
    cp, cn = (pos / 10.0).mean(), (neg / 10.0).mean()
    for i in range(20):
        d = (x * 0.5 + cn) + 8.0 * ((x * 0.5 + cp) - (x * 0.5 + cn))
        x = x + (sig[i + 1] - sig[i]) * d
    assert out["image"].shape == (2, 3, 512, 768)
    np.testing.assert_allclose(out["image"][:, :, ::8, ::8], x[:, :3], rtol=1e-5, atol=1e-5)
    assert len(calls) == 40 and calls[0] == ("denoiser", 0) and calls[-1] == ("denoiser", 19)
    # max_iterations from the request overrides the graph's step count
    calls.clear()
    run_workflow(doc, comps, {"request.positive_ids": pos, "request.negative_ids": neg, "request.noise": noise,
                              "request.max_iterations": np.array([3])})
    assert len(calls) == 6


def _decoder_components(vocab=8, eos=None):
    def lm(p):
        ids = np.asarray(p["input_ids"])
        logits = np.zeros((ids.shape[0], ids.shape[1], vocab), np.float32)
        logits[:, -1, (int(ids[0, -1]) + 1) % vocab] = 5.0
        return {"logits": logits}

    pick = lambda p: {"token": p["logits"][:, -1].argmax(-1)[:, None]}
    return {"lm": lm, "pick": pick, "pick_sampled": lambda p: {"token": p["logits"][:, -1].argmin(-1)[:, None]}}


def test_decoder_loop_greedy_branch_eos_and_stop():
    sess = WorkflowSession(copy.deepcopy(DOC), _decoder_components())
    out = sess.run({"request.input_ids": np.array([[1, 2]]), "request.max_new": np.array([5])})
    assert [int(t[0, 0]) for t in out["tokens"]] == [4, 5, 6, 7, 0]
    assert sess.stats["invocations"]["lm"] == 6 and sess.stats["invocations"]["pick"] == 6
    out = sess.run({"request.input_ids": np.array([[1, 2]]), "request.max_new": np.array([50])}, eos_token_ids=[6])
    assert [int(t[0, 0]) for t in out["tokens"]] == [4, 5, 6]
    seen = []
    out = sess.run({"request.input_ids": np.array([[1, 2]]), "request.max_new": np.array([50])},
                   on_emit=lambda name, v, mode: (seen.append((name, mode)), len(seen) < 2)[1])
    assert len(out["tokens"]) == 2 and seen == [("tokens", "append")] * 2
    # the default arm (sampling off the greedy flag) takes the other picker
    out = sess.run({"request.input_ids": np.array([[1, 2]]), "request.max_new": np.array([1]), "package.greedy": np.array([False])})
    assert int(out["tokens"][0][0, 0]) != 4


def test_session_cells_persist_and_checkpoint():
    doc = {"inputs": {"request.n": {"contract": {"dtype": "int64"}, "source": {"kind": "request"}, "required": True},
                      "package.zero": {"source": {"kind": "literal"}, "default": 0},
                      "package.on": {"source": {"kind": "literal"}, "default": True}},
           "outputs": {"total": {"contract": {"dtype": "int64"}}},
           "components": {"add": {"implementation": {"kind": "onnx", "artifact": "add.onnx"}}},
           "state": {"acc": {"scope": "session", "initializer": "package.zero"},
                     "go": {"scope": "invocation", "initializer": "package.on"}},
           "steps": [{"kind": "loop", "steps": [{"kind": "invoke", "component": "add", "inputs": {"a": "acc", "i": "it"},
                                                  "outputs": {"sum": "body.sum", "more": "body.more"}}],
                      "continue_when": "go", "max_iterations": "request.n", "iteration": {"value": "it"},
                      "carried": [{"cell": "acc", "next": "body.sum"}, {"cell": "go", "next": "body.more"}]},
                     {"kind": "emit", "value": "acc", "output": "total", "mode": "replace"}]}
    sess = WorkflowSession(doc, {"add": lambda p: {"sum": np.asarray(p["a"]) + 1, "more": np.array([True])}})
    assert int(sess.run({"request.n": np.array([3])})["total"][0]) == 3
    snap = sess.checkpoint()
    assert int(sess.run({"request.n": np.array([2])})["total"][0]) == 5
    sess.restore(snap)
    assert int(sess.run({"request.n": np.array([1])})["total"][0]) == 4
    sess.reset()
    assert int(sess.run({"request.n": np.array([1])})["total"][0]) == 1
    # the body's predicate ends the loop before the limit
    sess2 = WorkflowSession(doc, {"add": lambda p: {"sum": np.asarray(p["a"]) + 1, "more": np.array([int(p["i"][0]) < 1])}})
    assert int(sess2.run({"request.n": np.array([10])})["total"][0]) == 2


def test_errors_name_the_step_and_the_fix():
    with pytest.raises(WorkflowRuntimeError, match="no implementation bound for component\\(s\\) pick_sampled"):
        WorkflowSession(copy.deepcopy(DOC), {k: v for k, v in _decoder_components().items() if k != "pick_sampled"})
    sess = WorkflowSession(copy.deepcopy(DOC), _decoder_components() | {"pick": lambda p: {"tok": 1}})
    with pytest.raises(WorkflowRuntimeError, match="did not produce output port 'token'"):
        sess.run({"request.input_ids": np.array([[1]]), "request.max_new": np.array([1])})
    with pytest.raises(WorkflowRuntimeError, match="required input 'request.input_ids'"):
        WorkflowSession(copy.deepcopy(DOC), _decoder_components()).run({"request.max_new": np.array([1])})
    with pytest.raises(WorkflowRuntimeError, match="unknown input"):
        WorkflowSession(copy.deepcopy(DOC), _decoder_components()).run({"request.inputs": 1})
    bad = copy.deepcopy(DOC)
    bad["steps"][0]["steps"][0]["inputs"]["input_ids"] = "tokne"
    with pytest.raises(WorkflowRuntimeError, match="does not validate"):
        WorkflowSession(bad, _decoder_components())


FIXTURES = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")),
                        "tests", "fixtures", "onnx_genai_workflows")


def _synthetic_inputs(wf, rows=2):
    import torch

    feeds = {}
    for name, spec in wf.inputs.items():
        if spec["source"] in ("request", "application") and spec.get("default") is None:
            c = spec["contract"]
            shape = [s if isinstance(s, int) else rows for s in c.shape] or [1]
            feeds[name] = torch.rand(shape) if c.dtype.startswith("float") else (
                torch.ones(shape, dtype=torch.bool) if c.dtype == "bool" else torch.full(shape, 3, dtype=torch.int64))
    return feeds


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="the upstream workflow fixtures are not available on this machine")
@pytest.mark.parametrize("name, outputs", [("diffusion", {"latent": (2, 4, 2, 2), "image": (2, 3, 2, 2)}),
                                           ("diffusion_guided", {"latent": (2, 4, 4, 4), "image": (2, 3, 4, 4)}),
                                           ("codec", {"waveform": (2, 1, 2)}), ("masked", {"tokens": (2, 2)}),
                                           ("static_cache", {"logits": (2, 1, 8), "key_cache": (2, 8, 4)}), ("video", {}), ("decoder", {}),
                                           ("speech_wav", {"audio": (2, 2, 64)}), ("speech_wav_mixed_audio", {"waveform": (2, 1, 64)}),
                                           ("speech_wav_two_adapters", {"audio": (2, 2, 64)}), ("speech_wav_two_audio", {"audio": (2, 2, 64)})])
def test_upstream_workflow_packages_execute_end_to_end(name, outputs):
    """Whole packages of the upstream project -- text-format ONNX graphs for every model part and policy, wired by their
    workflow documents -- run unchanged: parsed, validated, every component on the generic graph executor."""
    import torch

    sess = WorkflowSession.from_package(os.path.join(FIXTURES, name))
    out = sess.run(_synthetic_inputs(sess.wf))
    for key, shape in outputs.items():
        assert tuple(out[key].shape) == shape, (key, tuple(out[key].shape))
    flat = [v for val in out.values() for v in (val if isinstance(val, list) else [val])]
    assert flat and all(bool(torch.isfinite(torch.as_tensor(v).float()).all()) for v in flat)
    assert sess.stats["invocations"] and (name not in ("diffusion", "diffusion_guided") or sess.stats["iterations"] >= 3)
    if name == "decoder":      # the whole token loop -- model, sampler, termination, cache bookkeeping -- is ONNX policy graphs
        assert len(out["tokens"]) == 3 and sess.stats["invocations"]["token_sampler"] >= 3
    # a second run of the same session gives the same result (invocation-scoped state starts over)
    again = sess.run(_synthetic_inputs(sess.wf)) if name in ("codec", "static_cache") else None
    if again is not None:
        assert set(again) == set(out)


def test_packages_with_unknown_adapter_components_say_what_to_supply(tmp_path):
    import yaml

    doc = {"pipeline": {"workflow": {"inputs": {"x": {"source": {"kind": "request"}}}, "outputs": {"y": {}},
                                     "components": {"telemetry": {"implementation": {"kind": "adapter", "abi": "onnx-genai.telemetry", "version": "1"}}},
                                     "steps": [{"kind": "invoke", "component": "telemetry", "inputs": {"v": "x"}, "outputs": {"o": "t"}},
                                               {"kind": "emit", "value": "t", "output": "y", "mode": "replace"}]}}}
    (tmp_path / "inference_metadata.yaml").write_text(yaml.safe_dump(doc))
    with pytest.raises(WorkflowRuntimeError, match=r"is a 'adapter' implementation \(onnx-genai.telemetry\), not an ONNX graph: pass a callable"):
        WorkflowSession.from_package(str(tmp_path))
    sess = WorkflowSession.from_package(str(tmp_path), components={"telemetry": lambda p: {"o": p["v"] * 2}})
    assert sess.run({"x": np.asarray([2.0])})["y"].tolist() == [4.0]


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="the upstream workflow fixtures are not available on this machine")
def test_upstream_vision_language_package_runs_from_image_bytes():
    """Encoded image -> declared preprocessing program (the image-preprocess adapter) -> vision encoder -> embedding merge ->
    decoder loop with ONNX sampler and termination policies -> tokens."""
    import io

    import torch
    from PIL import Image

    sess = WorkflowSession.from_package(os.path.join(FIXTURES, "vlm"))
    buf = io.BytesIO()
    Image.fromarray((np.random.default_rng(0).random((8, 8, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
    feeds = _synthetic_inputs(sess.wf)
    feeds["request.image"] = torch.from_numpy(np.frombuffer(buf.getvalue(), dtype=np.uint8).copy())
    out = sess.run(feeds)
    assert len(out["tokens"]) == 3 and sess.stats["invocations"]["image_preprocess"] == 1 and sess.stats["invocations"]["vision_encoder"] == 1
    feeds["request.image"] = torch.zeros(10, dtype=torch.uint8)
    with pytest.raises(Exception, match="cannot decode the image"):
        sess.run(feeds)


def test_grammar_guidance_adapter_walks_masks_and_forces():
    import torch

    from onnx_genai_b200.engine.constraints import grammar_guidance_adapter

    # state 0 accepts tokens 0,1 (-> 1); state 1 accepts only token 2 (-> 0)
    table = torch.tensor([[1, 1, -1], [-1, -1, 0]])
    ports = {"state": torch.tensor([0, 1]), "tokens": torch.tensor([[0, 2, 2], [2, 1, 0]]), "valid_length": torch.tensor([3, 3]),
             "transition_table": table}
    look = grammar_guidance_adapter("lookahead")(ports)
    assert look["next_state"].tolist() == [0, 1] and look["consumed_length"].tolist() == [2, 2]
    assert look["logits_mask"].tolist() == [[True, True, False], [False, False, True]]
    assert look["forced_tokens"].tolist() == [[0], [2]] and look["forced_length"].tolist() == [0, 1]
    clone = grammar_guidance_adapter("clone")(ports)
    assert clone["next_state"].tolist() == [0, 1] and clone["consumed_length"].tolist() == [0, 0]
    with pytest.raises(ValueError, match="token 2 at row 0, position 2 is not allowed in state 0"):
        grammar_guidance_adapter("commit")(ports)
    ok = grammar_guidance_adapter("commit")({**ports, "valid_length": torch.tensor([2, 2])})
    assert ok["consumed_length"].tolist() == [2, 2]
    with pytest.raises(ValueError, match="outside the table's 2 states"):
        grammar_guidance_adapter("clone")({**ports, "state": torch.tensor([0, 5])})
    with pytest.raises(ValueError, match="not clone, lookahead or commit"):
        grammar_guidance_adapter("peek")


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="the upstream workflow fixtures are not available on this machine")
def test_upstream_grammar_guided_speculative_package_runs():
    """Proposer and verifier graphs, grammar clone / lookahead / commit adapters over a transition table, ONNX acceptance and
    adaptive draft-length policies: the whole loop from the package's own document."""
    import torch

    sess = WorkflowSession.from_package(os.path.join(FIXTURES, "speculative"))
    rows, vocab = 2, 32
    table = torch.zeros(2, vocab, dtype=torch.int64)
    table[0, 5:] = 1
    table[1, :3] = -1
    feeds = {"request.tokens": torch.randint(0, vocab, (rows, 4), generator=torch.Generator().manual_seed(0)),
             "request.max_iterations": torch.tensor([3]), "request.grammar_state": torch.zeros(rows, dtype=torch.int64),
             "request.grammar_transition_table": table, "request.draft_ms": torch.ones(rows), "request.target_ms": torch.ones(rows) * 4,
             "request.verifier.past_key_values.0.key": torch.zeros(rows, 2, 0, 8),
             "request.verifier.past_key_values.0.value": torch.zeros(rows, 4, 0, 4)}
    out = sess.run(feeds)
    inv = sess.stats["invocations"]
    assert len(out["tokens"]) >= 2 and inv["grammar_clone"] == inv["grammar_lookahead"] == inv["grammar_commit"] == inv["verifier"] >= 2


COMFY_FIXTURE = os.path.join(os.path.dirname(os.path.dirname(FIXTURES)), "fixtures", "comfyui_workflows", "txt2img_sd15")


@pytest.mark.skipif(not os.path.exists(os.path.join(COMFY_FIXTURE, "reference.json")), reason="the upstream ComfyUI fixture is not available on this machine")
def test_upstream_text_to_image_package_reproduces_its_golden_latent_and_image():
    """The upstream converter's own package for a ComfyUI graph, with the pinned outputs it ships: seeded noise generated by
    an ONNX policy (64-bit integer hashing), four guided Euler steps, VAE decode -- all on the generic graph executor."""
    import json

    import torch

    with open(os.path.join(COMFY_FIXTURE, "reference.json"), encoding="utf-8") as f:
        ref = json.load(f)
    sess = WorkflowSession.from_package(COMFY_FIXTURE)
    out = sess.run({"request.input_ids": torch.tensor([ref["prompt_tokens"]]), "request.negative_input_ids": torch.tensor([ref["negative_tokens"]])})
    latent, image = torch.as_tensor(out["latent"]).float(), torch.as_tensor(out["image"]).float()
    assert list(latent.shape) == ref["latent_shape"] and list(image.shape) == ref["image_shape"]
    assert float((latent.reshape(-1) - torch.tensor(ref["latent"])).abs().max()) < ref["tolerance"]
    assert float((image.reshape(-1) - torch.tensor(ref["image"])).abs().max()) < ref["tolerance"]
    assert sess.stats["iterations"] == ref["steps"] and sess.stats["invocations"]["denoiser"] == 2 * ref["steps"]
    # the ComfyUI graph next to it goes through this package's own importer too
    from onnx_genai_b200.package.comfyui import import_comfyui

    with open(os.path.join(COMFY_FIXTURE, "workflow.json"), encoding="utf-8") as f:
        mine = import_comfyui(json.load(f))
    d = mine["generation"]["defaults"]
    assert (d["steps"], d["guidance_scale"], d["seed"], d["sampler"], d["scheduler"]) == (ref["steps"], ref["guidance_scale"], ref["seed"], "euler", "karras")
