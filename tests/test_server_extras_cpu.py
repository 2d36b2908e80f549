"""Embeddings, reasoning blocks, the multi-model registry and the debug endpoints."""
import numpy as np
import pytest
from fastapi.testclient import TestClient

from onnx_genai_b200 import reasoning
from onnx_genai_b200.bench.config_bench import _export
from onnx_genai_b200.engine.api import Engine
from onnx_genai_b200.server.app import create_app
from onnx_genai_b200.server.registry import ModelRegistry, RegistryApp


def test_reasoning_detection_split_and_streaming():
    tmpl = "{% for m in messages %}{{ m.content }}{% endfor %}{% if add_generation_prompt %}<|im_start|>assistant\n<think>\n{% endif %} ... </think>"
    d = reasoning.detect(tmpl)
    assert d == reasoning.ReasoningDelimiters("<think>", "</think>", prefilled=True)
    assert reasoning.detect("{{ messages }}") is None
    assert reasoning.split("step 1\nstep 2</think>\n\nThe answer is 4.", d) == ("step 1\nstep 2", "The answer is 4.")
    assert reasoning.split("still thinking", d) == ("still thinking", "")
    plain = reasoning.ReasoningDelimiters("<think>", "</think>")
    assert reasoning.split("<think>a</think>b", plain) == ("a", "b")
    assert reasoning.split("no block here", plain) == (None, "no block here")
    sp = reasoning.StreamSplitter(plain)
    r_all, a_all = "", ""
    for piece in ["<th", "ink>rea", "son</th", "ink>ans", "wer"]:          # tags arrive split across deltas
        r, a = sp.feed(piece)
        r_all, a_all = r_all + r, a_all + a
    r, a = sp.flush()
    assert (r_all + r, a_all + a) == ("reason", "answer")


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = []
    for name in ("alpha", "beta"):
        d = tmp_path_factory.mktemp(name)
        _export("tiny-llama", str(d), "fp32", layers=1)
        out.append(str(d))
    return out


def test_embeddings_endpoint_matches_engine_embed(dirs):
    eng = Engine.from_dir(dirs[0], device="cpu", max_seqs=4, max_seq_len=128)
    direct = eng.embed(["hello world", "goodbye"])
    assert direct.shape == (2, 256) and np.allclose(np.linalg.norm(direct, axis=1), 1.0, atol=1e-5)
    assert not np.allclose(direct[0], direct[1])
    with TestClient(create_app(eng, model_name="tiny", enable_debug_endpoints=True)) as client:
        r = client.post("/v1/embeddings", json={"model": "tiny", "input": ["hello world", "goodbye"]})
        assert r.status_code == 200, r.text
        data = r.json()["data"]
        got = np.array([d["embedding"] for d in data], dtype=np.float32)
        assert np.allclose(got, direct, atol=1e-5) and r.json()["usage"]["prompt_tokens"] > 0
        assert client.post("/v1/embeddings", json={"input": []}).status_code == 400
        # generation still works beside embedding traffic, and the debug endpoints answer
        g = client.post("/v1/completions", json={"model": "tiny", "prompt": "hi", "max_tokens": 4})
        assert g.status_code == 200 and g.json()["usage"]["completion_tokens"] == 4
        prof = client.get("/v1/debug/profile").json()
        assert prof["engine_steps"] > 0 and "launch_counts" in prof
        assert "sessions" in client.get("/v1/debug/sessions").json()
        assert "traceEvents" in client.get("/v1/debug/trace/perfetto").json()


def test_registry_loads_on_demand_and_evicts_least_recently_used(dirs):
    reg = ModelRegistry({"alpha": dirs[0], "beta": dirs[1]}, max_loaded=1,
                        loader=lambda path: Engine.from_dir(path, device="cpu", max_seqs=2, max_seq_len=64))
    with TestClient(RegistryApp(reg)) as client:
        listing = client.get("/v1/models").json()["data"]
        assert [m["id"] for m in listing] == ["alpha", "beta"] and not any(m["loaded"] for m in listing)
        for name in ("alpha", "beta", "alpha"):
            r = client.post("/v1/completions", json={"model": name, "prompt": "x", "max_tokens": 2})
            assert r.status_code == 200 and r.json()["model"] == name, r.text
        assert reg.loads == 3 and reg.evictions == 2 and list(reg.loaded) == ["alpha"]
        r = client.post("/v1/completions", json={"prompt": "x", "max_tokens": 1})          # no model named: the default
        assert r.status_code == 200 and r.json()["model"] == "alpha" and reg.loads == 3
        missing = client.post("/v1/completions", json={"model": "gamma", "prompt": "x"})
        assert missing.status_code == 404 and "available: alpha, beta" in missing.text
    assert not reg.loaded                                                                   # shutdown released everything


def test_admin_endpoints_and_media_routes(dirs):
    reg = ModelRegistry({"alpha": dirs[0], "beta": dirs[1]}, max_loaded=2, enable_debug_endpoints=True,
                        loader=lambda path: Engine.from_dir(path, device="cpu", max_seqs=2, max_seq_len=64))
    with TestClient(RegistryApp(reg)) as client:
        assert client.get("/v1/admin/models").status_code == 404                       # disabled unless asked for
    with TestClient(RegistryApp(reg, enable_admin_endpoints=True)) as client:
        assert [m["loaded"] for m in client.get("/v1/admin/models").json()["models"]] == [False, False]
        assert client.post("/v1/admin/models/alpha/load").json() == {"id": "alpha", "loaded": True, "action": "load"}
        assert client.post("/v1/admin/models/beta/warmup").json()["loaded"] is True
        listing = client.get("/v1/admin/models").json()
        assert [m["loaded"] for m in listing["models"]] == [True, True] and listing["loads"] == 2
        assert client.delete("/v1/admin/models/alpha").json() == {"id": "alpha", "loaded": False}
        assert list(reg.loaded) == ["beta"]
        assert client.post("/v1/admin/models/gamma/load").status_code == 404
        # media routes answer with the reason; the stage summary endpoint exists beside the Perfetto export
        r = client.post("/v1/audio/speech", json={"model": "beta", "input": "hi"})
        assert r.status_code == 501 and "decoder-only text models" in r.text
        assert client.post("/v1/images/generations", json={"model": "beta", "prompt": "x"}).status_code == 501
        assert "stages" in client.get("/v1/debug/trace?model=beta").json()


def test_reasoning_effort_reaches_the_chat_template_and_is_validated(tmp_path):
    import torch
    from fastapi.testclient import TestClient

    from onnx_genai_b200.engine.api import Engine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights
    from onnx_genai_b200.package.export import export_package
    from onnx_genai_b200.server.app import create_app

    cfg = DecoderConfig(name="t", num_layers=1, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                        rope_theta=1e4, tie_embeddings=True, max_position=512)
    d = export_package(cfg, random_weights(cfg, "cpu", seed=5, std=0.3, dtype=torch.float32), str(tmp_path / "pkg"))
    eng = Engine.from_dir(d, device="cpu", num_pages=64, max_seqs=4, max_tokens_per_step=128)
    eng.chat_template = ("{% if reasoning_effort is defined %}effort={{ reasoning_effort }}\n{% endif %}"
                         "{% for m in messages %}{{ m['content'] }}\n{% endfor %}")
    seen = []
    real = eng.apply_chat_template
    eng.apply_chat_template = lambda *a, **k: seen.append(real(*a, **k)) or seen[-1]
    with TestClient(create_app(eng, model_name="tiny", default_reasoning_effort="low")) as c:
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "temperature": 0}
        assert c.post("/v1/chat/completions", json=body).status_code == 200
        assert c.post("/v1/chat/completions", json={**body, "reasoning_effort": "high"}).status_code == 200
        r = c.post("/v1/chat/completions", json={**body, "reasoning_effort": "extreme"})
        assert r.status_code == 400 and "low, medium or high" in r.text
    assert seen[0].startswith("effort=low") and seen[1].startswith("effort=high")


def test_serve_reads_a_models_config_with_per_model_flags(tmp_path, monkeypatch):
    import subprocess
    import sys

    import uvicorn
    import yaml

    from onnx_genai_b200 import cli

    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    for out in (a, b):
        r = subprocess.run([sys.executable, "-m", "onnx_genai_b200", "export", "--preset", "tiny-llama", "--layers", "1", "--out", out],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    cfg = tmp_path / "models.yaml"
    cfg.write_text(yaml.safe_dump({"models": {"small": "a", "quantised-kv": {"path": "b", "kv-cache-dtype": "int8", "max-batch": 3}}}, sort_keys=False))
    captured = {}
    monkeypatch.setattr(uvicorn, "run", lambda app, **kw: captured.update(app=app, **kw))
    assert cli.main(["serve", "--models-config", str(cfg), "--device", "cpu", "--addr", "127.0.0.1:0", "--max-loaded-models", "2"]) == 0
    reg = captured["app"].registry
    assert reg.names() == ["small", "quantised-kv"]
    entry = reg.acquire("quantised-kv")
    try:
        assert entry["engine"].llm.cfg.kv_dtype == "int8" and entry["engine"].llm.cfg.max_seqs == 3
    finally:
        reg.release(entry)
    small = reg.acquire("small")
    assert small["engine"].llm.cfg.kv_dtype == "bf16"
    reg.release(small)
    empty = tmp_path / "empty.yaml"
    empty.write_text("models: {}\n")
    assert cli.main(["serve", "--models-config", str(empty), "--device", "cpu"]) == 2
