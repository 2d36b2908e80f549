"""HTTP surface driven in-process: completions, chat, SSE framing, sessions, tools, errors, metrics."""
import json

import pytest
import torch
from fastapi.testclient import TestClient

from onnx_genai_b200.engine.api import Engine
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package
from onnx_genai_b200.server import create_app
from onnx_genai_b200.server.tools import parse_tool_calls

CFG = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                    rope_theta=1e4, tie_embeddings=True, max_position=512)


@pytest.fixture(scope="module")
def client(tmp_path_factory):
    w = random_weights(CFG, "cpu", seed=5, std=0.3, dtype=torch.float32)
    d = export_package(CFG, w, str(tmp_path_factory.mktemp("pkg")))
    eng = Engine.from_dir(d, device="cpu", num_pages=128, max_seqs=8, max_tokens_per_step=128)
    with TestClient(create_app(eng, model_name="tiny", enable_debug_endpoints=True)) as c:
        yield c


def test_health_models_status(client):
    assert client.get("/health").json() == {"status": "ok"}
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    st = client.get("/v1/status").json()
    assert {"kv_usage", "queue_depth", "tokens_per_second", "batch_utilization", "node_id"} <= set(st)
    assert client.get("/v1/resources").json()["batching"]["continuous"] is True


def test_completion_and_determinism(client):
    body = {"model": "tiny", "prompt": "hello", "max_tokens": 6, "temperature": 0}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    assert a["choices"][0]["text"] == b["choices"][0]["text"]
    assert a["usage"]["completion_tokens"] <= 6 and a["object"] == "text_completion"


def test_chat_streaming_sse(client):
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "temperature": 0, "stream": True}
    with client.stream("POST", "/v1/chat/completions", json=body) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop") and "usage" in chunks[-1]
    plain = client.post("/v1/chat/completions", json={**body, "stream": False}).json()
    streamed = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    assert streamed == plain["choices"][0]["message"]["content"]


def test_logprobs_and_sampling_params(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 3,
                                                   "temperature": 0, "logprobs": True, "top_logprobs": 2}).json()
    lp = r["choices"][0]["logprobs"]["content"]
    assert len(lp) == r["usage"]["completion_tokens"] and len(lp[0]["top_logprobs"]) == 2
    r2 = client.post("/v1/completions", json={"prompt": "x", "max_tokens": 4, "temperature": 0.8, "top_p": 0.9, "top_k": 20,
                                               "seed": 7, "repetition_penalty": 1.2})
    assert r2.status_code == 200


def test_sessions_and_errors(client):
    sid = client.post("/v1/sessions").json()["id"]
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 3, "temperature": 0}, headers={"X-Session-Id": sid})
    assert r.status_code == 200
    assert client.delete(f"/v1/sessions/{sid}").json()["deleted"] is True
    assert client.delete(f"/v1/sessions/{sid}").status_code == 404
    assert client.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    assert client.post("/v1/completions", content=b"not json").status_code == 400
    assert client.post("/v1/embeddings", json={"input": "x"}).status_code == 200
    bad = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "image_url"}]}]})
    assert bad.status_code == 400 and "image_url needs a url" in bad.json()["detail"]
    bad = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "video", "video": "x"}]}]})
    assert bad.status_code == 400 and "not supported" in bad.json()["detail"]


def test_metrics_exposition(client):
    client.post("/v1/completions", json={"prompt": "m", "max_tokens": 2, "temperature": 0})
    text = client.get("/metrics").text
    assert 'onnx_genai_requests_total{endpoint="/v1/completions",status="200"}' in text
    assert "onnx_genai_ttft_seconds_bucket" in text and "onnx_genai_kv_pages_total" in text
    assert client.get("/v1/debug/kv").status_code == 200


def test_tool_call_parsing():
    calls = parse_tool_calls('ok <tool_call>{"name": "get_weather", "arguments": {"city": "Oslo"}}</tool_call> '
                             '<tool_call>{broken</tool_call>')
    assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo"}


def test_n_returns_independent_samples_and_shares_the_prompt(client):
    body = {"model": "tiny", "prompt": "once upon a time there was a", "max_tokens": 6, "temperature": 1.0, "seed": 3, "n": 3}
    r = client.post("/v1/completions", json=body)
    assert r.status_code == 200, r.text
    out = r.json()
    assert [c["index"] for c in out["choices"]] == [0, 1, 2] and out["usage"]["completion_tokens"] == 18
    assert len({c["text"] for c in out["choices"]}) >= 2                      # different seeds, different samples
    again = client.post("/v1/completions", json=body).json()
    assert [c["text"] for c in again["choices"]] == [c["text"] for c in out["choices"]]      # reproducible from the seed
    greedy = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                       "temperature": 0, "n": 2}).json()
    assert greedy["choices"][0]["message"]["content"] == greedy["choices"][1]["message"]["content"]
    assert client.post("/v1/completions", json={**body, "n": 0}).status_code == 400
    assert client.post("/v1/completions", json={**body, "stream": True}).status_code == 400
