"""HTTP benchmark tools against a real server socket on 127.0.0.1."""
import socket
import threading
import time

import pytest
import torch

from onnx_genai_b200.bench import http_bench
from onnx_genai_b200.engine.api import Engine
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package.export import export_package
from onnx_genai_b200.server.app import create_app
from test_server_cpu import CFG


@pytest.fixture(scope="module")
def server_url(tmp_path_factory):
    import uvicorn

    w = random_weights(CFG, "cpu", seed=5, std=0.3, dtype=torch.float32)
    d = export_package(CFG, w, str(tmp_path_factory.mktemp("pkg")))
    eng = Engine.from_dir(d, device="cpu", num_pages=256, max_seqs=8, max_tokens_per_step=256)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(create_app(eng, model_name="tiny"), host="127.0.0.1", port=port, log_level="error"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()
    url = f"http://127.0.0.1:{port}"
    for _ in range(200):
        try:
            if http_bench.request_json(url, "GET", "/health", timeout=1.0) == {"status": "ok"}:
                break
        except Exception:
            time.sleep(0.05)
    else:
        pytest.fail("server did not come up")
    yield url
    server.should_exit = True
    thread.join(timeout=10)


def test_stream_once_measures_first_token_and_rate(server_url):
    r = http_bench.stream_once(server_url, {"model": "tiny", "prompt": "hello", "max_tokens": 8, "temperature": 0}, chat=False)
    assert r["ttft_ms"] > 0 and r["total_ms"] >= r["ttft_ms"] and r["completion_tokens"] == 8 and r["text"]
    with pytest.raises(RuntimeError, match="-> 4"):
        http_bench.stream_once(server_url, {"model": "tiny", "max_tokens": 8}, chat=False)


def test_compare_two_targets(server_url):
    rep = http_bench.compare({"a": server_url, "b": server_url}, ["hello there", "what is a page"], max_tokens=6, concurrency=2,
                             repeats=2, warmup=1, chat=False)
    for name in ("a", "b"):
        assert rep[name]["requests"] == 4 and rep[name]["errors"] == [] and rep[name]["model"] == "tiny"
        assert rep[name]["ttft_ms"]["n"] == 4 and rep[name]["aggregate_tok_s"] > 0 and rep[name]["decode_tok_s"]["p50"] > 0
    assert rep["ratio"]["of"] == "a / b" and rep["ratio"]["ttft"] > 0


def test_multiturn_with_and_without_session(server_url):
    with_s = http_bench.multiturn(server_url, turns=3, max_tokens=4, use_session=True)
    without = http_bench.multiturn(server_url, turns=3, max_tokens=4, use_session=False)
    for rep in (with_s, without):
        assert [t["turn"] for t in rep["turns"]] == [1, 2, 3] and all(t["completion_tokens"] == 4 for t in rep["turns"])
    # the server-side history grows in the session; the client-side history grows without it
    p_s = [t["prompt_tokens"] for t in with_s["turns"]]
    p_n = [t["prompt_tokens"] for t in without["turns"]]
    assert p_s[0] < p_s[1] < p_s[2] and p_n[0] < p_n[1] < p_n[2]
    assert http_bench.main(["multiturn", "--url", server_url, "--turns", "1", "--max-tokens", "2"]) == 0
