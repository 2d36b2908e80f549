import pytest

from onnx_genai_b200.router import Router, prefix_hash
from onnx_genai_b200.utils.runtime_config import RuntimeConfig


def test_policy_affinity_prefix_least_loaded_and_health():
    r = Router(["http://a", "http://b", "http://c"])
    r.record_poll("http://a", {"kv_usage": 0.8, "queue_depth": 5})
    r.record_poll("http://b", {"kv_usage": 0.1, "queue_depth": 1, "prefix_hashes": []})
    r.record_poll("http://c", {"kv_usage": 0.5, "queue_depth": 0, "prefix_hashes": [prefix_hash("shared system prompt")]})
    assert r.pick().url == "http://b"                                        # least loaded
    assert r.pick(prompt_text="shared system prompt").url == "http://c"      # prefix co-location
    assert r.pick("s1").url == "http://b"
    r.record_poll("http://b", {"kv_usage": 0.99, "queue_depth": 50})
    assert r.pick("s1").url == "http://b"                                    # session affinity beats load
    for _ in range(3):
        r.record_poll("http://b", None)                                      # three missed polls -> demoted
    assert not r.nodes["http://b"].healthy
    assert r.sessions["s1"] != "http://b" and r.migrations[0].from_node == "http://b"
    r.drain("http://c")
    assert r.pick().url == "http://a"
    r.record_poll("http://b", {"kv_usage": 0.0, "queue_depth": 0})           # node returns
    assert r.nodes["http://b"].healthy and r.pick().url == "http://b"
    assert "onnx_genai_router_migrations_total 1" in r.metrics_text()


def test_runtime_config_env():
    cfg = RuntimeConfig.from_env({"ONNX_GENAI_CUDA_DEVICE": "3", "ONNX_GENAI_PROFILE": "1", "ONNX_GENAI_EP": "cuda"})
    assert cfg.cuda_device == 3 and cfg.profile and "ONNX_GENAI_EP" in cfg.ignored


def test_runtime_config_reaches_the_engine_loader(tmp_path, monkeypatch):
    """ONNX_GENAI_* variables are read by the engine loader (the caller's arguments win over them)."""
    import torch

    from onnx_genai_b200.engine.api import Engine
    from onnx_genai_b200.models.config import DecoderConfig
    from onnx_genai_b200.models.decoder import random_weights
    from onnx_genai_b200.package.export import export_package
    from onnx_genai_b200.utils import runtime_config as rc

    cfg = DecoderConfig(name="t", num_layers=1, hidden=32, num_heads=2, num_kv_heads=1, head_dim=16, intermediate=64, vocab=300,
                        rope_theta=1e4, tie_embeddings=True, max_position=128)
    d = export_package(cfg, random_weights(cfg, "cpu", seed=1, std=0.3, dtype=torch.float32), str(tmp_path / "pkg"))
    monkeypatch.setenv("ONNX_GENAI_CUDA_GQA_SPLITS", "4")
    monkeypatch.setenv("ONNX_GENAI_EP", "cuda")
    rc.runtime_config(refresh=True)
    try:
        eng = Engine.from_dir(d, device="cpu", num_pages=32, max_seqs=2, max_tokens_per_step=32)
        assert eng.llm.cfg.decode_splits == 4 and eng.llm.cfg.cuda_graphs is False
        assert Engine.from_dir(d, device="cpu", num_pages=32, max_seqs=2, max_tokens_per_step=32, decode_splits=2).llm.cfg.decode_splits == 2
        assert "ONNX_GENAI_EP" in rc.runtime_config().describe()["ignored"]
        monkeypatch.setenv("ONNX_GENAI_REQUIRE_CUDA", "1")
        rc.runtime_config(refresh=True)
        with pytest.raises(RuntimeError, match="ONNX_GENAI_REQUIRE_CUDA"):
            Engine.from_dir(d, device="cpu", num_pages=32, max_seqs=2, max_tokens_per_step=32)
    finally:
        monkeypatch.undo()
        rc.runtime_config(refresh=True)
