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
