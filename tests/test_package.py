"""ONNX wire codec, decoder graph export / structural lowering, metadata and package layouts."""
import json
import os

import numpy as np
import pytest
import torch
import yaml

from onnx_genai_b200 import metadata as md
from onnx_genai_b200 import package as pkg
from onnx_genai_b200.models.config import DecoderConfig
from onnx_genai_b200.models.decoder import random_weights
from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package.decoder_graph import GraphPatternError, lower_decoder
from onnx_genai_b200.package.export import export_package
from onnx_genai_b200.package.genai_config import import_genai_config

CFG = DecoderConfig(name="t", num_layers=2, hidden=64, num_heads=4, num_kv_heads=2, head_dim=16, intermediate=96, vocab=300,
                    rope_theta=1e4, tie_embeddings=True, qkv_bias=True, max_position=128)


def test_onnx_codec_roundtrip(tmp_path):
    g = pb.Graph(name="g")
    g.initializers["w"] = pb.Tensor("w", (3, 600), pb.FLOAT, np.arange(1800, dtype=np.float32).reshape(3, 600))
    g.initializers["small"] = pb.Tensor("small", (2,), pb.INT64, np.array([5, -7], dtype=np.int64))
    g.nodes.append(pb.Node("MatMul", ["x", "w"], ["y"], name="mm", attrs={"alpha": 0.5, "k": 3, "mode": "abc", "axes": [1, -2]}))
    g.inputs.append(pb.ValueInfo("x", pb.FLOAT, ("batch", 3)))
    g.outputs.append(pb.ValueInfo("y", pb.FLOAT, ("batch", 600)))
    path = str(tmp_path / "m.onnx")
    pb.save_model(pb.Model(graph=g, metadata={"k": "v"}), path)
    assert os.path.getsize(path + ".data") >= 7200            # the big tensor went to external data
    m = pb.load_model(path)
    assert m.metadata == {"k": "v"} and m.opsets["com.microsoft"] == 1
    assert np.array_equal(m.graph.initializers["w"].array, g.initializers["w"].array)
    assert m.graph.initializers["small"].array.tolist() == [5, -7]
    n = m.graph.nodes[0]
    assert n.op_type == "MatMul" and n.attrs["k"] == 3 and n.attrs["mode"] == "abc" and n.attrs["axes"] == [1, -2]
    assert abs(n.attrs["alpha"] - 0.5) < 1e-7
    assert m.graph.inputs[0].shape == ("batch", 3)


@pytest.mark.parametrize("int4", [False, True])
def test_export_then_lower_recovers_model(tmp_path, int4):
    w = random_weights(CFG, "cpu", seed=1, std=0.1, dtype=torch.float32)
    out = export_package(CFG, w, str(tmp_path / "pkg"), int4=int4)
    d = pkg.open_model_directory(out)
    meta = d.load_metadata()
    assert meta.io.num_layers == 2 and meta.vocab_size == 300
    cfg2, w2, _ = lower_decoder(pb.load_model(d.model_path))
    assert (cfg2.num_layers, cfg2.hidden, cfg2.num_heads, cfg2.num_kv_heads, cfg2.head_dim, cfg2.intermediate, cfg2.vocab) == \
        (2, 64, 4, 2, 16, 96, 300)
    assert cfg2.qkv_bias and (cfg2.weight_format == ("int4" if int4 else "bf16"))
    tol = 0.05 if int4 else 1e-6
    for a, b in zip(w.layers, w2.layers):
        assert float((a.qkv_w - b.qkv_w).abs().max()) <= tol
        assert float((a.gate_up_w - b.gate_up_w).abs().max()) <= tol
        assert torch.allclose(a.qkv_b, b.qkv_b, atol=1e-6)
    if not int4:
        assert cfg2.tie_embeddings


def test_lowering_rejects_non_decoder(tmp_path):
    g = pb.Graph()
    g.nodes.append(pb.Node("Relu", ["x"], ["y"]))
    with pytest.raises(GraphPatternError, match="not a recognised decoder"):
        lower_decoder(pb.Model(graph=g))


def test_metadata_closed_schema_and_capabilities():
    ok = md.parse(yaml.safe_load(open("/dev/stdin").read()) if False else {
        "model": {"max_sequence_length": 16, "io": {"token_input": "input_ids", "logits_output": "logits",
                                                    "kv_inputs": ["a.k", "a.v"], "kv_outputs": ["b.k", "b.v"]}}})
    assert ok.io.num_layers == 1 and ok.max_sequence_length == 16
    with pytest.raises(md.MetadataError, match="unknown field"):
        md.parse({"modle": {}})
    with pytest.raises(md.MetadataError, match="unknown capability"):
        md.parse({"required_capabilities": ["warp_drive"]})
    with pytest.raises(md.MetadataError, match="not implemented"):
        md.parse({"required_capabilities": ["workflow_ssa"]})
    with pytest.raises(md.MetadataError, match="positional pairs"):
        md.parse({"model": {"io": {"kv_inputs": ["k", "v"], "kv_outputs": ["k"]}}})
    sc = md.parse({"model": {"io": {"static_cache": {"write_indices_input": "wi", "kv_sequence_length_input": "n",
                                                     "key_cache_inputs": ["k0"], "value_cache_inputs": ["v0"],
                                                     "key_cache_outputs": ["uk0"], "value_cache_outputs": ["uv0"]}}}})
    assert sc.io.static_cache.write_indices_input == "wi" and sc.io.num_layers == 1


def test_reads_reference_fixture_metadata():
    for name in ("tiny-llm", "tiny-llm-scatter"):
        p = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")), "tests", "fixtures", name,
                         "inference_metadata.yaml")
        if os.path.exists(p):
            m = md.load(p)
            assert m.max_sequence_length == 16 and m.io is not None


def test_genai_config_import():
    doc = import_genai_config({"model": {"context_length": 4096, "vocab_size": 100, "eos_token_id": 2,
                                         "decoder": {"num_hidden_layers": 2, "inputs": {"input_ids": "input_ids", "attention_mask": "attention_mask"},
                                                     "outputs": {"logits": "logits"}}},
                               "search": {"temperature": 0.7, "top_p": 0.9, "do_sample": True}})
    m = md.parse(doc)
    assert m.io.kv_inputs[2] == "past_key_values.1.key" and m.generation_defaults["top_p"] == 0.9


def test_model_package_with_shared_assets(tmp_path):
    w = random_weights(CFG, "cpu", seed=1, dtype=torch.float32)
    flat = export_package(CFG, w, str(tmp_path / "flat"))
    root = str(tmp_path / "package")
    os.makedirs(root)
    variant = str(tmp_path / "variant")
    os.makedirs(variant)
    for f in ("decoder.onnx", "decoder.onnx.data", "inference_metadata.yaml"):
        os.replace(os.path.join(flat, f), os.path.join(variant, f))
    pkg.write_package(root, {"b200": {"ep": "cuda", "device": "gpu", "directory": variant},
                             "cpu": {"ep": "cpu", "device": "cpu", "directory": variant}},
                      shared_files={"tokenizer": os.path.join(flat, "tokenizer.json"),
                                    "chat_template": os.path.join(flat, "chat_template.jinja")})
    d = pkg.open_model_directory(root)
    assert d.variant == "b200" and d.tokenizer_path and "sha256-" in d.tokenizer_path and "im_start" in d.chat_template
    assert pkg.open_model_directory(root, ep="cpu", device="cpu").variant == "cpu"
    with pytest.raises(pkg.PackageError, match="escapes the package root"):
        pkg.resolve_ref(root, "../../etc/passwd")


def test_upstream_metadata_samples_parse_or_fail_with_reasons():
    import os

    import pytest

    from onnx_genai_b200 import metadata as md

    root = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")), "tests", "fixtures")
    if not os.path.exists(os.path.join(root, "sample_metadata.yaml")):
        pytest.skip("the upstream metadata samples are not available on this machine")
    y, j = md.load(os.path.join(root, "sample_metadata.yaml")), md.load(os.path.join(root, "sample_metadata.json"))
    assert y.max_sequence_length == j.max_sequence_length == 131072 and y.required_capabilities == j.required_capabilities
    assert {"grouped_query_attention", "kv_cache"} <= set(y.required_capabilities)
    with pytest.raises(md.MetadataError, match="required_capabilities: expected a list"):
        md.load(os.path.join(root, "invalid_metadata.yaml"))
    with pytest.raises(md.MetadataError, match="cannot parse"):
        md.load(os.path.join(root, "malformed_metadata.yaml"))


def test_every_upstream_fixture_metadata_document_parses():
    import glob
    import os

    import pytest

    from onnx_genai_b200 import metadata as md

    root = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")), "tests", "fixtures")
    docs = sorted(glob.glob(os.path.join(root, "**", "inference_metadata.yaml"), recursive=True))
    if not docs:
        pytest.skip("the upstream fixtures are not available on this machine")
    assert len(docs) >= 20
    for path in docs:
        md.load(path)          # unknown fields, capabilities or shapes would raise MetadataError naming the file


def test_context_cache_round_trips_dense_and_int4_lowerings(tmp_path):
    """The cached lowering gives the same configuration, the same tensors and the same tokens; touching the model file
    or changing the options makes it stale."""
    import dataclasses

    from onnx_genai_b200.bench.config_bench import _export
    from onnx_genai_b200.engine.api import Engine, GenerateOptions
    from onnx_genai_b200.package import context_cache as cc

    for fmt in ("fp32", "int4"):
        d = str(tmp_path / fmt)
        _export("tiny-llama", d, fmt, layers=2)
        first = Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64, context_cache=True)
        assert first.context_cache_hit is False and os.path.exists(os.path.join(d, "ogb_context", "weights.bin"))
        second = Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64, context_cache=True)
        assert second.context_cache_hit is True
        assert dataclasses.asdict(first.llm.cfg.model) == dataclasses.asdict(second.llm.cfg.model)
        opt = GenerateOptions(max_new_tokens=6, greedy=True)
        assert first.generate("hello", opt).token_ids == second.generate("hello", opt).token_ids
        plain = Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64)
        assert plain.context_cache_hit is None and plain.generate("hello", opt).token_ids == second.generate("hello", opt).token_ids
        # stale: another option, then a touched source file
        model_path = os.path.join(d, "decoder.onnx")
        key = cc.fingerprint(model_path, torch.float32, True)
        assert cc.load(os.path.join(d, "ogb_context"), key + "x", "cpu") is None
        os.utime(model_path, ns=(1, 1))
        assert cc.fingerprint(model_path, torch.float32, True) != key
        third = Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64, context_cache=True)
        assert third.context_cache_hit is False
    # a truncated blob is a miss, not a crash
    blob = os.path.join(d, "ogb_context", "weights.bin")
    with open(blob, "r+b") as f:
        f.truncate(100)
    assert Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64, context_cache=True).context_cache_hit is False
