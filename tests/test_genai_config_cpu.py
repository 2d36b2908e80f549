"""Legacy ``genai_config.json`` compatibility: structural classification, refusals, attention, KV naming, graph-derived ports."""
import pytest

from onnx_genai_b200 import metadata as md
from onnx_genai_b200.package import genai_config as gc


def _cfg(**decoder):
    dec = {"num_hidden_layers": 2, "num_attention_heads": 8, "num_key_value_heads": 2, "head_size": 16, "hidden_size": 128,
           "inputs": {"input_ids": "input_ids", "attention_mask": "attention_mask"}, "outputs": {"logits": "logits"}}
    dec.update(decoder)
    return {"model": {"type": "whatever", "context_length": 512, "vocab_size": 100, "eos_token_id": [2, 7], "decoder": dec},
            "search": {"max_length": 256, "temperature": 0.5, "num_return_sequences": 1, "length_penalty": 1.0, "no_repeat_ngram_size": 0,
                       "diversity_penalty": 0.0, "early_stopping": True, "past_present_share_buffer": True}}


def test_single_decoder_import_carries_attention_search_and_aliasing():
    doc = gc.import_genai_config(_cfg())
    att = doc["model"]["attention"]
    assert att == {"type": "group_query_attention", "num_kv_heads": 2, "num_attention_heads": 8, "head_dim": 16,
                   "key_sequence_lengths": {"scalar_broadcast": "unit_batch"}}
    assert doc["model"]["max_sequence_length"] == 512                      # context_length wins over search.max_length
    io = doc["model"]["io"]
    assert io["kv_inputs"] == ["past_key_values.0.key", "past_key_values.0.value", "past_key_values.1.key", "past_key_values.1.value"]
    assert io["kv_outputs"][3] == "present.1.value" and io["aliasing"] == "permitted"
    d = doc["generation"]["defaults"]
    assert d["early_stopping"] is True and d["length_penalty"] == 1.0 and "past_present_share_buffer" not in d
    m = md.parse(doc)
    assert m.io.aliasing == "permitted" and m.max_sequence_length == 512
    assert gc.eos_token_ids(_cfg()) == [2, 7]
    assert gc.check_compatibility(_cfg()) == []


def test_multi_head_when_kv_heads_are_absent_or_exceed_query_heads():
    c = _cfg()
    del c["model"]["decoder"]["num_key_value_heads"]
    assert gc.import_genai_config(c)["model"]["attention"]["type"] == "multi_head_attention"
    c = _cfg(num_key_value_heads=16)
    assert gc.import_genai_config(c)["model"]["attention"]["type"] == "multi_head_attention"
    assert any("num_key_value_heads=16" in p for p in gc.check_compatibility(c))
    with pytest.raises(gc.GenAiConfigError, match="num_key_value_heads=16"):
        gc.import_genai_config(c, strict=True)
    assert any("not a multiple" in p for p in gc.check_compatibility(_cfg(num_key_value_heads=3)))


def test_combined_and_custom_kv_patterns():
    c = _cfg(inputs={"input_ids": "ids", "past_names": "past_%d"}, outputs={"logits": "lg", "present_names": "present_%d"})
    io = gc.import_genai_config(c)["model"]["io"]
    assert io["kv_inputs"] == ["past_0", "past_1"] and io["kv_outputs"] == ["present_0", "present_1"]
    assert io["token_input"] == "ids" and io["logits_output"] == "lg"
    c = _cfg(inputs={"past_key_names": "k.%d", "past_value_names": "v.%d", "inputs_embeds": "embeds"})
    io = gc.import_genai_config(c)["model"]["io"]
    assert io["kv_inputs"][:2] == ["k.0", "v.0"] and io["inputs_embeds_input"] == "embeds" and "token_input" not in io
    with pytest.raises(gc.GenAiConfigError, match="no %d"):
        gc.import_genai_config(_cfg(inputs={"past_key_names": "key"}))
    with pytest.raises(gc.GenAiConfigError, match="combined"):
        gc.import_genai_config(_cfg(inputs={"past_names": "p%d"}))


@pytest.mark.parametrize("extra,shape", [
    ({"encoder": {"filename": "enc.onnx"}}, "encoder_decoder"),
    ({"vision": {"filename": "v.onnx"}}, "multimodal"),
    ({"embedding": {"filename": "e.onnx"}}, "multimodal"),
    ({"joiner": {"filename": "j.onnx"}, "encoder": {"filename": "enc.onnx"}}, "transducer"),
])
def test_composite_packages_are_classified_and_declined(extra, shape):
    c = _cfg()
    c["model"].update(extra)
    assert gc.model_shape(c) == shape
    with pytest.raises(gc.GenAiConfigError, match="transducer|pipeline.workflow"):
        gc.import_genai_config(c)
    assert gc.check_compatibility(c)


def test_lstm_prediction_network_is_a_transducer_even_with_an_encoder_block():
    c = _cfg(inputs={"input_ids": "targets", "lstm_hidden_state": "h", "lstm_cell_state": "c"})
    c["model"]["encoder"] = {"filename": "enc.onnx"}
    assert gc.is_transducer(c) and gc.model_shape(c) == "transducer"
    c = _cfg(inputs={"lstm_hidden_state": "h", "past_key_names": "k.%d"})          # has KV: not a prediction network
    assert not gc.is_transducer(c)
    c = _cfg(pipeline=[{"stage0": {"filename": "a.onnx"}}])
    assert gc.model_shape(c) == "decoder_pipeline"


def test_missing_blocks_name_the_field():
    with pytest.raises(gc.GenAiConfigError, match="`model` object"):
        gc.import_genai_config({})
    with pytest.raises(gc.GenAiConfigError, match="model.decoder"):
        gc.import_genai_config({"model": {}})
    assert any("num_hidden_layers" in p for p in gc.check_compatibility(_cfg(num_hidden_layers=0)))
    c = _cfg()
    c["search"]["max_length"] = 4096
    assert any("exceeds model.context_length" in p for p in gc.check_compatibility(c))


def _port(shape, dtype="float16"):
    return {"dtype": dtype, "shape": shape}


def test_graph_derived_ports_for_a_hybrid_decoder():
    kv = ["batch", 2, "past", 16]
    graph = {"inputs": {"input_ids": _port(["batch", "seq"], "int64"),
                        "past_key_values.1.key": _port(kv), "past_key_values.1.value": _port(kv),
                        "past_key_values.3.key": _port(kv), "past_key_values.3.value": _port(kv),
                        "past_conv_state.0": _port([1, 64, 4]), "past_recurrent_state.0": _port([1, 8, 16, 16]),
                        "past_orphan.0": _port([1, 4])},
             "outputs": {"logits": _port(["batch", "seq", 100]),
                         "present.1.key": _port(kv), "present.1.value": _port(kv), "present.3.key": _port(kv), "present.3.value": _port(kv),
                         "present_conv_state.0": _port([None, None, None]), "present_recurrent_state.0": _port([1, 8, 16, 16])}}
    got = gc.derive_decoder_io_from_graph(graph)
    assert got["kv_inputs"] == ["past_key_values.1.key", "past_key_values.1.value", "past_key_values.3.key", "past_key_values.3.value"]
    assert got["kv_outputs"] == ["present.1.key", "present.1.value", "present.3.key", "present.3.value"] and got["kv_dtype"] == "float16"
    assert got["state_pairs"] == [{"input": "past_conv_state.0", "output": "present_conv_state.0"},
                                  {"input": "past_recurrent_state.0", "output": "present_recurrent_state.0"}]
    exact = gc.derive_decoder_io_from_graph(graph, allow_symbolic=False)            # the fully symbolic output no longer pairs
    assert exact["state_pairs"] == [{"input": "past_recurrent_state.0", "output": "present_recurrent_state.0"}]
    doc = gc.import_genai_config(_cfg(num_hidden_layers=4), graph=graph)
    assert doc["model"]["io"]["kv_inputs"] == got["kv_inputs"] and len(doc["model"]["io"]["state_pairs"]) == 2
    m = md.parse(doc)
    assert len(m.io.kv_inputs) == 4


def test_graph_derivation_refuses_to_guess():
    kv = ["b", 2, "p", 16]
    g = {"inputs": {"past_key_values.0.key": _port(kv), "past_key_values.0.value": _port(kv, "float32")},
         "outputs": {"present.0.key": _port(kv), "present.0.value": _port(kv)}}
    assert gc.derive_decoder_io_from_graph(g) is None                                 # dtype conflict
    g = {"inputs": {"past_key_values.0.key": _port(kv)}, "outputs": {"present.0.key": _port(kv), "present.0.value": _port(kv)}}
    assert gc.derive_decoder_io_from_graph(g) is None                                 # half a layer
    assert gc.derive_decoder_io_from_graph({"inputs": {"input_ids": _port(["b", "s"], "int64")}, "outputs": {"logits": _port([1])}}) is None
    uniform = {"inputs": {f"past_key_values.{i}.{w}": _port(kv) for i in range(2) for w in ("key", "value")},
               "outputs": {f"present.{i}.{w}": _port(kv) for i in range(2) for w in ("key", "value")}}
    assert gc.import_genai_config(_cfg(), graph=uniform)["model"]["io"]["kv_inputs"] == gc.import_genai_config(_cfg())["model"]["io"]["kv_inputs"]


def test_a_directory_with_only_genai_config_loads_and_generates(tmp_path):
    import json
    import os

    from onnx_genai_b200 import package as pkg
    from onnx_genai_b200.bench.config_bench import _export
    from onnx_genai_b200.engine.api import Engine, GenerateOptions

    d = str(tmp_path)
    _export("tiny-llama", d, "fp32", layers=2)
    native = pkg.open_model_directory(d).load_metadata()
    os.remove(os.path.join(d, "inference_metadata.yaml"))
    json.dump({"model": {"context_length": 128, "eos_token_id": 2, "decoder": {"num_hidden_layers": 2, "num_attention_heads": 4,
                                                                             "num_key_value_heads": 2, "head_size": 16}},
               "search": {"max_length": 64}}, open(os.path.join(d, "genai_config.json"), "w"))
    m = pkg.open_model_directory(d).load_metadata()
    assert m.io.kv_inputs == native.io.kv_inputs and m.io.kv_outputs == native.io.kv_outputs and m.max_sequence_length == 128
    e = Engine.from_dir(d, device="cpu", max_seqs=2, max_seq_len=64)
    assert len(e.generate("hi", GenerateOptions(max_new_tokens=4, greedy=True)).token_ids) >= 1
