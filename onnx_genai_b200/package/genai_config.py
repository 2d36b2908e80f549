"""One-way import of an onnxruntime-genai ``genai_config.json`` into inference metadata.

Counterpart of the reference's `onnx-genai-genai-config` crate (src/import.rs, compatibility.rs):
the legacy file is only ever read; the result is an inference-metadata document (schema v1)
with the decode ABI spelled out as positional kv pairs.
"""
from __future__ import annotations


def import_genai_config(cfg: dict) -> dict:
    model = cfg.get("model") or {}
    dec = model.get("decoder") or {}
    n_layers = int(dec.get("num_hidden_layers", 0))
    ins, outs = dec.get("inputs") or {}, dec.get("outputs") or {}
    pk = ins.get("past_key_names", "past_key_values.%d.key")
    pv = ins.get("past_value_names", "past_key_values.%d.value")
    ok = outs.get("present_key_names", "present.%d.key")
    ov = outs.get("present_value_names", "present.%d.value")
    kv_in, kv_out = [], []
    for i in range(n_layers):
        kv_in += [pk % i, pv % i]
        kv_out += [ok % i, ov % i]
    io = {"token_input": ins.get("input_ids", "input_ids"), "logits_output": outs.get("logits", "logits"),
          "kv_inputs": kv_in, "kv_outputs": kv_out}
    if "attention_mask" in ins:
        io["attention_mask_input"] = ins["attention_mask"]
    if "position_ids" in ins:
        io["position_ids_input"] = ins["position_ids"]
    doc = {"schema_version": "v1", "required_capabilities": ["kv_cache"],
           "model": {"io": io}}
    if "context_length" in model:
        doc["model"]["max_sequence_length"] = int(model["context_length"])
    if "vocab_size" in model:
        doc["model"]["vocab_size"] = int(model["vocab_size"])
    search = cfg.get("search") or {}
    defaults = {}
    for src, dst in (("do_sample", "do_sample"), ("temperature", "temperature"), ("top_k", "top_k"), ("top_p", "top_p"),
                     ("repetition_penalty", "repetition_penalty"), ("max_length", "max_length"),
                     ("min_length", "min_length"), ("num_beams", "num_beams")):
        if src in search:
            defaults[dst] = search[src]
    if defaults:
        doc["generation"] = {"defaults": defaults}
    return doc


def eos_token_ids(cfg: dict) -> list:
    eos = (cfg.get("model") or {}).get("eos_token_id")
    if eos is None:
        return []
    return list(eos) if isinstance(eos, (list, tuple)) else [int(eos)]
