"""One-way import of an onnxruntime-genai ``genai_config.json`` into inference metadata.

Counterpart of the reference's ``onnx-genai-genai-config`` crate (src/import.rs and src/compatibility.rs:94-780):
the legacy file is only ever read; the result is an inference-metadata document (schema v1) with the decode ABI
spelled out as positional kv pairs.  What the compatibility layer does:

* classifies the package by structure, never by ``model.type`` or a model name: single decoder, decoder pipeline,
  multimodal (embedding / vision / speech front ends), encoder-decoder, RNN-T transducer (a joint network, or an
  LSTM prediction network that exposes no attention KV).  Only a single decoder is converted; the composite shapes
  need native metadata with a ``pipeline.workflow`` and are declined with an error that says so;
* describes attention (grouped-query when KV heads are declared and do not exceed the query heads, else multi-head),
  carries ``search`` into ``generation.defaults`` field for field, and ``past_present_share_buffer: true`` into
  ``model.io.aliasing: permitted`` (alias legality is a fact of the graph ABI, not a generation default);
* expands the ``%d`` KV name patterns over the layers -- key / value interleaved per layer, or one combined
  ``past_names`` / ``present_names`` entry per layer -- or, when the decoder graph's port inventory is supplied,
  derives the ports from the graph instead: hybrid decoders expose dense KV only for some layers plus fixed
  recurrent-state pairs (``conv_state`` / ``recurrent_state``), and only the ports the graph really has are declared.
  A uniform dense decoder yields the same lists either way.
"""
from __future__ import annotations

import re

DEFAULT_INPUT_IDS = "input_ids"
DEFAULT_LOGITS = "logits"
DEFAULT_PAST_KEY, DEFAULT_PAST_VALUE = "past_key_values.%d.key", "past_key_values.%d.value"
DEFAULT_PRESENT_KEY, DEFAULT_PRESENT_VALUE = "present.%d.key", "present.%d.value"

_SEARCH_FIELDS = ("do_sample", "temperature", "top_k", "top_p", "repetition_penalty", "num_beams", "num_return_sequences",
                  "min_length", "max_length", "length_penalty", "no_repeat_ngram_size", "diversity_penalty", "early_stopping")


class GenAiConfigError(ValueError):
    pass


def _decoder(cfg: dict) -> dict:
    model = cfg.get("model")
    if not isinstance(model, dict):
        raise GenAiConfigError("genai_config.json: the `model` object is missing")
    dec = model.get("decoder")
    if not isinstance(dec, dict):
        raise GenAiConfigError("genai_config.json: `model.decoder` is missing; only decoder packages can be imported")
    return dec


def is_transducer(cfg: dict) -> bool:
    """An RNN-T package: a joint network, and / or a decoder that is an LSTM prediction network (LSTM hidden / cell state
    inputs and no self- or cross-attention KV ports)."""
    model = cfg.get("model") or {}
    if model.get("joiner") is not None:
        return True
    ins = (model.get("decoder") or {}).get("inputs") or {}
    lstm = ins.get("lstm_hidden_state") is not None or ins.get("lstm_cell_state") is not None
    kv = any(ins.get(k) is not None for k in ("past_key_names", "past_value_names", "past_names", "cross_past_key_names",
                                               "cross_past_value_names"))
    return lstm and not kv


def model_shape(cfg: dict) -> str:
    """single_decoder | decoder_pipeline | multimodal | encoder_decoder | transducer.  The transducer check comes first:
    such a package also declares ``model.encoder``, and treating it as encoder-decoder would invent cross-attention
    bindings its graphs do not have."""
    model = cfg.get("model") or {}
    if is_transducer(cfg):
        return "transducer"
    if model.get("encoder") is not None:
        return "encoder_decoder"
    if any(model.get(k) is not None for k in ("embedding", "vision", "speech")):
        return "multimodal"
    if (model.get("decoder") or {}).get("pipeline"):
        return "decoder_pipeline"
    return "single_decoder"


def uses_group_query_attention_op(cfg: dict) -> bool:
    dec = _decoder(cfg)
    kv, attn = dec.get("num_key_value_heads"), dec.get("num_attention_heads")
    return kv is not None and attn is not None and 1 <= int(kv) <= int(attn)


def max_sequence_length(cfg: dict):
    v = (cfg.get("model") or {}).get("context_length")
    return v if v is not None else (cfg.get("search") or {}).get("max_length")


def _expand(combined, key_pat, value_pat, default_key, default_value, layers: int):
    if layers <= 0:
        return None
    for pat in (combined, key_pat, value_pat):
        if pat is not None and "%d" not in pat:
            raise GenAiConfigError(f"genai_config.json: the KV name pattern {pat!r} has no %d for the layer index")
    if combined is not None:
        return [combined % i for i in range(layers)]
    kp, vp = key_pat or default_key, value_pat or default_value
    out = []
    for i in range(layers):
        out += [kp % i, vp % i]
    return out


def _pattern_regex(pat: str):
    return re.compile("^" + re.escape(pat).replace("%d", r"(\d+)") + "$")


def _shapes_pair(a, b, allow_symbolic: bool) -> bool:
    """Do an input and an output port carry the same state?  Exact: every axis equal, symbolic ones included.  With
    ``allow_symbolic`` an unknown axis (None or a name) matches anything: stock exports often leave a ``present.*``
    recurrent-state shape fully symbolic although the paired ``past_*`` input is concrete."""
    if a is None or b is None:
        return allow_symbolic
    if len(a) != len(b):
        return False
    if not allow_symbolic:
        return list(a) == list(b)
    return all(x == y or not isinstance(x, int) or not isinstance(y, int) for x, y in zip(a, b))


def derive_decoder_io_from_graph(graph: dict, past_key=DEFAULT_PAST_KEY, past_value=DEFAULT_PAST_VALUE,
                                 present_key=DEFAULT_PRESENT_KEY, present_value=DEFAULT_PRESENT_VALUE, allow_symbolic=True):
    """KV / state topology from a graph's port inventory alone.

    ``graph`` = ``{"inputs": {name: {"dtype": str, "shape": [...]}}, "outputs": {...}}``.  Dense KV ports are those that
    match the four ``%d`` patterns, taken for the layers the graph really has (sparse for hybrid decoders) and paired
    positionally.  Every other ``past_*`` / ``present_*``-style pair whose names differ only by that prefix and whose
    shapes agree is a loop-carried state pair.  Returns ``None`` when the graph has no KV ports at all, or when the KV
    tensors disagree on dtype (no geometry is ever guessed)."""
    ins, outs = graph.get("inputs") or {}, graph.get("outputs") or {}
    rx = {k: _pattern_regex(p) for k, p in (("pk", past_key), ("pv", past_value), ("ok", present_key), ("ov", present_value))}
    layers_in: dict = {}
    for name in ins:
        for kind in ("pk", "pv"):
            m = rx[kind].match(name)
            if m:
                layers_in.setdefault(int(m.group(1)), {})[kind] = name
    layers_out: dict = {}
    for name in outs:
        for kind in ("ok", "ov"):
            m = rx[kind].match(name)
            if m:
                layers_out.setdefault(int(m.group(1)), {})[kind] = name
    kv_inputs, kv_outputs, dtypes = [], [], set()
    for layer in sorted(layers_in):
        i, o = layers_in[layer], layers_out.get(layer, {})
        if set(i) != {"pk", "pv"} or set(o) != {"ok", "ov"}:
            return None                       # a layer with half its ports: not a contract this importer may invent
        kv_inputs += [i["pk"], i["pv"]]
        kv_outputs += [o["ok"], o["ov"]]
        dtypes.update(str(ins[n].get("dtype")) for n in (i["pk"], i["pv"]))
    if set(layers_out) - set(layers_in):
        return None
    if len(dtypes) > 1:
        return None
    used_in, used_out = set(kv_inputs), set(kv_outputs)
    state_pairs = []
    for name, spec in ins.items():
        if name in used_in:
            continue
        for a, b in (("past_", "present_"), ("past.", "present."), ("past_key_values.", "present.")):
            if name.startswith(a):
                twin = b + name[len(a):]
                if twin in outs and twin not in used_out and _shapes_pair(spec.get("shape"), outs[twin].get("shape"), allow_symbolic):
                    state_pairs.append({"input": name, "output": twin})
                    used_out.add(twin)
                    break
    if not kv_inputs and not state_pairs:
        return None
    return {"kv_inputs": kv_inputs, "kv_outputs": kv_outputs, "state_pairs": state_pairs,
            "kv_dtype": next(iter(dtypes)) if dtypes else None}


def graph_ports(model) -> dict:
    """Port inventory of a parsed ONNX model (``onnx_pb.Model``) in the form :func:`derive_decoder_io_from_graph` takes.
    Initializers listed among the inputs (old exporters do that) are not ports."""
    g = model.graph

    def ports(values):
        return {v.name: {"dtype": str(v.elem_type), "shape": [d if isinstance(d, int) and d >= 0 else (d or None) for d in v.shape]}
                for v in values if v.name not in g.initializers}

    return {"inputs": ports(g.inputs), "outputs": ports(g.outputs)}


def decoder_io(cfg: dict, graph: dict | None = None) -> dict:
    dec = _decoder(cfg)
    ins, outs = dec.get("inputs") or {}, dec.get("outputs") or {}
    layers = int(dec.get("num_hidden_layers") or 0)
    io: dict = {}
    if ins.get("input_ids") is not None:
        io["token_input"] = ins["input_ids"]
    if ins.get("inputs_embeds") is not None:
        io["inputs_embeds_input"] = ins["inputs_embeds"]
    elif ins.get("input_ids") is None:
        io["token_input"] = DEFAULT_INPUT_IDS
    if ins.get("attention_mask") is not None:
        io["attention_mask_input"] = ins["attention_mask"]
    if ins.get("position_ids") is not None:
        io["position_ids_input"] = ins["position_ids"]
    io["logits_output"] = outs.get("logits") or DEFAULT_LOGITS
    derived = None
    if graph is not None:
        derived = derive_decoder_io_from_graph(graph, ins.get("past_key_names") or DEFAULT_PAST_KEY,
                                               ins.get("past_value_names") or DEFAULT_PAST_VALUE,
                                               outs.get("present_key_names") or DEFAULT_PRESENT_KEY,
                                               outs.get("present_value_names") or DEFAULT_PRESENT_VALUE)
    if derived is not None and derived["kv_inputs"]:
        io["kv_inputs"], io["kv_outputs"] = derived["kv_inputs"], derived["kv_outputs"]
        if derived["state_pairs"]:
            io["state_pairs"] = derived["state_pairs"]
    else:
        kv_in = _expand(ins.get("past_names"), ins.get("past_key_names"), ins.get("past_value_names"), DEFAULT_PAST_KEY,
                        DEFAULT_PAST_VALUE, layers)
        kv_out = _expand(outs.get("present_names"), outs.get("present_key_names"), outs.get("present_value_names"),
                         DEFAULT_PRESENT_KEY, DEFAULT_PRESENT_VALUE, layers)
        if kv_in is not None:
            io["kv_inputs"] = kv_in
        if kv_out is not None:
            io["kv_outputs"] = kv_out
        if kv_in is not None and kv_out is not None and len(kv_in) != len(kv_out):
            raise GenAiConfigError(f"genai_config.json: {len(kv_in)} KV inputs but {len(kv_out)} KV outputs; a combined `past_names` "
                                   "pattern needs a combined `present_names` pattern")
    if (cfg.get("search") or {}).get("past_present_share_buffer") is True:
        io["aliasing"] = "permitted"
    return io


def check_compatibility(cfg: dict) -> list:
    """Problems that would make the imported package misbehave, as strings (an empty list means none found)."""
    problems = []
    try:
        dec = _decoder(cfg)
    except GenAiConfigError as exc:
        return [str(exc)]
    shape = model_shape(cfg)
    if shape != "single_decoder":
        problems.append(f"the package is a {shape.replace('_', ' ')}: composite packages need native inference metadata with "
                        "pipeline.workflow; legacy pipeline synthesis is not provided")
    heads, kv = dec.get("num_attention_heads"), dec.get("num_key_value_heads")
    if heads is not None and kv is not None:
        if int(kv) < 1 or int(kv) > int(heads):
            problems.append(f"num_key_value_heads={kv} must lie in [1, num_attention_heads={heads}]")
        elif int(heads) % int(kv):
            problems.append(f"num_attention_heads={heads} is not a multiple of num_key_value_heads={kv}")
    hidden, hs = dec.get("hidden_size"), dec.get("head_size")
    if hidden is not None and heads is not None and hs is not None and int(hidden) != int(heads) * int(hs):
        problems.append(f"hidden_size={hidden} differs from num_attention_heads x head_size = {int(heads) * int(hs)} "
                        "(allowed, but the attention projections are then not square)")
    if int(dec.get("num_hidden_layers") or 0) <= 0:
        problems.append("model.decoder.num_hidden_layers is missing or zero: the KV name patterns cannot be expanded")
    ctx, mx = (cfg.get("model") or {}).get("context_length"), (cfg.get("search") or {}).get("max_length")
    if ctx is not None and mx is not None and int(mx) > int(ctx):
        problems.append(f"search.max_length={mx} exceeds model.context_length={ctx}")
    search = cfg.get("search") or {}
    if int(search.get("num_beams") or 1) > 1:
        problems.append(f"search.num_beams={search['num_beams']}: beam search is carried into the defaults but this engine samples one "
                        "sequence per request")
    return problems


def import_genai_config(cfg: dict, graph: dict | None = None, strict: bool = False) -> dict:
    """``genai_config.json`` (parsed) -> inference-metadata document.  ``graph``: the decoder graph's port inventory, when
    the caller has it (see :func:`derive_decoder_io_from_graph`).  ``strict``: raise on any compatibility problem, not
    only on the ones that make conversion impossible."""
    shape = model_shape(cfg)
    if shape == "transducer":
        raise GenAiConfigError("genai_config.json describes an RNN-T transducer (joint network / LSTM prediction network); "
                               "that pipeline family is not executed by this runtime")
    if shape != "single_decoder":
        raise GenAiConfigError(f"genai_config.json describes a {shape.replace('_', ' ')} package: composite packages require native "
                               "inference_metadata with pipeline.workflow; legacy genai_config pipeline synthesis is not provided")
    if strict:
        problems = [p for p in check_compatibility(cfg) if "allowed" not in p]
        if problems:
            raise GenAiConfigError("genai_config.json: " + "; ".join(problems))
    dec = _decoder(cfg)
    model = cfg.get("model") or {}
    attention = {"type": "group_query_attention" if uses_group_query_attention_op(cfg) else "multi_head_attention"}
    for src, dst in (("num_key_value_heads", "num_kv_heads"), ("num_attention_heads", "num_attention_heads"), ("head_size", "head_dim")):
        if dec.get(src) is not None:
            attention[dst] = int(dec[src])
    if attention["type"] == "group_query_attention":
        attention["key_sequence_lengths"] = {"scalar_broadcast": "unit_batch"}
    doc_model: dict = {"attention": attention}
    msl = max_sequence_length(cfg)
    if msl is not None:
        doc_model["max_sequence_length"] = int(msl)
    if model.get("vocab_size") is not None:
        doc_model["vocab_size"] = int(model["vocab_size"])
    io = decoder_io(cfg, graph)
    if io:
        doc_model["io"] = io
    doc = {"schema_version": "v1", "required_capabilities": ["kv_cache"], "model": doc_model}
    search = cfg.get("search") or {}
    defaults = {k: search[k] for k in _SEARCH_FIELDS if search.get(k) is not None}
    if defaults:
        doc["generation"] = {"defaults": defaults}
    return doc


def eos_token_ids(cfg: dict) -> list:
    eos = (cfg.get("model") or {}).get("eos_token_id")
    if eos is None:
        return []
    return [int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)]
