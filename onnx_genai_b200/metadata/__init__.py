"""Inference-metadata standard, schema v1: parse, validate, emit.

Format-compatible with the reference's `onnx-genai-metadata` crate
(crates/onnx-genai-metadata/src/schema/mod.rs:33-129): a closed top level
(``deny_unknown_fields``), a capability vocabulary whose unknown members make loading fail with a
precise error (src/lib.rs:10-90), the legacy ``model.io`` decode ABI
(schema/model_io.rs:84-265: token / mask / position inputs, logits output, positional
``kv_inputs`` / ``kv_outputs`` pairs, ``static_cache`` names, kv layout), MoE router facts
(schema/hardware.rs:31-98), tensor-parallel hints (hardware.rs:22-27, package.rs:295-345) and
generation defaults (schema/generation.rs).  Files may be YAML or JSON.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import yaml

SCHEMA_VERSION = "v1"

TOP_LEVEL_KEYS = {"schema_version", "required_capabilities", "model", "quantization", "pipeline", "adapters",
                  "hardware_requirements", "preprocessing", "package", "generation", "profiles", "speculative"}
MODEL_KEYS = {"attention", "max_sequence_length", "vocab_size", "runtime_configurable", "io", "mixture_of_experts",
              "sharding"}
IO_KEYS = {"sequence_source", "kv_ownership", "kv_layout", "token_input", "inputs_embeds_input", "attention_mask_input",
           "position_ids_input", "logits_output", "hidden_output", "kv_inputs", "kv_outputs", "aliasing",
           "cross_kv_inputs", "cross_kv_outputs", "state_pairs", "optional_inputs", "static_cache"}
STATIC_CACHE_KEYS = {"write_indices_input", "kv_sequence_length_input", "key_cache_inputs", "value_cache_inputs",
                     "key_cache_outputs", "value_cache_outputs"}

# capability identifiers built into this runtime (subset of the reference vocabulary that the
# fused executor can honour; anything else in required_capabilities is a load error)
SUPPORTED_CAPABILITIES = {
    "kv_cache", "grouped_query_attention", "multi_head_attention", "prefix_cache", "continuous_batching",
    "session_state_lease", "streaming_emit", "typed_emit", "emit_valid_length", "input_presence",
}
KNOWN_CAPABILITIES = SUPPORTED_CAPABILITIES | {
    "control_flow_loop", "image_preprocessing_program", "packed_image_outputs", "position_program",
    "multi_axis_positions", "loop_carried_state", "dual_sequence_inputs", "workflow_ssa", "linear_effects",
    "serving_service_contract", "parameter_adapters", "heterogeneous_adapter_batching", "bounded_state_recurrence",
    "advisory_state", "adaptive_proposal_budget", "grammar_guidance_adapter", "telemetry_adapter",
    "nested_control_flow", "loop_induction_values", "explicit_transfer",
}


class MetadataError(ValueError):
    """What is wrong, where, and how to fix it (every message names the offending key)."""


@dataclass
class StaticCacheIo:
    write_indices_input: str = ""
    kv_sequence_length_input: str = ""
    key_cache_inputs: list = field(default_factory=list)
    value_cache_inputs: list = field(default_factory=list)
    key_cache_outputs: list = field(default_factory=list)
    value_cache_outputs: list = field(default_factory=list)


@dataclass
class ModelIo:
    token_input: str = "input_ids"
    inputs_embeds_input: str | None = None
    attention_mask_input: str | None = None
    position_ids_input: str | None = None
    logits_output: str = "logits"
    hidden_output: str | None = None
    kv_inputs: list = field(default_factory=list)
    kv_outputs: list = field(default_factory=list)
    kv_layout: str = "head_major_bnsh"
    kv_ownership: str = "runtime"
    aliasing: str = "forbidden"
    static_cache: StaticCacheIo | None = None

    @property
    def num_layers(self) -> int:
        if self.static_cache is not None:
            return len(self.static_cache.key_cache_inputs)
        return len(self.kv_inputs) // 2


@dataclass
class MoERouter:
    score_function: str = "softmax"
    selection_method: str = "top_k"
    normalize_weights: bool = True
    scaling_factor: float = 1.0
    group_count: int | None = None
    groups_per_token: int | None = None


@dataclass
class MixtureOfExperts:
    representation: str = "expert_major"
    routed_expert_count: int = 0
    shared_expert_count: int = 0
    experts_per_token: int = 0
    expert_intermediate_size: int = 0
    activation: str = "swiglu"
    router: MoERouter = field(default_factory=MoERouter)


@dataclass
class InferenceMetadata:
    schema_version: str = SCHEMA_VERSION
    required_capabilities: list = field(default_factory=list)
    max_sequence_length: int | None = None
    vocab_size: int | None = None
    io: ModelIo | None = None
    chunked_prefill_size: int | None = None
    sliding_window: int | None = None      # model.attention.sliding_window: keys a query keeps seeing behind it
    sink_tokens: int = 0                   # model.attention.sink_tokens: leading keys kept under the window (attention sinks)
    mixture_of_experts: MixtureOfExperts | None = None
    supports_tensor_parallel: bool | None = None
    min_tp_degree: int | None = None
    tensor_parallel_max_shards: int | None = None
    generation_defaults: dict = field(default_factory=dict)
    speculative: dict = field(default_factory=dict)
    quantization: dict = field(default_factory=dict)
    workflow: object = None            # metadata.workflow.Workflow when the document carries pipeline.workflow
    raw: dict = field(default_factory=dict)


def _closed(d: dict, allowed: set, where: str):
    if not isinstance(d, dict):
        raise MetadataError(f"{where}: expected a mapping, found {type(d).__name__}")
    extra = sorted(set(d) - allowed)
    if extra:
        raise MetadataError(f"{where}: unknown field(s) {extra}; schema {SCHEMA_VERSION} allows {sorted(allowed)}. "
                            f"Remove the field or upgrade the runtime.")


def parse(doc: dict) -> InferenceMetadata:
    """Validate a decoded YAML/JSON document and return the typed view."""
    doc = doc or {}
    _closed(doc, TOP_LEVEL_KEYS, "inference_metadata")
    md = InferenceMetadata(raw=doc)
    md.schema_version = str(doc.get("schema_version", SCHEMA_VERSION))
    if md.schema_version not in (SCHEMA_VERSION, "1", "1.0"):
        raise MetadataError(f"schema_version: {md.schema_version!r} is not supported; this runtime reads {SCHEMA_VERSION!r}")
    caps = doc.get("required_capabilities") or []
    if not isinstance(caps, list):
        raise MetadataError("required_capabilities: expected a list of capability identifiers")
    for c in caps:
        if c not in KNOWN_CAPABILITIES:
            raise MetadataError(f"required_capabilities: unknown capability {c!r}; the package needs a newer runtime")
        if c not in SUPPORTED_CAPABILITIES:
            raise MetadataError(f"required_capabilities: capability {c!r} is known but not implemented by this runtime; "
                                f"the model cannot be served here")
    md.required_capabilities = list(caps)
    model = doc.get("model") or {}
    _closed(model, MODEL_KEYS, "model")
    md.max_sequence_length = model.get("max_sequence_length")
    att = model.get("attention")
    if isinstance(att, dict):
        win, sink = att.get("sliding_window"), att.get("sink_tokens")
        if win is not None:
            if not isinstance(win, int) or isinstance(win, bool) or win <= 0:
                raise MetadataError("model.attention.sliding_window must be an integer greater than zero")
            md.sliding_window = win
        if sink is not None:
            if not isinstance(sink, int) or isinstance(sink, bool) or sink < 0:
                raise MetadataError("model.attention.sink_tokens must be a non-negative integer")
            md.sink_tokens = sink if win is not None else 0     # only meaningful under a sliding window
    md.vocab_size = model.get("vocab_size")
    rc = model.get("runtime_configurable") or {}
    if isinstance(rc, dict) and isinstance(rc.get("chunked_prefill"), dict):
        md.chunked_prefill_size = rc["chunked_prefill"].get("chunk_size")
    io = model.get("io")
    if io is not None:
        _closed(io, IO_KEYS, "model.io")
        mio = ModelIo(token_input=io.get("token_input", "input_ids"), inputs_embeds_input=io.get("inputs_embeds_input"),
                      attention_mask_input=io.get("attention_mask_input"), position_ids_input=io.get("position_ids_input"),
                      logits_output=io.get("logits_output", "logits"), hidden_output=io.get("hidden_output"),
                      kv_inputs=list(io.get("kv_inputs") or []), kv_outputs=list(io.get("kv_outputs") or []),
                      kv_layout=io.get("kv_layout", "head_major_bnsh") if isinstance(io.get("kv_layout", ""), str) else "explicit",
                      kv_ownership=io.get("kv_ownership", "runtime"), aliasing=io.get("aliasing", "forbidden"))
        if len(mio.kv_inputs) != len(mio.kv_outputs):
            raise MetadataError(f"model.io: kv_inputs has {len(mio.kv_inputs)} names but kv_outputs has {len(mio.kv_outputs)}; "
                                f"they are positional pairs and must have equal length")
        if len(mio.kv_inputs) % 2:
            raise MetadataError("model.io.kv_inputs: expected key/value pairs (an even number of names)")
        if mio.aliasing not in ("forbidden", "permitted", "required"):
            raise MetadataError(f"model.io.aliasing: {mio.aliasing!r} is not one of forbidden | permitted | required")
        sc = io.get("static_cache")
        if sc is not None:
            _closed(sc, STATIC_CACHE_KEYS, "model.io.static_cache")
            mio.static_cache = StaticCacheIo(**{k: sc.get(k, [] if k.endswith("s") else "") for k in STATIC_CACHE_KEYS})
            n = len(mio.static_cache.key_cache_inputs)
            for k in ("value_cache_inputs", "key_cache_outputs", "value_cache_outputs"):
                if len(getattr(mio.static_cache, k)) != n:
                    raise MetadataError(f"model.io.static_cache.{k}: expected {n} names to match key_cache_inputs")
        md.io = mio
    moe = model.get("mixture_of_experts")
    if moe is not None:
        r = moe.get("router") or {}
        md.mixture_of_experts = MixtureOfExperts(
            representation=moe.get("representation", "expert_major"), routed_expert_count=int(moe.get("routed_expert_count", 0)),
            shared_expert_count=int(moe.get("shared_expert_count", 0)), experts_per_token=int(moe.get("experts_per_token", 0)),
            expert_intermediate_size=int(moe.get("expert_intermediate_size", 0)), activation=moe.get("activation", "swiglu"),
            router=MoERouter(score_function=r.get("score_function", "softmax"), selection_method=r.get("selection_method", "top_k"),
                             normalize_weights=bool(r.get("normalize_weights", True)), scaling_factor=float(r.get("scaling_factor", 1.0)),
                             group_count=r.get("group_count"), groups_per_token=r.get("groups_per_token")))
        if md.mixture_of_experts.router.score_function not in ("softmax", "sigmoid"):
            raise MetadataError(f"model.mixture_of_experts.router.score_function: "
                                f"{md.mixture_of_experts.router.score_function!r} is not softmax | sigmoid")
    sh = model.get("sharding") or {}
    if isinstance(sh.get("tensor_parallel"), dict):
        md.tensor_parallel_max_shards = sh["tensor_parallel"].get("max_shards")
    hw = doc.get("hardware_requirements") or {}
    md.supports_tensor_parallel = hw.get("supports_tensor_parallel")
    md.min_tp_degree = hw.get("min_tp_degree")
    gen = doc.get("generation") or {}
    md.generation_defaults = dict(gen.get("defaults") or {})
    md.speculative = dict(doc.get("speculative") or {})
    md.quantization = dict(doc.get("quantization") or {})
    # A package that carries the workflow form needs no model.io block: the decoder ABI is derived from it.
    wf_doc = (doc.get("pipeline") or {}).get("workflow") if isinstance(doc.get("pipeline"), dict) else None
    if wf_doc is not None:
        from . import workflow as _wf

        try:
            md.workflow = _wf.parse(wf_doc)
        except _wf.WorkflowError as exc:
            raise MetadataError(f"pipeline.workflow: {exc}") from exc
        problems = _wf.validate(md.workflow)
        if problems:
            raise MetadataError("pipeline.workflow is not valid: " + "; ".join(problems[:5]) +
                                (f" (and {len(problems) - 5} more)" if len(problems) > 5 else ""))
        if md.io is None:
            try:
                abi = _wf.decoder_abi(md.workflow)
            except _wf.WorkflowError:
                abi = None               # not a single-decoder workflow: nothing to derive for the decoder executor
            if abi is not None:
                layout = {"bnsh": "head_major_bnsh", "bsnh": "sequence_major_bsnh", "bsh": "sequence_major_bsh"}.get(abi.kv_layout or "", abi.kv_layout or "head_major_bnsh")
                md.io = ModelIo(token_input=abi.token_input, attention_mask_input=abi.attention_mask_input,
                                position_ids_input=abi.position_ids_input, logits_output=abi.logits_output,
                                kv_inputs=[a for a, _ in abi.kv_pairs], kv_outputs=[b for _, b in abi.kv_pairs], kv_layout=layout,
                                aliasing=abi.kv_aliasing or "forbidden")
    return md


def load(path: str) -> InferenceMetadata:
    with open(path, "r", encoding="utf-8") as f:
        text = f.read()
    try:
        doc = json.loads(text) if path.endswith(".json") else yaml.safe_load(text)
    except Exception as exc:
        raise MetadataError(f"{path}: cannot parse ({exc})") from exc
    try:
        return parse(doc)
    except MetadataError as exc:
        raise MetadataError(f"{path}: {exc}") from None


def find(model_dir: str) -> str | None:
    for name in ("inference_metadata.yaml", "inference_metadata.yml", "inference_metadata.json"):
        p = os.path.join(model_dir, name)
        if os.path.exists(p):
            return p
    return None


def emit(cfg, required_capabilities=("kv_cache", "grouped_query_attention"), generation_defaults=None,
         supports_tensor_parallel=True) -> dict:
    """Metadata document for a decoder exported by :mod:`onnx_genai_b200.package.decoder_graph`."""
    kv_in, kv_out = [], []
    for i in range(cfg.num_layers):
        kv_in += [f"past_key_values.{i}.key", f"past_key_values.{i}.value"]
        kv_out += [f"present.{i}.key", f"present.{i}.value"]
    doc = {
        "schema_version": SCHEMA_VERSION,
        "required_capabilities": list(required_capabilities),
        "model": {
            "max_sequence_length": int(cfg.max_position),
            "vocab_size": int(cfg.vocab),
            "runtime_configurable": {"chunked_prefill": {"chunk_size": 2048}},
            "io": {"token_input": "input_ids", "attention_mask_input": "attention_mask", "logits_output": "logits",
                   "kv_inputs": kv_in, "kv_outputs": kv_out, "kv_layout": "head_major_bnsh"},
        },
        "hardware_requirements": {"supports_tensor_parallel": bool(supports_tensor_parallel), "min_tp_degree": 1},
    }
    if cfg.sliding_window > 0:
        att = {"type": "group_query_attention", "sliding_window": int(cfg.sliding_window)}
        if cfg.attention_sinks > 0:
            att["sink_tokens"] = int(cfg.attention_sinks)
        doc["model"]["attention"] = att
    if cfg.moe.num_experts:
        doc["model"]["mixture_of_experts"] = {
            "representation": "expert_major", "routed_expert_count": cfg.moe.num_experts, "shared_expert_count": 0,
            "experts_per_token": cfg.moe.top_k, "expert_intermediate_size": cfg.moe.expert_intermediate,
            "shared_expert_intermediate_size": 0, "activation": "swiglu",
            "router": {"score_function": cfg.moe.score_function, "selection_method": "top_k",
                       "normalize_weights": bool(cfg.moe.renormalize), "scaling_factor": 1.0}}
    if generation_defaults:
        doc["generation"] = {"defaults": dict(generation_defaults)}
    return doc
