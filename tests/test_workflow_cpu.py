"""Workflow form of the inference metadata: parsing, SSA validation and the decoder-ABI lowering."""
import copy
import os

import pytest
import yaml

from onnx_genai_b200.metadata import workflow as wfm

DOC = yaml.safe_load("""
manifest: {capabilities: [workflow_ssa, typed_emit]}
inputs:
  request.input_ids: {contract: {dtype: int64, rank: 2, shape: [batch, sequence]}, source: {kind: request}, required: true,
                      role: {kind: runtime, role: prompt_tokens}}
  request.max_new: {contract: {dtype: int64, rank: 1, shape: [1]}, source: {kind: request}, required: true}
  package.greedy: {contract: {dtype: bool, rank: 1, shape: [1]}, source: {kind: literal}, default: true}
outputs:
  tokens: {contract: {dtype: int64, rank: 2, shape: [batch, generated]}}
components:
  lm:
    implementation: {kind: onnx, artifact: decoder.onnx}
    ports:
      inputs:
        input_ids: {dtype: int64, rank: 2}
        attention_mask: {dtype: int64, rank: 2, optional: true}
        past.0.key: {dtype: float16, rank: 4}
        past.0.value: {dtype: float16, rank: 4}
        past.1.key: {dtype: float16, rank: 4}
        past.1.value: {dtype: float16, rank: 4}
      outputs:
        logits: {dtype: float32, rank: 3}
        present.0.key: {dtype: float16, rank: 4}
        present.0.value: {dtype: float16, rank: 4}
        present.1.key: {dtype: float16, rank: 4}
        present.1.value: {dtype: float16, rank: 4}
      roles: {input_ids: token_ids, attention_mask: attention_mask, logits: logits}
  pick: {implementation: {kind: onnx, artifact: pick.onnx}}
  pick_sampled: {implementation: {kind: onnx, artifact: pick_sampled.onnx}}
state:
  token: {contract: {dtype: int64, rank: 2}, initializer: setup.token, recurrence: {kind: invariant}}
serving:
  active: active
  state_service:
    groups:
      kv:
        kind: full_attention
        layout: bnsh
        sequence_axis: 2
        aliasing: permitted
        capabilities: {rollback_positions: 8}
        reuse: {prefix_reusable: true}
        ports:
          lm:
            v1: {input: past.1.value, output: present.1.value, role: value, layer: 1}
            k1: {input: past.1.key, output: present.1.key, role: key, layer: 1}
            v0: {input: past.0.value, output: present.0.value, role: value, layer: 0}
            k0: {input: past.0.key, output: present.0.key, role: key, layer: 0}
steps:
- kind: loop
  setup:
  - {kind: invoke, component: lm, inputs: {input_ids: request.input_ids}, outputs: {logits: setup.logits}}
  - {kind: invoke, component: pick, inputs: {logits: setup.logits}, outputs: {token: setup.token}}
  steps:
  - {kind: invoke, component: lm, inputs: {input_ids: token}, outputs: {logits: body.logits}}
  - kind: branch
    predicate: package.greedy
    cases:
      'true': {kind: invoke, component: pick, inputs: {logits: body.logits}, outputs: {token: body.greedy_token}}
    default: {kind: invoke, component: pick_sampled, inputs: {logits: body.logits}, outputs: {token: body.sampled_token}}
    outputs:
      body.token: {cases: {'true': body.greedy_token}, default: body.sampled_token}
  - {kind: emit, value: body.token, output: tokens, mode: append, when: active}
  continue_when: active
  max_iterations: request.max_new
  termination: generation_eos
  carried:
  - {cell: token, next: body.token}
""")


def test_parse_validate_and_lower_a_decoder_workflow():
    wf = wfm.parse(copy.deepcopy(DOC))
    assert wfm.validate(wf) == []
    loop = wf.steps[0]
    assert loop.kind == "loop" and [s.kind for s in loop.steps] == ["invoke", "branch", "emit"] and loop.termination == "generation_eos"
    abi = wfm.decoder_abi(wf)
    assert (abi.component, abi.token_input, abi.attention_mask_input, abi.logits_output) == ("lm", "input_ids", "attention_mask", "logits")
    # layer order comes from the declared layer index, key before value, not from the order of the labels
    assert abi.kv_pairs == [("past.0.key", "present.0.key"), ("past.0.value", "present.0.value"),
                            ("past.1.key", "present.1.key"), ("past.1.value", "present.1.value")]
    assert abi.num_layers == 2 and abi.kv_layout == "bnsh" and abi.kv_update == "append"
    assert abi.rollback_positions == 8 and abi.prefix_reusable


def _mutated(fn):
    doc = copy.deepcopy(DOC)
    fn(doc)
    return wfm.validate(wfm.parse(doc))


def test_validator_reports_each_kind_of_mistake():
    undefined = _mutated(lambda d: d["steps"][0]["steps"][0]["inputs"].update(input_ids="tokne"))
    assert any("'tokne'" in p and "not defined" in p for p in undefined)
    unknown_comp = _mutated(lambda d: d["steps"][0]["setup"][1].update(component="picker"))
    assert any("component 'picker'" in p and "declared: lm, pick, pick_sampled" in p for p in unknown_comp)
    bad_port = _mutated(lambda d: d["steps"][0]["setup"][0]["inputs"].update(input_idz="request.input_ids"))
    assert any("'input_idz' is not an input port" in p for p in bad_port)
    missing_port = _mutated(lambda d: d["steps"][0]["setup"][0]["inputs"].pop("input_ids"))
    assert any("required input port 'input_ids'" in p for p in missing_port)
    twice = _mutated(lambda d: d["steps"][0]["setup"][1]["outputs"].update(token="setup.logits"))
    assert any("second time" in p for p in twice)
    bad_emit = _mutated(lambda d: d["steps"][0]["steps"][2].update(output="text"))
    assert any("emit targets 'text'" in p for p in bad_emit)
    bad_carry = _mutated(lambda d: d["steps"][0]["carried"][0].update(next="body.nothing"))
    assert any("continues with 'body.nothing'" in p for p in bad_carry)
    bad_case = _mutated(lambda d: d["steps"][0]["steps"][1]["outputs"]["body.token"]["cases"].update({"false": "x"}))
    assert any("names case 'false'" in p for p in bad_case)
    bad_state = _mutated(lambda d: d["serving"]["state_service"]["groups"]["kv"]["ports"]["lm"]["k0"].update(input="past.9.key"))
    assert any("'past.9.key' is not an input port" in p for p in bad_state)


def test_malformed_steps_are_parse_errors():
    for mutate, needle in ((lambda d: d["steps"].append({"kind": "goto"}), "unknown step kind 'goto'"),
                           (lambda d: d["steps"][0].pop("continue_when"), "loop needs 'continue_when'"),
                           (lambda d: d["steps"][0]["steps"][2].update(mode="stream"), "emit mode 'stream'"),
                           (lambda d: d.update(steps=[]), "steps is empty")):
        doc = copy.deepcopy(DOC)
        mutate(doc)
        with pytest.raises(wfm.WorkflowError, match=needle):
            wfm.parse(doc)
    doc = copy.deepcopy(DOC)
    del doc["components"]["lm"]["ports"]["roles"]["logits"]
    with pytest.raises(wfm.WorkflowError, match="no component declares both"):
        wfm.decoder_abi(wfm.parse(doc))


FIXTURES = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")),
                        "tests", "fixtures", "onnx_genai_workflows")


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="reference fixtures are not on this machine")
def test_reference_workflow_fixtures_parse_and_validate():
    """The reference's own workflow documents (decoder, static cache, speculative, VLM, TTS, diffusion, video, ...) read
    as data: every one must parse and validate, and the two single-decoder ones must lower to their ABI."""
    seen = 0
    for name in sorted(os.listdir(FIXTURES)):
        path = os.path.join(FIXTURES, name, "inference_metadata.yaml")
        if not os.path.exists(path):
            continue
        wf = wfm.load_document(yaml.safe_load(open(path, encoding="utf-8")))
        assert wf is not None and wfm.validate(wf) == [], name
        seen += 1
        if name == "decoder":
            abi = wfm.decoder_abi(wf)
            assert (abi.component, abi.token_input, abi.kv_layout, abi.kv_update, len(abi.kv_pairs)) == ("model", "input_ids", "bnsh", "append", 1)
        if name == "static_cache":
            assert wfm.decoder_abi(wf).kv_update == "indexed_scatter"
    assert seen >= 10


def test_metadata_document_with_a_workflow_derives_its_model_io():
    from onnx_genai_b200 import metadata as md

    meta = md.parse({"schema_version": "1.0", "pipeline": {"workflow": copy.deepcopy(DOC)}})
    assert meta.io is not None and meta.io.token_input == "input_ids" and meta.io.logits_output == "logits"
    assert meta.io.kv_inputs == ["past.0.key", "past.0.value", "past.1.key", "past.1.value"] and meta.io.num_layers == 2
    assert meta.io.kv_layout == "head_major_bnsh" and meta.io.aliasing == "permitted"
    broken = copy.deepcopy(DOC)
    broken["steps"][0]["steps"][0]["inputs"]["input_ids"] = "nowhere"
    with pytest.raises(md.MetadataError, match="pipeline.workflow is not valid.*'nowhere'"):
        md.parse({"schema_version": "1.0", "pipeline": {"workflow": broken}})
