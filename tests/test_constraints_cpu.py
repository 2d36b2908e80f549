"""Constrained decoding: the JSON recogniser, the schema compiler, and generation through the engine and server."""
import json

import pytest
import regex

from onnx_genai_b200.bench.config_bench import _export
from onnx_genai_b200.engine import constraints as cons
from onnx_genai_b200.engine.api import Engine, GenerateOptions

VALID = ['{}', '[]', '{"a": 1}', '[1, 2.5e-3, -0, true, false, null, "x\\n\\u00e9"]', ' {"k": {"n": [ ]}} ', '"s"', '-12.5E+7', '0']
INVALID = ['{', '{"a" 1}', '[1,]', '{"a":1,}', '01', '-', '"\n"', '"\\x"', 'tru', '[1 2]', '{"a":1}}', '1.', '.5', "{'a':1}"]


@pytest.mark.parametrize("doc", VALID)
def test_json_prefix_accepts_valid_documents(doc):
    st = cons.JsonPrefix()
    for i, ch in enumerate(doc):
        assert st.feed(ch), (doc, i)
    assert st.complete, doc
    json.loads(doc)


@pytest.mark.parametrize("doc", INVALID)
def test_json_prefix_rejects_or_leaves_incomplete(doc):
    st = cons.JsonPrefix()
    ok = st.feed_text(doc)
    assert not (ok and st.complete), doc
    with pytest.raises(json.JSONDecodeError):
        json.loads(doc)


def test_schema_compiles_to_a_regex_for_the_documented_subset():
    schema = {"type": "object", "properties": {
        "name": {"type": "string", "maxLength": 8}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 2},
        "ok": {"type": "boolean"}, "score": {"anyOf": [{"type": "number"}, {"type": "null"}]}}}
    rx = regex.compile(cons.schema_to_regex(schema))
    good = {"name": "bob", "age": 41, "tags": ["a", "b"], "ok": True, "score": None}
    assert rx.fullmatch(json.dumps(good)) and rx.fullmatch(json.dumps(good, indent=1)) and rx.fullmatch(json.dumps(good, separators=(",", ":")))
    assert rx.fullmatch(json.dumps({**good, "score": 1.5e3, "tags": []}))
    for bad in ({**good, "age": 1.5}, {**good, "tags": ["c"]}, {**good, "tags": ["a", "a", "a"]}, {**good, "name": "x" * 9}, {"name": "bob"}):
        assert not rx.fullmatch(json.dumps(bad)), bad
    with pytest.raises(ValueError, match="patternProperties"):
        cons.schema_to_regex({"type": "object", "patternProperties": {}})
    with pytest.raises(ValueError, match="Lark grammar, line 1"):
        cons.make_constraint(("lark", "start: 'a'"))          # Lark strings use double quotes


@pytest.fixture(scope="module")
def engine(tmp_path_factory):
    d = tmp_path_factory.mktemp("cons_model")
    _export("tiny-llama", str(d), "fp32", layers=1)
    return Engine.from_dir(str(d), device="cpu", max_seqs=4, max_seq_len=256)


@pytest.mark.parametrize("greedy,seed", [(True, 0), (False, 3), (False, 11)])
def test_generation_under_json_constraint_is_parseable(engine, greedy, seed):
    opt = GenerateOptions(max_new_tokens=200, greedy=greedy, temperature=1.0, seed=seed, constraint=("json_object",))
    res = engine.generate("data:", opt)
    if res.finish_reason == "stop":
        assert isinstance(json.loads(res.text), dict), res.text
    else:                                   # ran out of budget: what exists is still a valid prefix
        assert cons.JsonPrefix().feed_text(res.text), res.text


def test_regex_choice_and_schema_constraints_through_the_engine(engine):
    res = engine.generate("call", GenerateOptions(max_new_tokens=40, greedy=False, seed=5, constraint=("regex", r"[0-9]{3}-[0-9]{4}")))
    assert regex.fullmatch(r"[0-9]{3}-[0-9]{4}", res.text) and res.finish_reason == "stop", res.text
    res = engine.generate("pick", GenerateOptions(max_new_tokens=40, greedy=True, constraint=("choice", ["alpha", "beta", "alphabet"])))
    assert res.text in ("alpha", "beta", "alphabet") and res.finish_reason == "stop"
    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "ok": {"type": "boolean"}}}
    res = engine.generate("obj", GenerateOptions(max_new_tokens=120, greedy=False, seed=2, constraint=("json_schema", schema)))
    if res.finish_reason == "stop":
        doc = json.loads(res.text)
        assert isinstance(doc, dict) and isinstance(doc.get("n", 0), int) and isinstance(doc.get("ok", True), bool)    # neither is required
    batch = engine.generate_batch(["a", "b"], GenerateOptions(max_new_tokens=30, greedy=False, seed=9, constraint=("regex", r"(yes|no)!")))
    assert all(r.text in ("yes!", "no!") for r in batch)


def test_server_response_format_uses_the_constraint(engine):
    from fastapi.testclient import TestClient

    from onnx_genai_b200.server.app import create_app

    with TestClient(create_app(engine, model_name="tiny")) as client:
        body = {"model": "tiny", "messages": [{"role": "user", "content": "give json"}], "max_tokens": 160, "temperature": 0.8, "seed": 4,
                "response_format": {"type": "json_schema", "json_schema": {"name": "t", "schema": {
                    "type": "object", "properties": {"city": {"type": "string", "maxLength": 6}, "pop": {"type": "integer"}},
                    "required": ["city", "pop"], "additionalProperties": False}}}}
        r = client.post("/v1/chat/completions", json=body)
        assert r.status_code == 200, r.text
        choice = r.json()["choices"][0]
        if choice["finish_reason"] == "stop":
            doc = json.loads(choice["message"]["content"])
            assert set(doc) == {"city", "pop"}
        r = client.post("/v1/completions", json={"model": "tiny", "prompt": "x", "max_tokens": 20, "guided_choice": ["red", "green"]})
        assert r.status_code == 200 and r.json()["choices"][0]["text"] in ("red", "green")
        bad = client.post("/v1/chat/completions", json={**body, "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "object", "patternProperties": {}}}}})
        assert bad.status_code == 400 and "patternProperties" in bad.text
