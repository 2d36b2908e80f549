"""Grammar constraints: Lark-style grammars and JSON Schema on the incremental Earley recogniser."""
import json

import numpy as np
import pytest

from onnx_genai_b200.engine import constraints as cons
from onnx_genai_b200.engine.grammar import GrammarConstraint, parse_lark, schema_to_grammar

CALC = r"""
// arithmetic with the usual precedence
?start: sum
?sum: product (("+" | "-") product)*
?product: atom (("*" | "/") atom)*
atom: SIGNED_NUMBER | NAME | "(" sum ")" | NAME "(" [sum ("," sum)*] ")"
NAME: /[a-z_][a-z0-9_]*/i
%import common.SIGNED_NUMBER
%import common.WS
%ignore WS
"""


def test_lark_grammar_membership():
    c = GrammarConstraint(parse_lark(CALC))
    for text in ("1", "1 + 2*3", "f(1, g(x) - 2) / Y", "( ( 1 ) )", "-3.5e2 * k", "f()"):
        assert c.matches(text), text
    for text in ("", "1 +", "f(,)", "(1", "1 2", "1 ** 2", "3x"):
        assert not c.matches(text), text


def test_lark_operators_ranges_and_flags():
    g = parse_lark(r'''
start: GREETING " " id ("," id)~0..2 "!"?
GREETING: "hello"i | "hi"i
id: LETTER ("0".."9")~3
%import common.LETTER
''')
    c = GrammarConstraint(g)
    assert c.matches("HeLLo a123") and c.matches("hi a123,b456,c789!") and c.matches("hello z000!")
    assert not c.matches("hello a12") and not c.matches("hi a123,b456,c789,d000") and not c.matches("hey a123")
    with pytest.raises(ValueError, match="'undefined_rule', which is not defined"):
        parse_lark("start: undefined_rule")
    with pytest.raises(ValueError, match="only `%import common.NAME`"):
        parse_lark("%import other.X\nstart: X")
    with pytest.raises(ValueError, match="look-around"):
        parse_lark("start: /(?=a)b/")


def test_token_masks_follow_the_grammar_incrementally():
    vocab = ["", "1", "2", "+", "-", "(", ")", " ", "1+", "+(", ")+", "12", "x", "1)", ".5", "))", "f(", ", "]
    c = GrammarConstraint(parse_lark(CALC))
    ok = lambda: {v for v, a in zip(vocab, c.allowed(vocab)) if a}
    first = ok()
    assert {"1", "2", "(", " ", "-", "1+", "12", "x", ".5", "f("} <= first and not ({")", ")+", "1)", "))", ", "} & first)      # "+" may start a signed number
    c.advance("f(")
    assert ")" in ok() and ", " not in ok()                 # an empty argument list may close, a comma needs an argument first
    c.advance("1")
    assert {", ", ")", "+", ")+", "12"} <= ok() and "f(" not in ok() and not c.complete
    c.advance(")+")
    assert not c.complete and "(" in ok() and ")" not in ok()
    c.advance("x")
    assert c.complete
    with pytest.raises(ValueError, match="cannot continue"):
        c.advance(")")
    # every allowed token keeps the text a prefix of a sentence; every refused one does not (checked by brute force)
    c2 = GrammarConstraint(parse_lark(CALC))
    c2.advance("(1 ")
    mask = c2.allowed(vocab)
    for tok, a in zip(vocab, mask):
        if tok:
            assert a == (c2.state.feed_text(tok) is not None), tok


SCHEMA = {
    "$defs": {"node": {"type": "object", "properties": {"value": {"type": ["integer", "null"]},
                                                       "children": {"type": "array", "items": {"$ref": "#/$defs/node"}, "maxItems": 2}},
                       "required": ["value"], "additionalProperties": False}},
    "type": "object",
    "properties": {
        "id": {"type": "string", "format": "uuid"},
        "kind": {"enum": ["leaf", "tree", 3]},
        "root": {"$ref": "#/$defs/node"},
        "when": {"type": "string", "format": "date"},
        "pair": {"type": "array", "prefixItems": [{"type": "string"}, {"type": "number"}], "items": False, "minItems": 2},
        "note": {"anyOf": [{"type": "string", "maxLength": 3}, {"type": "boolean"}]},
        "code": {"type": "string", "pattern": "^[A-Z]{2}-[0-9]+$"},
    },
    "required": ["id", "kind"],
    "additionalProperties": {"type": "integer"},
}


def test_json_schema_with_refs_optionals_and_additional_properties():
    c = GrammarConstraint(schema_to_grammar(SCHEMA))
    uid = "123e4567-e89b-12d3-a456-426614174000"
    good = [
        {"id": uid, "kind": "leaf"},
        {"id": uid, "kind": 3, "root": {"value": 1, "children": [{"value": None}, {"value": 2, "children": []}]}},
        {"id": uid, "kind": "tree", "when": "2024-02-29", "pair": ["a", 1.5], "note": "abc", "code": "AB-12", "extra": 7, "more": -1},
        {"id": uid, "kind": "tree", "note": False},
    ]
    for doc in good:
        assert c.matches(json.dumps(doc)), doc
        assert c.matches(json.dumps(doc, indent=1)), doc
    bad = [
        {"kind": "leaf"},                                            # required id missing
        {"id": "not-a-uuid", "kind": "leaf"},
        {"id": uid, "kind": "bush"},
        {"id": uid, "kind": "leaf", "root": {"children": []}},       # nested required
        {"id": uid, "kind": "leaf", "root": {"value": 1, "children": [{"value": 1}, {"value": 2}, {"value": 3}]}},   # maxItems
        {"id": uid, "kind": "leaf", "root": {"value": 1, "other": 2}},                                                # additionalProperties false
        {"id": uid, "kind": "leaf", "when": "2024-13-01"},
        {"id": uid, "kind": "leaf", "pair": ["a"]},
        {"id": uid, "kind": "leaf", "pair": ["a", 1, 2]},
        {"id": uid, "kind": "leaf", "note": "abcd"},
        {"id": uid, "kind": "leaf", "code": "ab-1"},
        {"id": uid, "kind": "leaf", "extra": "text"},                # additional properties must be integers
    ]
    for doc in bad:
        assert not c.matches(json.dumps(doc)), doc
    with pytest.raises(ValueError, match="patternProperties"):
        schema_to_grammar({"type": "object", "patternProperties": {}})
    with pytest.raises(ValueError, match="points nowhere"):
        schema_to_grammar({"$ref": "#/$defs/missing"})


def test_constraint_processor_drives_a_grammar_to_completion():
    """A greedy walk over random logits under the processor always ends in a sentence of the grammar."""
    vocab = ["", "<eos>"] + list('{}[]":, 0123456789abcxyz-.') + ['{"', '":', '", "', "true", "false", "null", '"}', "},", "[]", "12", " {"]
    schema = {"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "array", "items": {"type": "boolean"}, "maxItems": 3},
                                                "c": {"type": "string", "maxLength": 4}}, "required": ["a", "c"], "additionalProperties": False}
    rng = np.random.default_rng(0)
    for trial in range(8):
        proc = cons.ConstraintProcessor(cons.make_constraint(("json_schema", schema)), vocab, eos_ids=[1])
        out = []
        for _ in range(200):
            logits = proc.process(out, rng.normal(size=len(vocab)).astype(np.float32))
            tok = int(np.argmax(logits))
            if tok == 1:
                break
            out.append(tok)
            proc.observe(tok)
        text = "".join(vocab[t] for t in out)
        doc = json.loads(text)
        assert set(doc) <= {"a", "b", "c"} and isinstance(doc["a"], int) and len(doc["c"]) <= 4 and len(doc.get("b", [])) <= 3, text
    lark = cons.make_constraint(("lark", 'start: "yes" | "no" | "maybe"'))
    assert [v for v, a in zip(["y", "ye", "n", "m", "x", "yes!"], lark.allowed(["y", "ye", "n", "m", "x", "yes!"])) if a] == ["y", "ye", "n", "m"]
