"""Constrained decoding: JSON, JSON-Schema (a documented subset), regular expressions and fixed choices.

A constraint answers one question per step -- which next tokens keep the output a valid prefix -- and the
:class:`ConstraintProcessor` turns the answer into a logit mask (disallowed tokens become ``-inf``; the
end-of-sequence token is allowed only once the output is complete).  This is the contract of the reference's
``Constraint`` trait (crates/onnx-genai-engine/src/logits.rs:67-81) and its ``GenerateConstraint`` options
(src/config.rs:1483-1492).  The reference validates every vocabulary token's text at the character level and
delegates JSON-Schema/regex/Lark grammars to llguidance; that library is not available offline, so here

* ``json``         is a hand-written incremental JSON recogniser (a pushdown automaton over characters);
* ``regex``        uses the ``regex`` package's partial matching;
* ``json_schema``  compiles the schema to a context-free grammar (engine/grammar.py: nested and recursive schemas,
                   required / optional properties, additionalProperties, prefixItems, $ref, formats) run by an
                   incremental Earley recogniser; :func:`schema_to_regex` remains for callers that want a pattern;
* ``choice``       accepts prefixes of the listed strings;
* ``lark``         parses the grammar text (the commonly used part of Lark's syntax) into the same recogniser.

A schema keyword the compiler does not know raises ``ValueError`` naming it.
"""
from __future__ import annotations

import json
import re as _re

import numpy as np

from .processors import LogitProcessor

_WS = " \t\n\r"
_DIGITS = "0123456789"
_HEX = "0123456789abcdefABCDEF"


class JsonPrefix:
    """Incremental recogniser for one JSON value.  ``feed`` returns False at the first character that cannot
    continue a valid document; the object is then dead.  ``key()`` identifies the state for memoisation."""

    __slots__ = ("stack", "mode", "aux", "done")

    def __init__(self):
        self.stack = ()      # 'o' / 'a' for every open container
        self.mode = "value"  # value | str | esc | hex | num | lit | after | objfirst | key | colon | arrfirst
        self.aux = None      # str/esc/hex: (is_key, hex digits left); num: sub-state; lit: remaining characters
        self.done = False    # a complete top-level value has been seen

    def clone(self):
        c = JsonPrefix.__new__(JsonPrefix)
        c.stack, c.mode, c.aux, c.done = self.stack, self.mode, self.aux, self.done
        return c

    def key(self):
        return (self.stack, self.mode, self.aux, self.done)

    @property
    def complete(self) -> bool:
        if self.done and self.mode == "after":
            return True
        return self.mode == "num" and not self.stack and self.aux in ("zero", "int", "frac", "exp")

    # -- transitions ---------------------------------------------------------------------------
    def _end_value(self):
        if not self.stack:
            self.done = True
        self.mode = "after"

    def _start_value(self, ch) -> bool:
        if ch == "{":
            self.stack += ("o",)
            self.mode = "objfirst"
        elif ch == "[":
            self.stack += ("a",)
            self.mode = "arrfirst"
        elif ch == '"':
            self.mode, self.aux = "str", (False, 0)
        elif ch == "-":
            self.mode, self.aux = "num", "minus"
        elif ch == "0":
            self.mode, self.aux = "num", "zero"
        elif ch in "123456789":
            self.mode, self.aux = "num", "int"
        elif ch == "t":
            self.mode, self.aux = "lit", "rue"
        elif ch == "f":
            self.mode, self.aux = "lit", "alse"
        elif ch == "n":
            self.mode, self.aux = "lit", "ull"
        else:
            return False
        return True

    def _after(self, ch) -> bool:
        if ch in _WS:
            return True
        if not self.stack:
            return False
        top = self.stack[-1]
        if ch == ",":
            self.mode = "key" if top == "o" else "value"
            return True
        if (ch == "}" and top == "o") or (ch == "]" and top == "a"):
            self.stack = self.stack[:-1]
            self._end_value()
            return True
        return False

    def feed(self, ch) -> bool:
        m = self.mode
        if m == "str":
            is_key = self.aux[0]
            if ch == '"':
                if is_key:
                    self.mode, self.aux = "colon", None
                else:
                    self.aux = None
                    self._end_value()
                return True
            if ch == "\\":
                self.mode = "esc"
                return True
            return ord(ch) >= 0x20
        if m == "esc":
            if ch in '"\\/bfnrt':
                self.mode = "str"
                return True
            if ch == "u":
                self.mode, self.aux = "hex", (self.aux[0], 4)
                return True
            return False
        if m == "hex":
            if ch not in _HEX:
                return False
            left = self.aux[1] - 1
            self.mode, self.aux = ("str", (self.aux[0], 0)) if left == 0 else ("hex", (self.aux[0], left))
            return True
        if m == "num":
            s = self.aux
            if s == "minus":
                if ch == "0":
                    self.aux = "zero"
                    return True
                if ch in "123456789":
                    self.aux = "int"
                    return True
                return False
            if s in ("zero", "int"):
                if ch in _DIGITS and s == "int":
                    return True
                if ch == ".":
                    self.aux = "dot"
                    return True
                if ch in "eE":
                    self.aux = "e"
                    return True
            elif s == "dot":
                if ch in _DIGITS:
                    self.aux = "frac"
                    return True
                return False
            elif s == "frac":
                if ch in _DIGITS:
                    return True
                if ch in "eE":
                    self.aux = "e"
                    return True
            elif s == "e":
                if ch in "+-":
                    self.aux = "esign"
                    return True
                if ch in _DIGITS:
                    self.aux = "exp"
                    return True
                return False
            elif s == "esign":
                if ch in _DIGITS:
                    self.aux = "exp"
                    return True
                return False
            elif s == "exp":
                if ch in _DIGITS:
                    return True
            if s in ("zero", "int", "frac", "exp"):   # the number ends here; the character belongs to what follows
                self.aux = None
                self._end_value()
                return self._after(ch)
            return False
        if m == "lit":
            if ch != self.aux[0]:
                return False
            self.aux = self.aux[1:]
            if not self.aux:
                self.aux = None
                self._end_value()
            return True
        if m == "after":
            return self._after(ch)
        if ch in _WS:
            return True
        if m == "value":
            return self._start_value(ch)
        if m == "arrfirst":
            if ch == "]":
                self.stack = self.stack[:-1]
                self._end_value()
                return True
            self.mode = "value"
            return self._start_value(ch)
        if m in ("objfirst", "key"):
            if ch == '"':
                self.mode, self.aux = "str", (True, 0)
                return True
            if ch == "}" and m == "objfirst":
                self.stack = self.stack[:-1]
                self._end_value()
                return True
            return False
        if m == "colon":
            if ch == ":":
                self.mode = "value"
                return True
            return False
        return False

    def feed_text(self, text) -> bool:
        for ch in text:
            if not self.feed(ch):
                return False
        return True


class Constraint:
    """``advance(token_text)`` consumes an accepted token; ``allowed(token_texts)`` returns a bool mask of the
    tokens that may come next; ``complete`` says whether the output may end here."""

    name = "constraint"

    def allowed(self, token_texts) -> np.ndarray:
        raise NotImplementedError

    def advance(self, text: str) -> None:
        raise NotImplementedError

    @property
    def complete(self) -> bool:
        raise NotImplementedError

    def terminal(self, token_texts) -> bool:
        """The output is complete and generation should stop now (nothing, or only padding, could follow)."""
        return self.complete and not self.allowed(token_texts).any()


class JsonConstraint(Constraint):
    """One complete, well-formed JSON value (``require_object``: the value must be an object)."""

    name = "json"

    def __init__(self, require_object: bool = False):
        self.state = JsonPrefix()
        self.require_object = require_object
        self.seen_any = False
        self._memo: dict = {}

    def allowed(self, token_texts):
        key = (self.state.key(), self.seen_any)
        hit = self._memo.get(key)
        if hit is not None:
            return hit
        mask = np.zeros(len(token_texts), dtype=bool)
        for i, t in enumerate(token_texts):
            if not t:
                continue
            if self.require_object and not self.seen_any:
                stripped = t.lstrip(_WS)
                if stripped and stripped[0] != "{":
                    continue
            s = self.state.clone()
            mask[i] = s.feed_text(t)
        if len(self._memo) < 512:
            self._memo[key] = mask
        return mask

    def advance(self, text):
        if text.strip(_WS):
            self.seen_any = True
        self.state.feed_text(text)

    @property
    def complete(self):
        return self.state.complete

    def terminal(self, token_texts):
        return self.state.done and self.state.mode == "after"   # a closed value: only whitespace could follow


class RegexConstraint(Constraint):
    """The whole output must match ``pattern`` (anchored at both ends)."""

    name = "regex"

    def __init__(self, pattern: str):
        try:
            import regex
        except ImportError as exc:   # pragma: no cover - the package is part of the environment
            raise RuntimeError("regex constraints need the 'regex' package (partial matching)") from exc
        try:
            self.rx = regex.compile(pattern, regex.DOTALL)
        except regex.error as exc:
            raise ValueError(f"invalid regular expression {pattern!r}: {exc}") from exc
        self.text = ""

    def allowed(self, token_texts):
        mask = np.zeros(len(token_texts), dtype=bool)
        base = self.text
        fm = self.rx.fullmatch
        for i, t in enumerate(token_texts):
            if t:
                mask[i] = fm(base + t, partial=True) is not None
        return mask

    def advance(self, text):
        self.text += text

    @property
    def complete(self):
        return self.rx.fullmatch(self.text) is not None


class ChoiceConstraint(Constraint):
    name = "choice"

    def __init__(self, options):
        self.options = [str(o) for o in options]
        if not self.options:
            raise ValueError("a choice constraint needs at least one option")
        self.text = ""

    def allowed(self, token_texts):
        mask = np.zeros(len(token_texts), dtype=bool)
        live = [o[len(self.text):] for o in self.options if o.startswith(self.text)]
        for i, t in enumerate(token_texts):
            if t:
                mask[i] = any(rest.startswith(t) for rest in live)
        return mask

    def advance(self, text):
        self.text += text

    @property
    def complete(self):
        return self.text in self.options


# ---------------------------------------------------------------------------------------------
# JSON Schema -> regular expression (subset)
# ---------------------------------------------------------------------------------------------
_STR_CHAR = r'(?:[^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
_INT = r"-?(?:0|[1-9][0-9]*)"
_NUM = _INT + r"(?:\.[0-9]+)?(?:[eE][+-]?[0-9]+)?"
_WSX = r"[ \n\t]*"
_SUPPORTED = {"type", "enum", "const", "items", "minItems", "maxItems", "properties", "required", "additionalProperties",
              "anyOf", "oneOf", "pattern", "minLength", "maxLength", "title", "description", "$schema", "default", "examples"}


def _lit(value) -> str:
    return _re.escape(json.dumps(value, ensure_ascii=False))


def schema_to_regex(schema) -> str:
    """Regular expression accepting exactly the JSON texts of the supported schema subset (compact or with
    spaces/newlines between tokens)."""
    if schema is True or schema == {}:
        raise ValueError("an unconstrained schema ({} or true) cannot be compiled; use the 'json' constraint instead")
    if not isinstance(schema, dict):
        raise ValueError(f"schema must be an object, got {type(schema).__name__}")
    unknown = set(schema) - _SUPPORTED
    if unknown:
        raise ValueError(f"JSON-Schema keyword(s) {sorted(unknown)} are not supported by the built-in grammar compiler; "
                         f"supported: {sorted(_SUPPORTED)}")
    if "const" in schema:
        return _lit(schema["const"])
    if "enum" in schema:
        return "(?:" + "|".join(_lit(v) for v in schema["enum"]) + ")"
    for comb in ("anyOf", "oneOf"):
        if comb in schema:
            return "(?:" + "|".join(schema_to_regex(s) for s in schema[comb]) + ")"
    t = schema.get("type")
    if isinstance(t, list):
        return "(?:" + "|".join(schema_to_regex({**schema, "type": one}) for one in t) + ")"
    if t == "string":
        if "pattern" in schema:
            inner = schema["pattern"]
            inner = inner[1:] if inner.startswith("^") else inner
            inner = inner[:-1] if inner.endswith("$") and not inner.endswith("\\$") else inner
            return '"(?:' + inner + ')"'
        lo, hi = schema.get("minLength", 0), schema.get("maxLength")
        quant = "*" if (lo == 0 and hi is None) else "{%d,%s}" % (lo, "" if hi is None else hi)
        return '"' + _STR_CHAR + quant + '"'
    if t == "integer":
        return _INT
    if t == "number":
        return _NUM
    if t == "boolean":
        return "(?:true|false)"
    if t == "null":
        return "null"
    if t == "array":
        if "items" not in schema:
            raise ValueError("array schemas need 'items' in the built-in grammar compiler")
        item = schema_to_regex(schema["items"])
        lo, hi = schema.get("minItems", 0), schema.get("maxItems")
        sep = _WSX + "," + _WSX
        if hi is not None and hi == 0:
            return r"\[" + _WSX + r"\]"
        more = "{%d,%s}" % (max(lo - 1, 0), "" if hi is None else hi - 1)
        body = item + "(?:" + sep + item + ")" + more
        if lo == 0:
            body = "(?:" + body + ")?"
        return r"\[" + _WSX + body + _WSX + r"\]"
    if t == "object":
        props = schema.get("properties") or {}
        if not props:
            return r"\{" + _WSX + r"\}"
        parts = [_lit(name) + _WSX + ":" + _WSX + schema_to_regex(sub) for name, sub in props.items()]
        return r"\{" + _WSX + (_WSX + "," + _WSX).join(parts) + _WSX + r"\}"
    raise ValueError(f"schema type {t!r} is not supported; give one of string, integer, number, boolean, null, array, object")


def make_constraint(spec) -> Constraint | None:
    """``spec``: a Constraint, None, or a tuple/list ``(kind, argument)`` with kind in json, json_object,
    json_schema, regex, choice, lark."""
    if spec is None or isinstance(spec, Constraint):
        return spec
    if isinstance(spec, str):
        spec = (spec,)
    kind = spec[0]
    arg = spec[1] if len(spec) > 1 else None
    if kind == "json":
        return JsonConstraint()
    if kind == "json_object":
        return JsonConstraint(require_object=True)
    if kind == "json_schema":
        from .grammar import GrammarConstraint, schema_to_grammar

        schema = json.loads(arg) if isinstance(arg, str) else arg
        return _GrammarAdapter(GrammarConstraint(schema_to_grammar(schema), "json_schema"))
    if kind == "regex":
        return RegexConstraint(arg)
    if kind == "choice":
        return ChoiceConstraint(arg)
    if kind == "lark":
        from .grammar import GrammarConstraint, parse_lark

        return _GrammarAdapter(GrammarConstraint(parse_lark(arg), "lark"))
    raise ValueError(f"unknown constraint kind {kind!r}; use json, json_object, json_schema, regex, choice or lark")


class _GrammarAdapter(Constraint):
    """A grammar recogniser (engine/grammar.py) behind the :class:`Constraint` interface."""

    def __init__(self, inner):
        self.inner = inner
        self.name = inner.name

    def allowed(self, token_texts):
        return self.inner.allowed(token_texts)

    def advance(self, text):
        self.inner.advance(text)

    @property
    def complete(self):
        return self.inner.complete

    def terminal(self, token_texts):
        return self.inner.terminal(token_texts)


class ConstraintProcessor(LogitProcessor):
    """Masks logits so only tokens the constraint allows survive; end-of-sequence only when complete.

    ``token_texts[i]`` is the decoded text of token ``i`` ('' for tokens that decode to nothing or to an
    incomplete byte sequence: those are never allowed).  ``observe(token)`` must be called with every
    accepted token (the engine's host sampling path does).  If nothing is allowed (the constraint is
    complete, or the vocabulary cannot continue it) only end-of-sequence tokens survive.
    """

    preserves_argmax = False

    def __init__(self, constraint: Constraint, token_texts, eos_ids=()):
        self.constraint = constraint
        self.token_texts = token_texts
        self.eos_ids = [int(e) for e in eos_ids if e is not None and 0 <= int(e) < len(token_texts)]
        self.dead_ends = 0

    def process(self, token_ids, logits):
        mask = self.constraint.allowed(self.token_texts).copy()
        for e in self.eos_ids:
            mask[e] = self.constraint.complete
        if not mask.any():
            self.dead_ends += 1
            if self.eos_ids:
                for e in self.eos_ids:
                    mask[e] = True
            else:
                return logits
        out = np.where(mask[: logits.shape[0]], logits, -np.inf).astype(logits.dtype, copy=False)
        return out

    def observe(self, token: int) -> None:
        if token in self.eos_ids:
            return
        self.constraint.advance(self.token_texts[token])


# ---------------------------------------------------------------------------------------------
# table-driven grammar guidance for workflow documents (the ``onnx-genai.grammar-guidance`` adapter)
# ---------------------------------------------------------------------------------------------
def grammar_guidance_adapter(action: str = "lookahead"):
    """A workflow component that advances per-row grammar states through a transition table.

    Ports: ``state`` [B], ``tokens`` [B, P], ``valid_length`` [B], ``transition_table`` [states, vocab] (next state, or a
    negative entry where the token is not allowed) -> ``next_state`` [B], ``consumed_length`` [B] (tokens the grammar
    accepted, in order, before the first one it rejects), ``logits_mask`` [B, vocab] (tokens allowed in ``next_state``),
    ``forced_tokens`` [B, 1] / ``forced_length`` [B] (the token, when the state allows exactly one).
    ``clone`` consumes nothing (it only reports the state's mask), ``lookahead`` stops at the first rejected token,
    ``commit`` treats a rejected token as an error -- the verifier must never commit what the grammar refused.
    Same behaviour as the reference's adapter (crates/onnx-genai-engine/src/pipeline/workflow.rs:2383-2516)."""
    if action not in ("clone", "lookahead", "commit"):
        raise ValueError(f"grammar guidance action {action!r} is not clone, lookahead or commit")

    def component(ports: dict) -> dict:
        import torch

        table = torch.as_tensor(np.asarray(ports["transition_table"])).long()
        states = torch.as_tensor(np.asarray(ports["state"])).long().reshape(-1)
        tokens = torch.as_tensor(np.asarray(ports["tokens"])).long()
        tokens = tokens.reshape(states.numel(), -1)
        lengths = torch.as_tensor(np.asarray(ports["valid_length"])).long().reshape(-1)
        n_states, vocab = table.shape
        next_state, consumed = [], []
        for row in range(states.numel()):
            s = int(states[row])
            if not 0 <= s < n_states:
                raise ValueError(f"grammar state {s} of row {row} is outside the table's {n_states} states")
            want = 0 if action == "clone" else int(lengths[row])
            if want < 0 or want > tokens.shape[1]:
                raise ValueError(f"valid_length {want} of row {row} does not fit the {tokens.shape[1]} proposed tokens")
            taken = 0
            for col in range(want):
                tok = int(tokens[row, col])
                nxt = int(table[s, tok]) if 0 <= tok < vocab else -1
                if nxt < 0:
                    if action == "commit":
                        raise ValueError(f"grammar commit: token {tok} at row {row}, position {col} is not allowed in state {s}")
                    break
                if nxt >= n_states:
                    raise ValueError(f"the transition table sends state {s} on token {tok} to state {nxt}, which does not exist")
                s, taken = nxt, taken + 1
            next_state.append(s)
            consumed.append(taken)
        ns = torch.tensor(next_state, dtype=torch.int64)
        mask = table[ns] >= 0
        single = mask.sum(dim=1) == 1
        forced = torch.where(single, mask.float().argmax(dim=1), torch.zeros_like(ns))
        return {"next_state": ns, "consumed_length": torch.tensor(consumed, dtype=torch.int64), "logits_mask": mask,
                "forced_tokens": forced.reshape(-1, 1), "forced_length": single.long()}

    return component
