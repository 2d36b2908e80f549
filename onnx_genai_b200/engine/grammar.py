"""Context-free grammar constraints: Lark-style grammars and JSON Schema compiled to grammars.

The reference hands ``lark`` and ``json_schema`` constraints to llguidance (crates/onnx-genai-engine/src/
logits.rs:86,325-400).  That library is not part of this build, so the same two inputs are served by a small
grammar engine of its own:

* :func:`parse_lark` reads the commonly used part of Lark's grammar syntax -- rules and terminals, string literals
  (with the ``i`` flag), regular-expression terminals (character classes, ``.``, groups, alternation, ``? * +
  {m,n}``), the operators ``| ? * + ~n ~n..m``, ``( )`` groups, ``[ ]`` options, ``%ignore`` and ``%import
  common.X`` for the usual terminals -- into a scannerless grammar over character classes;
* :func:`schema_to_grammar` turns a JSON Schema into such a grammar: nested objects with required and optional
  properties, ``additionalProperties``, arrays with ``items`` / ``prefixItems`` / ``minItems`` / ``maxItems``,
  ``enum`` / ``const``, ``anyOf`` / ``oneOf``, type unions, ``$ref`` into ``$defs`` (recursive schemas included),
  string ``pattern`` / ``minLength`` / ``maxLength`` / a few ``format`` values;
* :class:`GrammarConstraint` is an incremental Earley recogniser over characters whose item sets are hash-consed
  into a lazily built automaton (origins are set ids, not input positions), so a transition is computed once.
  ``allowed`` walks the vocabulary as a trie -- tokens that share a prefix share the work -- and masks are memoised
  per automaton state.

Everything is exact at the character level: a token is allowed iff the text so far plus the token is a prefix of
some sentence of the grammar.
"""
from __future__ import annotations

import json
import re as _re

import numpy as np

# ---------------------------------------------------------------------------------------------
# grammar representation: rules[name] = list of productions; a production is a tuple of symbols;
# a symbol is a rule name (str) or a CharSet
# ---------------------------------------------------------------------------------------------


class CharSet:
    """A set of characters given as sorted code-point ranges, possibly negated."""

    __slots__ = ("ranges", "negated", "_hash")

    def __init__(self, ranges, negated=False):
        rs = sorted((int(a), int(b)) for a, b in ranges)
        merged = []
        for a, b in rs:
            if merged and a <= merged[-1][1] + 1:
                merged[-1] = (merged[-1][0], max(merged[-1][1], b))
            else:
                merged.append((a, b))
        self.ranges = tuple(merged)
        self.negated = bool(negated)
        self._hash = hash((self.ranges, self.negated))

    @classmethod
    def of(cls, chars: str):
        return cls([(ord(c), ord(c)) for c in chars])

    def __contains__(self, ch: str) -> bool:
        o = ord(ch)
        hit = False
        for a, b in self.ranges:
            if a <= o <= b:
                hit = True
                break
            if o < a:
                break
        return hit != self.negated

    def __eq__(self, other):
        return isinstance(other, CharSet) and self.ranges == other.ranges and self.negated == other.negated

    def __hash__(self):
        return self._hash

    def __repr__(self):
        return ("^" if self.negated else "") + "".join(chr(a) if a == b else f"{chr(a)}-{chr(b)}" for a, b in self.ranges)


class Grammar:
    def __init__(self, start: str = "start"):
        self.rules: dict[str, list[tuple]] = {}
        self.start = start
        self._n = 0

    def fresh(self, hint: str = "g") -> str:
        self._n += 1
        return f"_{hint}{self._n}"

    def add(self, name: str, *productions) -> str:
        self.rules.setdefault(name, []).extend(tuple(p) for p in productions)
        return name

    # -- combinators that allocate helper rules ------------------------------------------------
    def lit(self, text: str, ignore_case: bool = False) -> tuple:
        if not ignore_case:
            return tuple(CharSet.of(c) for c in text)
        return tuple(CharSet.of(c.lower() + c.upper()) if c.lower() != c.upper() else CharSet.of(c) for c in text)

    def alt(self, *alternatives) -> str:
        return self.add(self.fresh("alt"), *alternatives)

    def opt(self, seq) -> str:
        return self.add(self.fresh("opt"), tuple(seq), ())

    def star(self, seq) -> str:
        # left-recursive on purpose: the recogniser's item sets then repeat inside a loop (same origin at every turn),
        # which is what lets its transition table stay small
        name = self.fresh("star")
        return self.add(name, (), (name,) + tuple(seq))

    def plus(self, seq) -> str:
        return self.add(self.fresh("plus"), tuple(seq) + (self.star(seq),))

    def repeat(self, seq, lo: int, hi: int | None) -> tuple:
        seq = tuple(seq)
        out = seq * lo
        if hi is None:
            return out + (self.star(seq),)
        tail = ()
        for _ in range(hi - lo):                      # nested options: (x (x (x)?)?)?
            tail = (self.opt(seq + tail),)
        return out + tail

    def validate(self) -> None:
        for name, prods in self.rules.items():
            for p in prods:
                for sym in p:
                    if isinstance(sym, str) and sym not in self.rules:
                        raise ValueError(f"rule {name!r} uses {sym!r}, which is not defined")
        if self.start not in self.rules:
            raise ValueError(f"the grammar has no {self.start!r} rule")


# ---------------------------------------------------------------------------------------------
# a regular-expression subset compiled into grammar rules
# ---------------------------------------------------------------------------------------------
_CLASS_ESC = {"d": [(48, 57)], "w": [(48, 57), (65, 90), (95, 95), (97, 122)], "s": [(9, 13), (32, 32)]}
_SIMPLE_ESC = {"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v", "0": "\0"}
ANY_CHAR = CharSet([], negated=True)
ANY_BUT_NEWLINE = CharSet([(10, 10)], negated=True)


def _invert(ranges):
    out, prev = [], 0
    for a, b in sorted(ranges):
        if a > prev:
            out.append((prev, a - 1))
        prev = max(prev, b + 1)
    out.append((prev, 0x10FFFF))
    return out


class _RegexCompiler:
    def __init__(self, g: Grammar, pattern: str, ignore_case: bool = False, dotall: bool = False):
        self.g, self.p, self.i, self.ic, self.dotall = g, pattern, 0, ignore_case, dotall

    def error(self, msg):
        return ValueError(f"regular expression {self.p!r}: {msg} at position {self.i}")

    def parse(self) -> tuple:
        seq = self.alternation()
        if self.i != len(self.p):
            raise self.error("unbalanced ')'")
        return seq

    def alternation(self) -> tuple:
        branches = [self.sequence()]
        while self.i < len(self.p) and self.p[self.i] == "|":
            self.i += 1
            branches.append(self.sequence())
        return branches[0] if len(branches) == 1 else (self.g.alt(*branches),)

    def sequence(self) -> tuple:
        out = ()
        while self.i < len(self.p) and self.p[self.i] not in "|)":
            atom = self.atom()
            out += self.quantified(atom)
        return out

    def quantified(self, atom: tuple) -> tuple:
        if self.i >= len(self.p):
            return atom
        c = self.p[self.i]
        if c in "?*+":
            self.i += 1
            if self.i < len(self.p) and self.p[self.i] in "?+":      # lazy / possessive marks do not change the language
                self.i += 1
            return (self.g.opt(atom),) if c == "?" else (self.g.star(atom),) if c == "*" else (self.g.plus(atom),)
        if c == "{":
            m = _re.match(r"\{(\d*)(,?)(\d*)\}", self.p[self.i:])
            if m and (m.group(1) or m.group(3)):
                self.i += m.end()
                lo = int(m.group(1) or 0)
                hi = lo if not m.group(2) else (int(m.group(3)) if m.group(3) else None)
                if hi is not None and hi < lo:
                    raise self.error("a repetition range runs backwards")
                if (hi or lo) > 1000:
                    raise self.error("a repetition count above 1000")
                return self.g.repeat(atom, lo, hi)
        return atom

    def charset(self, ranges, negated=False) -> CharSet:
        if self.ic:
            extra = []
            for a, b in ranges:
                for lo, hi, delta in ((65, 90, 32), (97, 122, -32)):
                    x, y = max(a, lo), min(b, hi)
                    if x <= y:
                        extra.append((x + delta, y + delta))
            ranges = list(ranges) + extra
        return CharSet(ranges, negated)

    def escape(self):
        """After a backslash: returns ranges (a class) for \\d \\w \\s and their negations, or a single character."""
        if self.i >= len(self.p):
            raise self.error("a trailing backslash")
        c = self.p[self.i]
        self.i += 1
        if c in _CLASS_ESC:
            return list(_CLASS_ESC[c])
        if c.lower() in _CLASS_ESC and c.isupper():
            return _invert(_CLASS_ESC[c.lower()])
        if c in _SIMPLE_ESC:
            return _SIMPLE_ESC[c]
        if c == "x":
            h = self.p[self.i:self.i + 2]
            if not _re.fullmatch(r"[0-9a-fA-F]{2}", h):
                raise self.error("\\x needs two hex digits")
            self.i += 2
            return chr(int(h, 16))
        if c == "u":
            h = self.p[self.i:self.i + 4]
            if not _re.fullmatch(r"[0-9a-fA-F]{4}", h):
                raise self.error("\\u needs four hex digits")
            self.i += 4
            return chr(int(h, 16))
        if c.isalnum():
            raise self.error(f"the escape \\{c} is not supported")
        return c

    def atom(self) -> tuple:
        c = self.p[self.i]
        if c == "(":
            self.i += 1
            if self.p.startswith("?:", self.i):
                self.i += 2
            elif self.p.startswith("?", self.i):
                raise self.error("look-around and named groups are not supported")
            inner = self.alternation()
            if self.i >= len(self.p) or self.p[self.i] != ")":
                raise self.error("a '(' without its ')'")
            self.i += 1
            return (self.g.add(self.g.fresh("grp"), inner),)
        if c == "[":
            return (self.char_class(),)
        self.i += 1
        if c == ".":
            return (ANY_CHAR if self.dotall else ANY_BUT_NEWLINE,)
        if c in "^$":
            return ()                                     # the whole output is matched: anchors are implied
        if c == "\\":
            e = self.escape()
            return (self.charset(e),) if isinstance(e, list) else (self.charset([(ord(e), ord(e))]),)
        if c in "*+?{" and c != "{":
            raise self.error(f"nothing to repeat before '{c}'")
        return (self.charset([(ord(c), ord(c))]),)

    def char_class(self) -> CharSet:
        self.i += 1
        negated = self.p.startswith("^", self.i)
        if negated:
            self.i += 1
        ranges, first = [], True
        while True:
            if self.i >= len(self.p):
                raise self.error("a '[' without its ']'")
            c = self.p[self.i]
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            if c == "\\":
                e = self.escape()
                if isinstance(e, list):
                    ranges += e
                    continue
                c = e
            if self.p.startswith("-", self.i) and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                self.i += 1
                hi = self.p[self.i]
                self.i += 1
                if hi == "\\":
                    e = self.escape()
                    if isinstance(e, list):
                        raise self.error("a character class cannot end a range")
                    hi = e
                if ord(hi) < ord(c):
                    raise self.error("a character range runs backwards")
                ranges.append((ord(c), ord(hi)))
            else:
                ranges.append((ord(c), ord(c)))
        return self.charset(ranges, negated)


def regex_to_symbols(g: Grammar, pattern: str, ignore_case=False, dotall=False) -> tuple:
    return _RegexCompiler(g, pattern, ignore_case, dotall).parse()


# ---------------------------------------------------------------------------------------------
# Lark syntax
# ---------------------------------------------------------------------------------------------
_COMMON = {
    "DIGIT": r"[0-9]", "HEXDIGIT": r"[0-9a-fA-F]", "INT": r"[0-9]+", "SIGNED_INT": r"[+-]?[0-9]+",
    "DECIMAL": r"[0-9]+\.[0-9]*|\.[0-9]+", "FLOAT": r"[0-9]+(\.[0-9]*)?[eE][+-]?[0-9]+|[0-9]+\.[0-9]*|\.[0-9]+",
    "NUMBER": r"[0-9]+(\.[0-9]*)?([eE][+-]?[0-9]+)?|\.[0-9]+([eE][+-]?[0-9]+)?",
    "SIGNED_NUMBER": r"[+-]?([0-9]+(\.[0-9]*)?([eE][+-]?[0-9]+)?|\.[0-9]+([eE][+-]?[0-9]+)?)",
    "ESCAPED_STRING": r'"([^"\\\n]|\\.)*"', "LCASE_LETTER": r"[a-z]", "UCASE_LETTER": r"[A-Z]", "LETTER": r"[a-zA-Z]",
    "WORD": r"[a-zA-Z]+", "CNAME": r"[a-zA-Z_][a-zA-Z0-9_]*", "WS_INLINE": r"[ \t]+", "WS": r"[ \t\f\r\n]+", "CR": r"\r",
    "LF": r"\n", "NEWLINE": r"(\r?\n)+", "SH_COMMENT": r"#[^\n]*", "CPP_COMMENT": r"//[^\n]*",
}
_TOKEN_RE = _re.compile(r"""
    (?P<ws>[ \t]+) | (?P<comment>//[^\n]*) | (?P<nl>\r?\n) |
    (?P<string>"(?:[^"\\\n]|\\.)*"i?) | (?P<regex>/(?:[^/\\\n]|\\.)+/[imslux]*) |
    (?P<name>[?!]?[a-zA-Z_][a-zA-Z0-9_]*(?:\.[a-zA-Z_][a-zA-Z0-9_.]*)?) | (?P<directive>%[a-z]+) |
    (?P<range>~\s*\d+(?:\s*\.\.\s*\d+)?) | (?P<num>\d+) | (?P<arrow>->\s*[a-zA-Z_][a-zA-Z0-9_]*) | (?P<op>[:|()\[\]?*+,.])
""", _re.X)


def _unquote(tok: str):
    ic = tok.endswith("i")
    body = tok[1:-2] if ic else tok[1:-1]
    out, i = [], 0
    while i < len(body):
        c = body[i]
        if c == "\\" and i + 1 < len(body):
            n = body[i + 1]
            if n in _SIMPLE_ESC:
                out.append(_SIMPLE_ESC[n]); i += 2; continue
            if n == "x" and _re.fullmatch(r"[0-9a-fA-F]{2}", body[i + 2:i + 4]):
                out.append(chr(int(body[i + 2:i + 4], 16))); i += 4; continue
            if n == "u" and _re.fullmatch(r"[0-9a-fA-F]{4}", body[i + 2:i + 6]):
                out.append(chr(int(body[i + 2:i + 6], 16))); i += 6; continue
            out.append(n); i += 2; continue
        out.append(c); i += 1
    return "".join(out), ic


def parse_lark(text: str, start: str = "start") -> Grammar:
    """Lark grammar text -> :class:`Grammar` (scannerless: terminals become rules over characters).  ``%ignore``d
    terminals may appear between any two items of a rule (lower-case name) and at both ends of the input."""
    g = Grammar(start)
    toks, line, pos = [], 1, 0
    while pos < len(text):
        m = _TOKEN_RE.match(text, pos)
        if not m:
            raise ValueError(f"Lark grammar, line {line}: cannot read {text[pos:pos + 20]!r}")
        pos = m.end()
        kind = m.lastgroup
        if kind == "nl":
            toks.append(("nl", "\n", line))
            line += 1
        elif kind not in ("ws", "comment"):
            toks.append((kind, m.group(), line))
    toks.append(("nl", "\n", line))
    # split into statements: a statement ends at a newline unless the next line starts with '|'
    stmts, cur = [], []
    for i, t in enumerate(toks):
        if t[0] == "nl":
            nxt = next((u for u in toks[i + 1:] if u[0] != "nl"), None)
            if cur and not (nxt and nxt[1] == "|"):
                stmts.append(cur)
                cur = []
        else:
            cur.append(t)
    ignored: list[str] = []
    defs: list = []
    for st in stmts:
        kind, val, ln = st[0]
        if kind == "directive":
            if val == "%ignore":
                defs.append(("ignore", st[1:], ln))
            elif val == "%import":
                names = [t[1] for t in st[1:] if t[0] == "name"]
                if not names or not names[0].startswith("common."):
                    raise ValueError(f"Lark grammar, line {ln}: only `%import common.NAME` is available")
                src = names[0].split(".", 1)[1]
                alias = st[-1][1].split()[-1] if st[-1][0] == "arrow" else (names[1] if len(names) > 1 else src)
                imports = [src] if not any(t[1] == "(" for t in st) else [t[1] for t in st[2:] if t[0] == "name"]
                for name in imports:
                    if name not in _COMMON:
                        raise ValueError(f"Lark grammar, line {ln}: common.{name} is not one of {sorted(_COMMON)}")
                    target = alias if len(imports) == 1 else name
                    g.add(target, regex_to_symbols(g, _COMMON[name]))
            elif val in ("%declare", "%override", "%extend"):
                raise ValueError(f"Lark grammar, line {ln}: {val} is not supported")
            else:
                raise ValueError(f"Lark grammar, line {ln}: unknown directive {val}")
            continue
        if kind != "name" or len(st) < 2:
            raise ValueError(f"Lark grammar, line {ln}: expected `name: expansion`")
        name = val.lstrip("?!")
        j = 1
        if st[j][0] == "op" and st[j][1] == "." and st[j + 1][0] == "num":       # priority: NAME.2: ...
            j += 2
        if not (st[j][0] == "op" and st[j][1] == ":"):
            raise ValueError(f"Lark grammar, line {ln}: expected ':' after {name!r}")
        defs.append(("rule", name, st[j + 1:], ln))
    ign_rule = None
    ign_defs = [d for d in defs if d[0] == "ignore"]
    if ign_defs:
        ign_rule = "_ignored"
    parser = _LarkBody(g)
    for d in defs:
        if d[0] == "rule":
            _, name, body, ln = d
            is_terminal = name.isupper() or name.lstrip("_").isupper()
            alts = parser.expansions(body, ln, None if is_terminal else ign_rule)
            g.add(name, *alts)
    if ign_rule:
        items = []
        for _, body, ln in ign_defs:
            items += parser.expansions(body, ln, None)
        one = g.add(g.fresh("ign"), *items)
        g.add(ign_rule, (), (ign_rule, one))
        real = g.start
        g.start = g.add("_start_with_ignored", (ign_rule, real, ign_rule))
    g.validate()
    return g


class _LarkBody:
    def __init__(self, g: Grammar):
        self.g = g

    def expansions(self, toks, ln, ign):
        self.t, self.i, self.ln, self.ign = [t for t in toks if t[0] != "arrow"], 0, ln, ign
        alts = self.alts()
        if self.i != len(self.t):
            raise ValueError(f"Lark grammar, line {ln}: unexpected {self.t[self.i][1]!r}")
        return alts

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None, self.ln)

    def alts(self):
        out = [self.seq()]
        while self.peek()[1] == "|":
            self.i += 1
            out.append(self.seq())
        return out

    def seq(self):
        items = []
        while self.peek()[0] is not None and self.peek()[1] not in ("|", ")", "]"):
            items.append(self.item())
        out = ()
        for k, it in enumerate(items):
            if k and self.ign:
                out += (self.ign,)
            out += it
        return out

    def item(self):
        kind, val, _ = self.peek()
        self.i += 1
        g = self.g
        if val == "(":
            alts = self.alts()
            if self.peek()[1] != ")":
                raise ValueError(f"Lark grammar, line {self.ln}: a '(' without its ')'")
            self.i += 1
            atom = (g.add(g.fresh("grp"), *alts),)
        elif val == "[":
            alts = self.alts()
            if self.peek()[1] != "]":
                raise ValueError(f"Lark grammar, line {self.ln}: a '[' without its ']'")
            self.i += 1
            atom = (g.add(g.fresh("opt"), *alts, ()),)
        elif kind == "string":
            s, ic = _unquote(val)
            atom = g.lit(s, ic)
            if self.peek()[1] == "." and self.i + 2 < len(self.t) + 1 and self.t[self.i + 1][1] == "." and self.t[self.i + 2][0] == "string":
                hi, _ = _unquote(self.t[self.i + 2][1])          # "a".."z"
                if len(s) != 1 or len(hi) != 1:
                    raise ValueError(f"Lark grammar, line {self.ln}: a character range needs one-character strings")
                atom = (CharSet([(ord(s), ord(hi))]),)
                self.i += 3
        elif kind == "regex":
            end = val.rindex("/")
            flags = val[end + 1:]
            atom = (g.add(g.fresh("rx"), regex_to_symbols(g, val[1:end], "i" in flags, "s" in flags)),)
        elif kind == "name":
            atom = (val.lstrip("?!"),)
        else:
            raise ValueError(f"Lark grammar, line {self.ln}: unexpected {val!r}")
        # postfix operators
        while True:
            kind, val, _ = self.peek()
            sep = (self.ign,) if self.ign else ()
            if val == "?":
                atom = (g.opt(atom),)
            elif val == "*":
                atom = (g.star(atom + sep),) if sep else (g.star(atom),)
                if sep:                                   # x (ign x)* without a trailing ignored run inside the loop
                    inner = atom
                    atom = inner
            elif val == "+":
                atom = (g.plus(atom + sep),) if sep else (g.plus(atom),)
            elif kind == "range":
                nums = [int(n) for n in _re.findall(r"\d+", val)]
                lo, hi = nums[0], nums[-1]
                if hi < lo:
                    raise ValueError(f"Lark grammar, line {self.ln}: the repetition {val} runs backwards")
                atom = g.repeat(atom + sep, lo, hi)
            else:
                return atom
            self.i += 1


# ---------------------------------------------------------------------------------------------
# JSON Schema -> grammar
# ---------------------------------------------------------------------------------------------
_JSON_WS = CharSet.of(" \t\n\r")
_FORMATS = {
    "date": r"[0-9]{4}-(0[1-9]|1[0-2])-(0[1-9]|[12][0-9]|3[01])",
    "time": r"([01][0-9]|2[0-3]):[0-5][0-9]:[0-5][0-9](\.[0-9]+)?(Z|[+-]([01][0-9]|2[0-3]):[0-5][0-9])?",
    "date-time": r"[0-9]{4}-(0[1-9]|1[0-2])-(0[1-9]|[12][0-9]|3[01])T([01][0-9]|2[0-3]):[0-5][0-9]:[0-5][0-9](\.[0-9]+)?(Z|[+-]([01][0-9]|2[0-3]):[0-5][0-9])",
    "uuid": r"[0-9a-fA-F]{8}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{12}",
    "ipv4": r"((25[0-5]|2[0-4][0-9]|1[0-9][0-9]|[1-9]?[0-9])\.){3}(25[0-5]|2[0-4][0-9]|1[0-9][0-9]|[1-9]?[0-9])",
    "email": r"[a-zA-Z0-9._%+-]+@[a-zA-Z0-9-]+(\.[a-zA-Z0-9-]+)+",
}
_IGNORED_KEYS = {"title", "description", "default", "examples", "$schema", "$id", "$comment", "deprecated", "readOnly", "writeOnly",
                 "minimum", "maximum", "exclusiveMinimum", "exclusiveMaximum", "multipleOf", "uniqueItems", "$defs", "definitions",
                 "propertyNames", "minProperties", "maxProperties", "contentEncoding", "contentMediaType"}
_KNOWN_KEYS = _IGNORED_KEYS | {"type", "enum", "const", "properties", "required", "additionalProperties", "items", "prefixItems",
                               "minItems", "maxItems", "anyOf", "oneOf", "allOf", "$ref", "pattern", "minLength", "maxLength", "format",
                               "nullable"}


class _SchemaCompiler:
    def __init__(self, root):
        self.g = Grammar("start")
        self.root = root
        self.refs: dict[str, str] = {}
        g = self.g
        g.add("ws", (), ("ws", _JSON_WS))
        plain = CharSet([(0, 31), (34, 34), (92, 92)], negated=True)
        hexd = CharSet([(48, 57), (65, 70), (97, 102)])
        g.add("char", (plain,), (CharSet.of("\\"), CharSet.of('"\\/bfnrt')), (CharSet.of("\\"), CharSet.of("u"), hexd, hexd, hexd, hexd))
        g.add("chars", (), ("chars", "char"))
        g.add("string", (CharSet.of('"'), "chars", CharSet.of('"')))
        g.add("integer", regex_to_symbols(g, r"-?(0|[1-9][0-9]*)"))
        g.add("number", regex_to_symbols(g, r"-?(0|[1-9][0-9]*)(\.[0-9]+)?([eE][+-]?[0-9]+)?"))
        g.add("boolean", g.lit("true"), g.lit("false"))
        g.add("null", g.lit("null"))
        g.add("value", ("string",), ("number",), ("boolean",), ("null",), ("any_object",), ("any_array",))
        g.add("member", ("string", "ws", CharSet.of(":"), "ws", "value"))
        g.add("members", ("member",), ("members", "ws", CharSet.of(","), "ws", "member"))
        g.add("any_object", (CharSet.of("{"), "ws", CharSet.of("}")), (CharSet.of("{"), "ws", "members", "ws", CharSet.of("}")))
        g.add("elements", ("value",), ("elements", "ws", CharSet.of(","), "ws", "value"))
        g.add("any_array", (CharSet.of("["), "ws", CharSet.of("]")), (CharSet.of("["), "ws", "elements", "ws", CharSet.of("]")))

    def compile(self) -> Grammar:
        top = self.node(self.root, "#")
        self.g.add("start", ("ws", top, "ws"))
        self.g.validate()
        return self.g

    def resolve(self, ref: str):
        if not ref.startswith("#"):
            raise ValueError(f"JSON schema: only local references are supported, not {ref!r}")
        node = self.root
        for part in [p for p in ref[1:].split("/") if p]:
            part = part.replace("~1", "/").replace("~0", "~")
            if not isinstance(node, dict) or part not in node:
                raise ValueError(f"JSON schema: the reference {ref!r} points nowhere")
            node = node[part]
        return node

    def node(self, schema, where: str) -> str:
        """Returns the name of a rule that derives exactly the JSON texts valid against ``schema``."""
        g = self.g
        if schema is True or schema == {}:
            return "value"
        if schema is False:
            raise ValueError(f"JSON schema at {where}: `false` admits nothing")
        if not isinstance(schema, dict):
            raise ValueError(f"JSON schema at {where}: a schema must be an object or a boolean")
        unknown = [k for k in schema if k not in _KNOWN_KEYS and not k.startswith("x-")]
        if unknown:
            raise ValueError(f"JSON schema at {where}: keyword {unknown[0]!r} is not supported")
        if "$ref" in schema:
            ref = schema["$ref"]
            if ref not in self.refs:
                self.refs[ref] = g.fresh("ref")                  # registered before it is compiled: recursion closes the loop
                target = self.node(self.resolve(ref), ref)
                g.add(self.refs[ref], (target,))
            return self.refs[ref]
        if "const" in schema:
            return g.add(g.fresh("const"), g.lit(json.dumps(schema["const"], ensure_ascii=False)))
        if "enum" in schema:
            if not schema["enum"]:
                raise ValueError(f"JSON schema at {where}: an empty enum admits nothing")
            return g.add(g.fresh("enum"), *[g.lit(json.dumps(v, ensure_ascii=False)) for v in schema["enum"]])
        for key in ("anyOf", "oneOf"):
            if key in schema:
                rest = {k: v for k, v in schema.items() if k != key}
                alts = [self.node({**rest, **alt} if isinstance(alt, dict) else alt, f"{where}/{key}/{i}")
                        for i, alt in enumerate(schema[key])]
                return g.add(g.fresh("any"), *[(a,) for a in alts])
        if "allOf" in schema:
            merged = {k: v for k, v in schema.items() if k != "allOf"}
            for i, part in enumerate(schema["allOf"]):
                if not isinstance(part, dict):
                    raise ValueError(f"JSON schema at {where}/allOf/{i}: only object schemas can be merged")
                part = self.resolve(part["$ref"]) if set(part) == {"$ref"} else part
                for k, v in part.items():
                    if k == "properties":
                        merged.setdefault("properties", {}).update(v)
                    elif k == "required":
                        merged["required"] = list(merged.get("required", [])) + [r for r in v if r not in merged.get("required", [])]
                    elif k in merged and merged[k] != v and k not in _IGNORED_KEYS:
                        raise ValueError(f"JSON schema at {where}/allOf: parts disagree on {k!r}")
                    else:
                        merged[k] = v
            return self.node(merged, where)
        types = schema.get("type")
        if types is None:
            if "properties" in schema or "required" in schema or "additionalProperties" in schema:
                types = "object"
            elif "items" in schema or "prefixItems" in schema:
                types = "array"
            elif any(k in schema for k in ("pattern", "minLength", "maxLength", "format")):
                types = "string"
            else:
                return "value"
        if isinstance(types, list):
            alts = [self.node({**schema, "type": t}, where) for t in types]
            if schema.get("nullable") and "null" not in types:
                alts.append("null")
            return g.add(g.fresh("types"), *[(a,) for a in alts])
        if schema.get("nullable") and types != "null":
            inner = self.node({k: v for k, v in schema.items() if k != "nullable"}, where)
            return g.add(g.fresh("nullable"), (inner,), ("null",))
        if types in ("integer", "number", "boolean", "null"):
            return types
        if types == "string":
            return self.string(schema, where)
        if types == "array":
            return self.array(schema, where)
        if types == "object":
            return self.object(schema, where)
        raise ValueError(f"JSON schema at {where}: unknown type {types!r}")

    def string(self, schema, where):
        g = self.g
        if "pattern" in schema or schema.get("format") in _FORMATS:
            pat = schema.get("pattern") or _FORMATS[schema["format"]]
            # the pattern describes the string's value; characters JSON must escape cannot occur unescaped, so patterns
            # are taken to speak about the text between the quotes
            body = regex_to_symbols(g, pat.lstrip("^").rstrip("$") if not pat.endswith("\\$") else pat.lstrip("^"))
            return g.add(g.fresh("pstr"), (CharSet.of('"'),) + body + (CharSet.of('"'),))
        lo, hi = int(schema.get("minLength", 0)), schema.get("maxLength")
        if lo == 0 and hi is None:
            return "string"
        if hi is not None and int(hi) < lo:
            raise ValueError(f"JSON schema at {where}: maxLength is below minLength")
        return g.add(g.fresh("lstr"), (CharSet.of('"'),) + g.repeat(("char",), lo, None if hi is None else int(hi)) + (CharSet.of('"'),))

    def array(self, schema, where):
        g = self.g
        prefix = [self.node(s, f"{where}/prefixItems/{i}") for i, s in enumerate(schema.get("prefixItems", []))]
        items = schema.get("items", True)
        item = None if items is False else self.node(items, f"{where}/items")
        lo = int(schema.get("minItems", 0))
        hi = schema.get("maxItems")
        hi = None if hi is None else int(hi)
        if hi is not None and hi < lo:
            raise ValueError(f"JSON schema at {where}: maxItems is below minItems")
        comma = ("ws", CharSet.of(","), "ws")
        # positions: prefix items first, then `item` repeated
        seqs = []
        max_n = hi if hi is not None else max(lo, len(prefix)) + 1
        for n in range(lo, max_n + 1):
            if n > len(prefix) and item is None:
                break
            elems = [prefix[i] if i < len(prefix) else item for i in range(n)]
            seq = ()
            for k, e in enumerate(elems):
                seq += (comma if k else ()) + (e,)
            if hi is None and n == max_n and item is not None:
                more = g.star(comma + (item,))
                seq = seq + (more,) if n else (g.opt((item, more)),)
            seqs.append(seq)
        if not seqs:
            raise ValueError(f"JSON schema at {where}: the array bounds admit nothing")
        body = g.add(g.fresh("elems"), *seqs)
        return g.add(g.fresh("arr"), (CharSet.of("["), "ws", body, "ws", CharSet.of("]")))

    def object(self, schema, where):
        g = self.g
        props = schema.get("properties", {})
        required = set(schema.get("required", []))
        missing = required - set(props)
        extra = schema.get("additionalProperties", True)
        comma = ("ws", CharSet.of(","), "ws")
        members = []
        for name, sub in props.items():
            val = self.node(sub, f"{where}/properties/{name}")
            members.append((g.lit(json.dumps(name, ensure_ascii=False)) + ("ws", CharSet.of(":"), "ws", val), name in required))
        for name in sorted(missing):                          # required but undeclared: any value
            members.append((g.lit(json.dumps(name, ensure_ascii=False)) + ("ws", CharSet.of(":"), "ws", "value"), True))
        extra_member = None
        if extra is not False:
            ev = "value" if extra is True else self.node(extra, f"{where}/additionalProperties")
            extra_member = ("string", "ws", CharSet.of(":"), "ws", ev)
        # Declared properties appear in declaration order, optional ones may be skipped, additional ones follow.
        # rest[i] derives the members from position i on, each preceded by a comma when something came before.
        n = len(members)
        tail_first = tail_more = None
        if extra_member is not None:
            more = g.star(comma + extra_member)
            tail_more = g.add(g.fresh("xmore"), (more,))                         # after at least one member
            tail_first = g.add(g.fresh("xfirst"), (), extra_member + (more,))    # nothing before it
        after = [None] * (n + 1)       # after[i]: members i.. given that something precedes
        first = [None] * (n + 1)       # first[i]: members i.. given that nothing precedes
        after[n] = tail_more if tail_more else g.add(g.fresh("end"), ())
        first[n] = tail_first if tail_first else g.add(g.fresh("end"), ())
        for i in range(n - 1, -1, -1):
            seq, req = members[i]
            a_alts = [comma + seq + (after[i + 1],)]
            f_alts = [seq + (after[i + 1],)]
            if not req:
                a_alts.append((after[i + 1],))
                f_alts.append((first[i + 1],))
            after[i] = g.add(g.fresh("oa"), *a_alts)
            first[i] = g.add(g.fresh("of"), *f_alts)
        return g.add(g.fresh("obj"), (CharSet.of("{"), "ws", first[0], "ws", CharSet.of("}")))


def schema_to_grammar(schema) -> Grammar:
    return _SchemaCompiler(schema).compile()


# ---------------------------------------------------------------------------------------------
# Earley recogniser over characters
# ---------------------------------------------------------------------------------------------
class _Compiled:
    """Rules numbered, nullable set, and per-rule production lists in a form the recogniser indexes quickly."""

    def __init__(self, g: Grammar):
        g.validate()
        self.names = list(g.rules)
        self.index = {n: i for i, n in enumerate(self.names)}
        self.prods: list[list[tuple]] = []
        for n in self.names:
            self.prods.append([tuple(self.index[s] if isinstance(s, str) else s for s in p) for p in g.rules[n]])
        self.start = self.index[g.start]
        nullable = set()
        changed = True
        while changed:
            changed = False
            for r, prods in enumerate(self.prods):
                if r not in nullable and any(all(isinstance(s, int) and s in nullable for s in p) for p in prods):
                    nullable.add(r)
                    changed = True
        self.nullable = nullable


_SELF = -1      # origin marker: "the set this item sits in"


class _Automaton:
    """Earley item sets of one grammar, hash-consed, with a cached transition table.

    An item is ``(rule, production, dot, origin)`` where ``origin`` is the id of the item set in which the item's
    rule was predicted (``_SELF`` while that is the set being described).  Because origins are set ids rather than
    input positions, a set's content says everything about what can follow it: two prefixes that reach the same set
    id have the same futures, ``(set id, character) -> set id`` is a function, and it is built lazily like the
    transition table of a deterministic automaton.  Left-recursive repetition (see :meth:`Grammar.star`) keeps the
    number of sets small."""

    def __init__(self, compiled: _Compiled):
        self.c = compiled
        self.sets: list[frozenset] = []
        self.ids: dict = {}
        self.trans: dict = {}
        self.complete: list[bool] = []
        c = compiled
        self.start_id = self._intern(self._close({(c.start, k, 0, _SELF) for k in range(len(c.prods[c.start]))}), root=True)

    def _intern(self, items: frozenset, root: bool = False) -> int:
        sid = self.ids.get(items)
        if sid is None:
            sid = len(self.sets)
            self.ids[items] = sid
            self.sets.append(items)
            c = self.c
            # the start rule is predicted only in the root set, whose items carry origin _SELF there and the root's id
            # (0) once they have been scanned into later sets
            self.complete.append(any(r == c.start and d == len(c.prods[r][k]) and (o == 0 or (root and o == _SELF))
                                     for (r, k, d, o) in items))
        return sid

    def _close(self, kernel) -> frozenset:
        c = self.c
        out = set(kernel)
        work = list(kernel)
        while work:
            r, k, d, o = work.pop()
            prod = c.prods[r][k]
            if d < len(prod):
                sym = prod[d]
                if isinstance(sym, int):
                    for k2 in range(len(c.prods[sym])):
                        it = (sym, k2, 0, _SELF)
                        if it not in out:
                            out.add(it)
                            work.append(it)
                    if sym in c.nullable:
                        it = (r, k, d + 1, o)
                        if it not in out:
                            out.add(it)
                            work.append(it)
            elif o == _SELF:
                for (r2, k2, d2, o2) in list(out):                   # an empty derivation: its parents sit in this very set
                    p2 = c.prods[r2][k2]
                    if d2 < len(p2) and p2[d2] == r:
                        it = (r2, k2, d2 + 1, o2)
                        if it not in out:
                            out.add(it)
                            work.append(it)
            else:
                for (r2, k2, d2, o2) in self.sets[o]:
                    p2 = c.prods[r2][k2]
                    if d2 < len(p2) and p2[d2] == r:
                        it = (r2, k2, d2 + 1, o if o2 == _SELF else o2)   # "that set itself" becomes its id when seen from here
                        if it not in out:
                            out.add(it)
                            work.append(it)
        return frozenset(out)

    def step(self, sid: int, ch: str) -> int:
        """Id of the set after ``ch``, or -1 when no sentence continues that way."""
        key = (sid, ch)
        hit = self.trans.get(key)
        if hit is not None:
            return hit
        c = self.c
        kernel = set()
        for (r, k, d, o) in self.sets[sid]:
            prod = c.prods[r][k]
            if d < len(prod):
                sym = prod[d]
                if not isinstance(sym, int) and ch in sym:
                    kernel.add((r, k, d + 1, sid if o == _SELF else o))
        nxt = self._intern(self._close(kernel)) if kernel else -1
        self.trans[key] = nxt
        return nxt


class EarleyState:
    """A position in the automaton of item sets (immutable: ``feed`` returns a new state)."""

    __slots__ = ("a", "sid")

    def __init__(self, automaton: _Automaton, sid: int | None = None):
        self.a = automaton
        self.sid = automaton.start_id if sid is None else sid

    def feed(self, ch: str):
        nxt = self.a.step(self.sid, ch)
        return None if nxt < 0 else EarleyState(self.a, nxt)

    def feed_text(self, text: str):
        sid, step = self.sid, self.a.step
        for ch in text:
            sid = step(sid, ch)
            if sid < 0:
                return None
        return EarleyState(self.a, sid)

    @property
    def complete(self) -> bool:
        return self.a.complete[self.sid]

    def signature(self):
        return self.sid


class _Trie:
    __slots__ = ("children", "tokens")

    def __init__(self):
        self.children: dict = {}
        self.tokens: list = []


_TRIES: dict = {}


def _trie_for(token_texts):
    key = id(token_texts)
    hit = _TRIES.get(key)
    if hit is not None and hit[0] is token_texts:
        return hit[1]
    root = _Trie()
    for i, t in enumerate(token_texts):
        if not t:
            continue
        node = root
        for ch in t:
            nxt = node.children.get(ch)
            if nxt is None:
                nxt = node.children[ch] = _Trie()
            node = nxt
        node.tokens.append(i)
    if len(_TRIES) > 8:
        _TRIES.clear()
    _TRIES[key] = (token_texts, root)
    return root


class GrammarConstraint:
    """The whole output must be a sentence of ``grammar``."""

    name = "grammar"

    def __init__(self, grammar: Grammar, name: str = "grammar"):
        self.automaton = _Automaton(_Compiled(grammar))
        self.state = EarleyState(self.automaton)
        self.name = name
        self._memo: dict = {}

    def allowed(self, token_texts) -> np.ndarray:
        key = (self.state.signature(), len(token_texts))
        hit = self._memo.get(key)
        if hit is not None:
            return hit
        mask = np.zeros(len(token_texts), dtype=bool)
        step = self.automaton.step
        stack = [(_trie_for(token_texts), self.state.sid)]
        while stack:
            node, sid = stack.pop()
            for ch, child in node.children.items():
                nxt = step(sid, ch)
                if nxt < 0:
                    continue
                if child.tokens:
                    mask[child.tokens] = True
                if child.children:
                    stack.append((child, nxt))
        if len(self._memo) < 1024:
            self._memo[key] = mask
        return mask

    def advance(self, text: str) -> None:
        nxt = self.state.feed_text(text)
        if nxt is None:
            raise ValueError(f"the text {text!r} cannot continue any sentence of the grammar")
        self.state = nxt

    @property
    def complete(self) -> bool:
        return self.state.complete

    def terminal(self, token_texts) -> bool:
        return self.complete and not self.allowed(token_texts).any()

    def matches(self, text: str) -> bool:
        """Whole-string membership (does not disturb the running state)."""
        st = EarleyState(self.automaton).feed_text(text)
        return st is not None and st.complete
