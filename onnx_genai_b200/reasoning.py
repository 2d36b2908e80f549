"""Reasoning ("thinking") delimiters: detect them from a chat template, split them out of generated text.

The reference derives the delimiter pair from the model's chat template and returns the enclosed text
separately from the answer (crates/onnx-genai/src/reasoning.rs; the server's ``reasoning_content``).  The same
rules here: a template that mentions an opening tag from the known list together with its closing tag declares
that pair; generated text may start inside the block (templates that pre-fill the opening tag) or contain it.
"""
from __future__ import annotations

import re
from dataclasses import dataclass

KNOWN_PAIRS = (("<think>", "</think>"), ("<thinking>", "</thinking>"), ("<reasoning>", "</reasoning>"),
               ("<|begin_of_thought|>", "<|end_of_thought|>"), ("[THINK]", "[/THINK]"))


@dataclass(frozen=True)
class ReasoningDelimiters:
    open: str
    close: str
    prefilled: bool = False   # the template itself emits the opening tag at the end of the generation prompt


def detect(chat_template: str | None) -> ReasoningDelimiters | None:
    """The delimiter pair a chat template declares, or None."""
    if not chat_template:
        return None
    for o, c in KNOWN_PAIRS:
        if c in chat_template:
            # pre-filled when the opening tag follows the generation prompt branch of the template
            tail = chat_template[chat_template.rfind("add_generation_prompt"):] if "add_generation_prompt" in chat_template else ""
            return ReasoningDelimiters(o, c, prefilled=o in tail)
    return None


def split(text: str, delims: ReasoningDelimiters | None):
    """(reasoning, answer).  Without delimiters, or without a reasoning block in ``text``, reasoning is None.
    An unterminated block (generation stopped while thinking) is all reasoning and an empty answer."""
    if delims is None or not text:
        return None, text
    o, c = delims.open, delims.close
    start = text.find(o)
    if start < 0:
        if delims.prefilled or c in text:      # the block was opened by the prompt
            end = text.find(c)
            if end < 0:
                return (text.strip(), "") if delims.prefilled else (None, text)
            return text[:end].strip(), text[end + len(c):].lstrip("\n")
        return None, text
    end = text.find(c, start + len(o))
    if end < 0:
        return text[start + len(o):].strip(), text[:start].rstrip()
    reasoning = text[start + len(o):end].strip()
    answer = (text[:start] + text[end + len(c):]).lstrip("\n")
    return reasoning, answer


class StreamSplitter:
    """Incremental version of :func:`split` for streamed deltas: ``feed(delta)`` returns
    ``(reasoning_delta, answer_delta)``; tags split across deltas are held back until they can be decided."""

    def __init__(self, delims: ReasoningDelimiters | None):
        self.d = delims
        self.buf = ""
        self.inside = bool(delims and delims.prefilled)
        self.seen_block = self.inside

    def feed(self, delta: str):
        if self.d is None:
            return "", delta
        self.buf += delta
        r_out, a_out = "", ""
        while self.buf:
            tag = self.d.close if self.inside else self.d.open
            pos = self.buf.find(tag)
            if pos >= 0:
                chunk, self.buf = self.buf[:pos], self.buf[pos + len(tag):]
                if self.inside:
                    r_out += chunk
                else:
                    a_out += chunk
                self.inside = not self.inside
                self.seen_block = True
                continue
            # keep a possible partial tag at the end of the buffer
            keep = 0
            for n in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-n:]):
                    keep = n
                    break
            chunk, self.buf = (self.buf[:-keep], self.buf[-keep:]) if keep else (self.buf, "")
            if self.inside:
                r_out += chunk
            else:
                a_out += chunk
            break
        return r_out, a_out

    def flush(self):
        rest, self.buf = self.buf, ""
        return (rest, "") if self.inside else ("", rest)


def strip_for_history(text: str, delims: ReasoningDelimiters | None) -> str:
    """Assistant turns are stored without their reasoning block, as chat templates expect."""
    return split(text, delims)[1] if delims else text


_TAG_RE = re.compile("|".join(re.escape(t) for pair in KNOWN_PAIRS for t in pair))


def contains_reasoning_tags(text: str) -> bool:
    return bool(_TAG_RE.search(text or ""))
