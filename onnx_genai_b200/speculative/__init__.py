"""Speculative decoding: proposers behind one seam, verification inside the scheduler core.

`SpeculativeProposer` mirrors the reference's trait (crates/onnx-genai-engine/src/speculative/
mod.rs:929-945).  Proposers shipped here: prompt-lookup n-grams (`NgramProposer`, the reference's
NgramProposer / prompt_lookup) and a draft model (`DraftModelProposer`).  Verification follows
the reference's greedy rule -- keep the longest draft prefix the target's own choices confirm,
then append the target's correction / bonus token (speculative/mod.rs:1608-1835) -- but it is
not a separate loop: the scheduler core feeds `last token + drafts` as one short chunk of the
regular batched step, samples every fed position on the device and rewinds the KV pages of the
rejected tail (csrc/runtime/core.cpp, commit_step).  `SpeculativeStats` carries the same four
counters as speculative/mod.rs:896-902.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class SpeculativeStats:
    verification_steps: int = 0
    proposed_tokens: int = 0
    accepted_tokens: int = 0

    @property
    def accepted_per_step(self) -> float:
        return self.accepted_tokens / self.verification_steps if self.verification_steps else 0.0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted_tokens / self.proposed_tokens if self.proposed_tokens else 0.0


class SpeculativeProposer:
    """``propose(token_ids, k) -> up to k draft token ids`` continuing ``token_ids``."""

    name = "proposer"

    def propose(self, token_ids, k: int):
        raise NotImplementedError

    def notify(self, accepted: int, proposed: int) -> None:
        """Called after verification; adaptive proposers may resize their next draft."""


class NgramProposer(SpeculativeProposer):
    """Prompt lookup: find the most recent earlier occurrence of the trailing n-gram and propose what followed."""

    name = "ngram"

    def __init__(self, max_ngram: int = 4, min_ngram: int = 1):
        self.max_ngram, self.min_ngram = max_ngram, min_ngram

    def propose(self, token_ids, k):
        ids = np.asarray(token_ids)
        n = len(ids)
        for g in range(min(self.max_ngram, n - 1), self.min_ngram - 1, -1):
            tail = ids[n - g:]
            # windows ending before the tail itself
            for start in range(n - g - 1, -1, -1):
                if np.array_equal(ids[start:start + g], tail):
                    follow = ids[start + g:start + g + k]
                    if len(follow):
                        return follow.astype(np.int32)
        return np.zeros(0, dtype=np.int32)


class DraftModelProposer(SpeculativeProposer):
    """Greedy continuation from a smaller engine.  The draft engine keeps one live sequence per target
    sequence and is rewound to the verified prefix before each proposal, so its KV pages are reused."""

    name = "draft_model"

    def __init__(self, draft_engine):
        self.eng = draft_engine
        self.sid = None
        self.synced = []

    @property
    def batch_key(self):
        """Proposers that share a draft engine are asked together (see :meth:`propose_many`)."""
        return ("draft_model", id(self.eng))

    def _align(self, ids):
        """Make the draft's sequence equal to ``ids``: keep the common prefix (and its KV pages), drop what the
        target rejected, feed what the target chose instead."""
        eng = self.eng
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        if self.sid is None:
            self.sid = eng.add_request(ids, max_new_tokens=1 << 20, temperature=0.0, ignore_eos=True)
            return
        have = np.asarray(eng.core.seq_tokens(self.sid), dtype=np.int32)
        n = min(len(have), len(ids))
        diff = np.flatnonzero(have[:n] != ids[:n])          # contexts run to tens of thousands of tokens: no Python loop
        common = int(diff[0]) if len(diff) else n
        ok = common >= 1
        if ok and common < len(have):
            ok = eng.core.rewind(self.sid, common)
        if ok and common < len(ids):
            ok = eng.core.append_tokens(self.sid, ids[common:])
        if not ok:
            eng.core.release(self.sid)
            self.sid = eng.add_request(ids, max_new_tokens=1 << 20, temperature=0.0, ignore_eos=True)

    def propose(self, token_ids, k):
        return self.propose_many([self], [token_ids], k)[0]

    @staticmethod
    def propose_many(proposers, token_lists, k):
        """Drafts for several target sequences from one draft engine: every draft sequence is re-aligned first,
        then the engine is stepped until each has k new tokens, so the draft model runs batched steps instead of
        k steps per target sequence."""
        eng = proposers[0].eng
        for p, toks in zip(proposers, token_lists):
            p._align(toks)
        out = {p.sid: [] for p in proposers}
        guard = 0
        while any(len(v) < k for v in out.values()) and guard < k + 64 and eng.has_work:
            guard += 1
            for sid, tok, fin in eng.step().events:
                if sid in out:
                    out[sid].append(tok)
        return [np.asarray(out[p.sid][:k], dtype=np.int32) for p in proposers]

    def close(self):
        if self.sid is not None:
            self.eng.core.release(self.sid)
            self.sid = None
