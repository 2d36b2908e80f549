"""A small explicit-state model checker for the concurrency protocols of this runtime.

A model is an initial state (any hashable value) and a function from a state to its enabled transitions, each a
``(label, next_state)`` pair.  :func:`explore` visits every reachable state breadth-first, so a reported trace is a
shortest one, and checks three things: every invariant holds in every state, no state without transitions fails the
``done`` predicate (a deadlock), and the state count stays under a bound.  It plays the role the TLC runs over
``specs/tla/*.tla`` play for the reference (bounded safety models of its memory and collective protocols, each with an
"unguarded" configuration that must fail); the models live in ``onnx_genai_b200/specs`` and run as tests.
"""
from __future__ import annotations

import dataclasses
from collections import deque
from typing import Callable, Hashable, Iterable


@dataclasses.dataclass
class Result:
    ok: bool
    states: int
    kind: str = ""                 # "", "invariant", "deadlock", "bound"
    detail: str = ""
    trace: tuple = ()              # labels from the initial state to the offending one

    def __str__(self):
        if self.ok:
            return f"ok: {self.states} states"
        return f"{self.kind}: {self.detail} after {' -> '.join(self.trace) or '(initial state)'} ({self.states} states seen)"


def explore(init: Hashable, step: Callable[[Hashable], Iterable], invariants: dict, done: Callable[[Hashable], bool],
            max_states: int = 2_000_000) -> Result:
    """Exhaustive breadth-first search.  ``invariants`` maps a name to a predicate over states."""
    parent = {init: None}
    queue = deque([init])

    def trace_of(s):
        out = []
        while parent[s] is not None:
            s, label = parent[s]
            out.append(label)
        return tuple(reversed(out))

    while queue:
        s = queue.popleft()
        for name, pred in invariants.items():
            if not pred(s):
                return Result(False, len(parent), "invariant", name, trace_of(s))
        succ = list(step(s))
        if not succ and not done(s):
            return Result(False, len(parent), "deadlock", "no transition is enabled and the run is not complete", trace_of(s))
        for label, t in succ:
            if t not in parent:
                if len(parent) >= max_states:
                    return Result(False, len(parent), "bound", f"more than {max_states} states", trace_of(s))
                parent[t] = (s, label)
                queue.append(t)
    return Result(True, len(parent))
