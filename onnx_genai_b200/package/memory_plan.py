"""Static memory plan of an interpreted graph: value lifetimes, an arena layout, and the peak it needs.

For a graph whose shapes are known (shape inference with concrete inputs, or symbolic shapes plus a binding of the
symbols) every intermediate value has a size and a lifetime: it is born at the node that writes it and dies after the
last node that reads it.  From those the planner derives

* the *lower bound* -- the largest sum of sizes alive at one moment, which no layout can beat,
* an *arena layout* -- one offset per value such that values alive together never overlap, found greedily by size
  (largest first, lowest gap that fits), which lands within a few percent of the bound on transformer graphs,
* the *naive* figure -- every intermediate held to the end, which is what an interpreter that never releases costs.

Views (Reshape, Squeeze, Unsqueeze, Flatten, Identity) share their input's storage: they take no space of their own and
extend the lifetime of the value they alias.  Control-flow bodies count as readers of the outer values they capture.
Graph inputs and initializers are the caller's memory and are not planned; graph outputs live to the end.

``GraphExecutor(model, release=True)`` uses the same lifetimes at run time: an intermediate is dropped from the
interpreter's scope right after its last reader, so the live set of a run is the plan's live set.

Role of the reference's activation memory planner (crates/onnx-runtime-memory/src/lib.rs:3-100 with liveness.rs,
view_map.rs and plan.rs: liveness intervals, view lifetimes folded into the owning value, buffer sharing among values
whose lifetimes do not overlap); the fused decoder path does not need it -- its activation arena is bound once, by hand,
in models/decoder.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from . import onnx_pb
from . import shape_inference as si

VIEW_OPS = {"Reshape", "Squeeze", "Unsqueeze", "Flatten", "Identity"}


class MemoryPlanError(ValueError):
    pass


@dataclass
class Lifetime:
    name: str
    born: int                  # index of the producing node in execution order
    dies: int                  # index of the last reading node (len(order) for graph outputs)
    bytes: int
    offset: int = -1           # in the arena; -1 for views
    alias_of: str | None = None


@dataclass
class MemoryPlan:
    order: list                                    # node names / first outputs, in execution order
    values: dict = field(default_factory=dict)     # name -> Lifetime
    arena_bytes: int = 0
    lower_bound_bytes: int = 0
    naive_bytes: int = 0
    peak_step: int = 0                             # execution index at which the live set is largest
    unsized: list = field(default_factory=list)    # values whose size could not be determined (left out of the plan)
    last_use: dict = field(default_factory=dict)   # name -> execution index after which the value may be dropped

    @property
    def efficiency(self) -> float:
        """Lower bound over arena size: 1.0 means the layout wastes nothing."""
        return self.lower_bound_bytes / self.arena_bytes if self.arena_bytes else 1.0

    def check(self) -> None:
        """No two values alive at the same time overlap in the arena."""
        vals = [v for v in self.values.values() if v.alias_of is None and v.bytes > 0]
        for i, a in enumerate(vals):
            for b in vals[i + 1:]:
                if a.born <= b.dies and b.born <= a.dies and a.offset < b.offset + b.bytes and b.offset < a.offset + a.bytes:
                    raise MemoryPlanError(f"{a.name} and {b.name} are alive together and overlap in the arena")

    def summary(self) -> dict:
        return {"values": len(self.values), "arena_bytes": self.arena_bytes, "lower_bound_bytes": self.lower_bound_bytes,
                "naive_bytes": self.naive_bytes, "efficiency": round(self.efficiency, 4), "peak_at": self.order[self.peak_step] if self.order else None,
                "unsized": len(self.unsized)}


def _eval_dim(d, symbols: dict):
    if d is None:
        return None
    total = 0
    for mono, coeff in d.terms.items():
        term = coeff
        for s in mono:
            if s not in symbols:
                return None
            term *= int(symbols[s])
        total += term
    return total


def _value_bytes(tt, symbols: dict):
    if tt is None or tt.dtype is None or tt.shape is None:
        return None
    n = 1
    for d in tt.shape:
        v = _eval_dim(d, symbols)
        if v is None or v < 0:
            return None
        n *= v
    item = onnx_pb._ITEM.get(tt.dtype)
    return None if item is None else n * item


def _subgraphs(node):
    for v in node.attrs.values():
        if isinstance(v, onnx_pb.Graph):
            yield v
        elif isinstance(v, (list, tuple)):
            for x in v:
                if isinstance(x, onnx_pb.Graph):
                    yield x


def _captured(graph) -> set:
    """Names a body reads from enclosing scopes."""
    defined = set(graph.initializers) | {vi.name for vi in graph.inputs}
    free = set()
    for n in graph.nodes:
        for x in n.inputs:
            if x and x not in defined:
                free.add(x)
        for sub in _subgraphs(n):
            free |= {x for x in _captured(sub) if x not in defined}
        defined.update(o for o in n.outputs if o)
    return free


def lifetimes(model, order=None):
    """``(order, born, last_use)`` of the main graph: execution order (default: shape inference's topological order), the
    index at which each intermediate is written, and the index of its last reader (graph outputs: ``len(order)``)."""
    g = model.graph
    order = list(order) if order is not None else si._toposort(g)
    born, last = {}, {}
    for i, n in enumerate(order):
        reads = [x for x in n.inputs if x]
        for sub in _subgraphs(n):
            reads += list(_captured(sub))
        for x in reads:
            last[x] = i
        for o in n.outputs:
            if o:
                born[o] = i
                last.setdefault(o, i)
    for vi in g.outputs:
        if vi.name in born:
            last[vi.name] = len(order)
    return order, born, last


def plan_memory(model, input_shapes: dict | None = None, symbols: dict | None = None, alignment: int = 256, order=None) -> MemoryPlan:
    """Plan the intermediates of ``model.graph``.  ``input_shapes`` as for :func:`shape_inference.infer`; ``symbols`` binds
    the symbolic extents that remain (``{"batch": 4, "seq": 128}``).  Values that stay unsized are listed in
    ``plan.unsized`` and left out."""
    symbols = symbols or {}
    report = si.infer(model, input_shapes)
    order, born, last = lifetimes(model, order)
    by_output = {o: n for n in order for o in n.outputs if o}
    plan = MemoryPlan(order=[n.name or (n.outputs[0] if n.outputs else n.op_type) for n in order])

    def root_of(name):
        seen = set()
        while name in by_output and by_output[name].op_type in VIEW_OPS and by_output[name].inputs and name not in seen:
            seen.add(name)
            name = by_output[name].inputs[0]
        return name

    for name, b in born.items():
        size = _value_bytes(report.types.get(name), symbols)
        root = root_of(name)
        if root != name:                       # a view: no storage, but it keeps its root alive
            plan.values[name] = Lifetime(name, b, last[name], 0, alias_of=root)
            continue
        if size is None:
            plan.unsized.append(name)
            continue
        plan.values[name] = Lifetime(name, b, last[name], (size + alignment - 1) // alignment * alignment)
    for v in plan.values.values():             # extend roots by their views' lifetimes
        if v.alias_of is not None and v.alias_of in plan.values:
            r = plan.values[v.alias_of]
            r.dies = max(r.dies, v.dies)
    plan.last_use = {}
    for name in born:
        v = plan.values.get(name)
        plan.last_use[name] = last[name] if v is None else v.dies
    for v in plan.values.values():             # a value read through a view may only be dropped when the view is done
        if v.alias_of is not None:
            plan.last_use[v.alias_of] = max(plan.last_use.get(v.alias_of, 0), v.dies)

    real = [v for v in plan.values.values() if v.alias_of is None and v.bytes > 0]
    plan.naive_bytes = sum(v.bytes for v in real)
    # lower bound: sweep the execution order
    delta = [0] * (len(order) + 2)
    for v in real:
        delta[v.born] += v.bytes
        delta[min(v.dies, len(order)) + 1] -= v.bytes
    live = 0
    for i, dlt in enumerate(delta):
        live += dlt
        if live > plan.lower_bound_bytes:
            plan.lower_bound_bytes, plan.peak_step = live, min(i, max(0, len(order) - 1))
    # greedy by size: largest first, lowest offset whose gap fits among the already placed values that overlap in time
    placed: list = []
    for v in sorted(real, key=lambda x: (-x.bytes, x.born)):
        busy = sorted((p.offset, p.offset + p.bytes) for p in placed if p.born <= v.dies and v.born <= p.dies)
        at = 0
        for a, b in busy:
            if a - at >= v.bytes:
                break
            at = max(at, b)
        v.offset = at
        placed.append(v)
        plan.arena_bytes = max(plan.arena_bytes, at + v.bytes)
    return plan
