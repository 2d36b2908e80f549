"""Device-independent graph -> graph rewrites for ONNX graphs run by the graph executor.

Counterpart of the reference's ``onnx-runtime-optimizer`` crate (src/lib.rs:1-60: pass contract, bounded constant
folding, dead-node elimination, pattern fusion applied to a fixpoint), written against this package's own graph objects
(:mod:`onnx_pb`).  The fused decoder path does not use it -- there the fusions are the kernels' prologues and epilogues --
but every other graph of a package (vision towers, codecs, policy graphs, unrecognised decoders) is interpreted node by
node, and each node removed is a launch and a temporary saved.

Passes (``default_passes()`` order; ``optimize`` repeats the pipeline until nothing changes):

* ``fold_constants``      evaluates nodes whose inputs are all constants with the executor's own operator table (so folding
                          can never disagree with execution), bounded by an element budget; ``Shape`` of a value whose
                          extents shape inference resolved to integers folds too;
* ``eliminate_identities``  Identity, inference-mode Dropout, Cast to the type a value already has, Transpose by the identity
                          permutation, Reshape / Expand / Squeeze / Unsqueeze / Flatten that shape inference proves to be no-ops,
                          Concat of one input;
* ``merge_transposes``    Transpose of a Transpose becomes one Transpose (or nothing);
* ``fuse_patterns``       the erf form of GELU -> ``Gelu``; the ReduceMean / Sub / Pow / ReduceMean / Add / Sqrt / Div / Mul / Add
                          chain -> ``LayerNormalization``; 2-D ``MatMul`` + bias ``Add`` (+ ``Relu``) -> ``Gemm`` / ``FusedGemm``;
* ``eliminate_dead_nodes``  nodes and initializers nothing reads.

Every rewrite keeps the graph's inputs and outputs by name; ``tests/test_graph_optimizer_cpu.py`` runs graphs before and
after on the same inputs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from . import onnx_pb as pb

FOLD_ELEMENT_BUDGET = 1 << 20
_NEVER_FOLD = {"RandomNormal", "RandomUniform", "RandomNormalLike", "RandomUniformLike", "Bernoulli", "Multinomial", "If", "Loop", "Scan",
               "Constant"}


@dataclass
class OptimizationReport:
    nodes_before: int = 0
    nodes_after: int = 0
    rounds: int = 0
    changes: dict = field(default_factory=dict)      # pass name -> rewrites applied

    def count(self, name, n):
        if n:
            self.changes[name] = self.changes.get(name, 0) + n


class _View:
    """Producer / consumer maps over a graph; rebuilt after every structural change."""

    def __init__(self, g):
        self.g = g
        self.refresh()

    def refresh(self):
        g = self.g
        self.producer = {o: n for n in g.nodes for o in n.outputs if o}
        self.consumers: dict = {}
        for n in g.nodes:
            for i in n.inputs:
                if i:
                    self.consumers.setdefault(i, []).append(n)
            for sub in _subgraphs(n):
                for name in _free_names(sub):
                    self.consumers.setdefault(name, []).append(n)
        self.outputs = {vo.name for vo in g.outputs}

    def uses(self, name) -> int:
        return len(self.consumers.get(name, ())) + (1 if name in self.outputs else 0)

    def only_consumer(self, name):
        c = self.consumers.get(name, ())
        return c[0] if len(c) == 1 and name not in self.outputs else None


def _subgraphs(n):
    return [v for v in n.attrs.values() if isinstance(v, pb.Graph)]


def _free_names(graph) -> set:
    bound = {vi.name for vi in graph.inputs} | set(graph.initializers)
    free = set()
    for n in graph.nodes:
        free |= {i for i in n.inputs if i and i not in bound}
        for sub in _subgraphs(n):
            free |= _free_names(sub) - bound
        bound |= {o for o in n.outputs if o}
    return free


def _rename_uses(g, old, new):
    for n in g.nodes:
        n.inputs = [new if i == old else i for i in n.inputs]
        for sub in _subgraphs(n):
            _rename_uses(sub, old, new)


def _bypass(g, view, node, src) -> bool:
    """Remove ``node`` (one output) by letting its readers read ``src``.  A graph output keeps its name: then the producer
    of ``src`` is renamed instead, which is only possible when nothing else reads ``src``."""
    out = node.outputs[0]
    if out in view.outputs:
        prod = view.producer.get(src)
        if prod is None or src in view.outputs or view.uses(src) != 1:
            return False
        prod.outputs = [out if o == src else o for o in prod.outputs]
    else:
        _rename_uses(g, out, src)
    g.nodes.remove(node)
    view.refresh()
    return True


def _const_array(g, name):
    t = g.initializers.get(name)
    if t is None or t.numpy() is None:
        return None
    return np.asarray(t.numpy()).reshape(tuple(int(d) for d in t.dims))


def _scalar_const(g, name):
    a = _const_array(g, name)
    if a is None or a.size != 1 or a.dtype.kind not in "fiu":
        return None
    return float(a.reshape(-1)[0])


# ---------------------------------------------------------------------------------------------------------------------
# passes: each takes (model, shapes) and returns the number of rewrites it made
# ---------------------------------------------------------------------------------------------------------------------
def fold_constants(model, shapes) -> int:
    from .graph_executor import OPS, _constant, tensor_to_torch

    g = model.graph
    done = 0
    known = {}
    for n in list(g.nodes):
        if n.op_type == "Shape" and n.inputs[0] not in g.initializers and shapes is not None:
            s = shapes.shape(n.inputs[0])
            if s is not None and all(isinstance(d, int) for d in s):
                rank = len(s)
                start = int(n.attrs.get("start", 0))
                end = n.attrs.get("end")
                start = max(0, min(rank, start + rank if start < 0 else start))
                end = rank if end is None else max(0, min(rank, int(end) + rank if int(end) < 0 else int(end)))
                arr = np.asarray(s[start:end], dtype=np.int64)
                g.initializers[n.outputs[0]] = pb.Tensor(name=n.outputs[0], dims=arr.shape, data_type=pb.INT64, array=arr)
                g.nodes.remove(n)
                done += 1
                continue
        if n.op_type in _NEVER_FOLD and n.op_type != "Constant":
            continue
        if n.op_type == "Constant":
            if "value" not in n.attrs and not any(k in n.attrs for k in ("value_int", "value_float", "value_ints", "value_floats")):
                continue
            val = _constant([], n.attrs, "cpu")
        else:
            if _subgraphs(n) or not n.inputs or any(i and i not in g.initializers for i in n.inputs):
                continue
            fn = OPS.get(f"{n.domain}::{n.op_type}") or OPS.get(n.op_type)
            if fn is None or n.op_type == "Split":
                continue
            ins = []
            for i in n.inputs:
                if not i:
                    ins.append(None)
                    continue
                if i not in known:
                    t = g.initializers[i]
                    if t.numpy() is None or t.data_type in (pb.BFLOAT16, pb.FLOAT8E4M3FN) or int(np.prod(t.dims, dtype=np.int64)) > FOLD_ELEMENT_BUDGET:
                        known[i] = None
                    else:
                        known[i] = tensor_to_torch(t, "cpu")
                if known[i] is None:
                    ins = None
                    break
                ins.append(known[i])
            if ins is None:
                continue
            try:
                val = fn(ins, n.attrs)
            except Exception:
                continue                                     # leave the node for the executor to report at run time
        vals = list(val) if isinstance(val, (list, tuple)) else [val]
        if len(vals) < len([o for o in n.outputs if o]) or any(not isinstance(v, torch.Tensor) or v.numel() > FOLD_ELEMENT_BUDGET or
                                                               v.dtype in (torch.bfloat16,) for v in vals[:len(n.outputs)]):
            continue
        for name, v in zip(n.outputs, vals):
            if not name:
                continue
            arr = v.detach().cpu().numpy()
            dt = {np.dtype(np.float32): pb.FLOAT, np.dtype(np.float64): pb.DOUBLE, np.dtype(np.float16): pb.FLOAT16, np.dtype(np.int64): pb.INT64,
                  np.dtype(np.int32): pb.INT32, np.dtype(np.int16): pb.INT16, np.dtype(np.int8): pb.INT8, np.dtype(np.uint8): pb.UINT8,
                  np.dtype(np.bool_): pb.BOOL}.get(arr.dtype)
            if dt is None:
                break
            g.initializers[name] = pb.Tensor(name=name, dims=tuple(arr.shape), data_type=dt, array=np.ascontiguousarray(arr))
        else:
            g.nodes.remove(n)
            done += 1
    return done


def eliminate_identities(model, shapes) -> int:
    g = model.graph
    view = _View(g)
    done = 0
    for n in list(g.nodes):
        if n not in g.nodes or not n.inputs or not n.inputs[0] or len([o for o in n.outputs if o]) != 1:
            continue
        src, op = n.inputs[0], n.op_type
        noop = False
        if op == "Identity" or (op == "Dropout" and view.uses(n.outputs[1] if len(n.outputs) > 1 else "") == 0) or \
                (op == "Concat" and len(n.inputs) == 1):
            noop = True
        elif op == "Cast" and shapes is not None and shapes.dtype(src) is not None:
            noop = shapes.dtype(src) == int(n.attrs["to"])
        elif op == "Transpose" and "perm" in n.attrs:
            noop = list(n.attrs["perm"]) == list(range(len(n.attrs["perm"])))
        elif op in ("Reshape", "Expand", "Squeeze", "Unsqueeze", "Flatten") and shapes is not None:
            a, b = shapes.shape(src), shapes.shape(n.outputs[0])
            noop = a is not None and b is not None and a == b and all(d is not None for d in a)
        if noop and _bypass(g, view, n, src):
            done += 1
    return done


def merge_transposes(model, shapes) -> int:
    g = model.graph
    view = _View(g)
    done = 0
    for n in list(g.nodes):
        if n not in g.nodes or n.op_type != "Transpose" or "perm" not in n.attrs:
            continue
        inner = view.producer.get(n.inputs[0])
        if inner is None or inner.op_type != "Transpose" or "perm" not in inner.attrs or view.only_consumer(inner.outputs[0]) is not n:
            continue
        p1, p2 = list(inner.attrs["perm"]), list(n.attrs["perm"])
        if len(p1) != len(p2):
            continue
        n.attrs["perm"] = [p1[i] for i in p2]
        n.inputs = [inner.inputs[0]]
        g.nodes.remove(inner)
        view.refresh()
        done += 1
    return done


def _match_gelu(g, view, div):
    """x / sqrt(2) -> Erf -> + 1 -> * x -> * 0.5 (the multiplications in either order)."""
    c = _scalar_const(g, div.inputs[1]) if len(div.inputs) > 1 else None
    if c is None or abs(c - math.sqrt(2.0)) > 1e-3:
        return None
    x = div.inputs[0]
    erf = view.only_consumer(div.outputs[0])
    if erf is None or erf.op_type != "Erf":
        return None
    add = view.only_consumer(erf.outputs[0])
    if add is None or add.op_type != "Add":
        return None
    one = [i for i in add.inputs if i != erf.outputs[0]]
    if len(one) != 1 or _scalar_const(g, one[0]) != 1.0:
        return None
    m1 = view.only_consumer(add.outputs[0])
    if m1 is None or m1.op_type != "Mul":
        return None
    other = [i for i in m1.inputs if i != add.outputs[0]]
    if len(other) != 1:
        return None
    m2 = view.only_consumer(m1.outputs[0])
    if m2 is None or m2.op_type != "Mul":
        return None
    rest = [i for i in m2.inputs if i != m1.outputs[0]]
    if len(rest) != 1:
        return None
    half_first = _scalar_const(g, other[0]) == 0.5 and rest[0] == x
    x_first = other[0] == x and _scalar_const(g, rest[0]) == 0.5
    if not (half_first or x_first):
        return None
    return x, [div, erf, add, m1, m2]


def _match_layer_norm(g, view, mean):
    """ReduceMean(x, -1) -> Sub(x, mean) -> Pow(., 2) -> ReduceMean -> Add eps -> Sqrt -> Div(sub, .) -> Mul gamma -> Add beta."""
    def last_axis(n):
        axes = n.attrs.get("axes")
        if axes is None and len(n.inputs) > 1:
            a = _const_array(g, n.inputs[1])
            axes = None if a is None else [int(v) for v in a.reshape(-1)]
        return axes is not None and list(axes) == [-1] and int(n.attrs.get("keepdims", 1)) == 1

    if not last_axis(mean):
        return None
    x = mean.inputs[0]
    subs = [c for c in view.consumers.get(mean.outputs[0], ()) if c.op_type == "Sub" and c.inputs[0] == x]
    if len(subs) != 1 or view.uses(mean.outputs[0]) != 1:
        return None
    sub = subs[0]
    cons = view.consumers.get(sub.outputs[0], ())
    if len(cons) != 2 or sub.outputs[0] in view.outputs:
        return None
    pw = next((c for c in cons if c.op_type == "Pow"), None)
    div = next((c for c in cons if c.op_type == "Div" and c.inputs[0] == sub.outputs[0]), None)
    if pw is None or div is None or _scalar_const(g, pw.inputs[1]) != 2.0:
        return None
    var = view.only_consumer(pw.outputs[0])
    if var is None or var.op_type != "ReduceMean" or not last_axis(var):
        return None
    add = view.only_consumer(var.outputs[0])
    if add is None or add.op_type != "Add":
        return None
    eps_name = [i for i in add.inputs if i != var.outputs[0]]
    eps = _scalar_const(g, eps_name[0]) if len(eps_name) == 1 else None
    if eps is None:
        return None
    sq = view.only_consumer(add.outputs[0])
    if sq is None or sq.op_type != "Sqrt" or view.only_consumer(sq.outputs[0]) is not div or div.inputs[1] != sq.outputs[0]:
        return None
    mul = view.only_consumer(div.outputs[0])
    if mul is None or mul.op_type != "Mul":
        return None
    gamma = [i for i in mul.inputs if i != div.outputs[0]]
    if len(gamma) != 1 or gamma[0] not in g.initializers or len(g.initializers[gamma[0]].dims) != 1:
        return None
    nodes = [mean, sub, pw, var, add, sq, div, mul]
    out, beta = mul.outputs[0], None
    badd = view.only_consumer(mul.outputs[0])
    if badd is not None and badd.op_type == "Add":
        b = [i for i in badd.inputs if i != mul.outputs[0]]
        if len(b) == 1 and b[0] in g.initializers and tuple(g.initializers[b[0]].dims) == tuple(g.initializers[gamma[0]].dims):
            beta, out = b[0], badd.outputs[0]
            nodes.append(badd)
    return x, gamma[0], beta, eps, out, nodes


def fuse_patterns(model, shapes) -> int:
    g = model.graph
    done = 0
    changed = True
    while changed:
        changed = False
        view = _View(g)
        for n in list(g.nodes):
            if n.op_type == "Div":
                m = _match_gelu(g, view, n)
                if m:
                    x, nodes = m
                    pos = g.nodes.index(nodes[0])
                    for d in nodes:
                        g.nodes.remove(d)
                    g.nodes.insert(pos, pb.Node("Gelu", [x], [nodes[-1].outputs[0]], name=(nodes[-1].name or "gelu") + "_fused"))
                    done, changed = done + 1, True
                    break
            if n.op_type == "ReduceMean":
                m = _match_layer_norm(g, view, n)
                if m:
                    x, gamma, beta, eps, out, nodes = m
                    pos = g.nodes.index(nodes[0])
                    for d in nodes:
                        g.nodes.remove(d)
                    g.nodes.insert(pos, pb.Node("LayerNormalization", [x, gamma] + ([beta] if beta else []), [out],
                                                name=(nodes[-1].name or "layer_norm") + "_fused", attrs={"axis": -1, "epsilon": float(eps)}))
                    done, changed = done + 1, True
                    break
            if n.op_type == "MatMul" and shapes is not None:
                a, b = shapes.shape(n.inputs[0]), shapes.shape(n.inputs[1])
                add = view.only_consumer(n.outputs[0])
                if a is None or b is None or len(a) != 2 or len(b) != 2 or add is None or add.op_type != "Add":
                    continue
                bias = [i for i in add.inputs if i != n.outputs[0]]
                if len(bias) != 1 or bias[0] not in g.initializers or len(g.initializers[bias[0]].dims) != 1 or \
                        shapes.dtype(n.inputs[0]) not in (pb.FLOAT, pb.FLOAT16, pb.DOUBLE):
                    continue
                relu = view.only_consumer(add.outputs[0])
                pos = g.nodes.index(n)
                if relu is not None and relu.op_type == "Relu":
                    fused = pb.Node("FusedGemm", [n.inputs[0], n.inputs[1], bias[0]], [relu.outputs[0]], domain="com.microsoft",
                                    name=(n.name or "matmul") + "_bias_relu", attrs={"activation": "Relu"})
                    g.nodes.remove(relu)
                else:
                    fused = pb.Node("Gemm", [n.inputs[0], n.inputs[1], bias[0]], [add.outputs[0]], name=(n.name or "matmul") + "_bias")
                g.nodes.remove(add)
                g.nodes.remove(n)
                g.nodes.insert(pos, fused)
                done, changed = done + 1, True
                break
    return done


def eliminate_dead_nodes(model, shapes) -> int:
    g = model.graph
    done = 0
    while True:
        view = _View(g)
        dead = [n for n in g.nodes if all(view.uses(o) == 0 for o in n.outputs if o)]
        if not dead:
            break
        for n in dead:
            g.nodes.remove(n)
        done += len(dead)
    view = _View(g)
    inputs = {vi.name for vi in g.inputs}
    for name in [k for k in g.initializers if view.uses(k) == 0 and k not in inputs]:
        del g.initializers[name]
        done += 1
    return done


def default_passes():
    return [("fold_constants", fold_constants), ("eliminate_identities", eliminate_identities), ("merge_transposes", merge_transposes),
            ("fuse_patterns", fuse_patterns), ("eliminate_dead_nodes", eliminate_dead_nodes)]


def optimize(model, passes=None, max_rounds: int = 6, input_shapes: dict | None = None) -> OptimizationReport:
    """Rewrite ``model.graph`` in place; returns what was done.  Shape inference runs before every round (the identity and
    fusion passes only act on what it proves)."""
    from . import shape_inference as si

    passes = passes or default_passes()
    rep = OptimizationReport(nodes_before=len(model.graph.nodes))
    for _ in range(max_rounds):
        try:
            shapes = si.infer(model, input_shapes=input_shapes)
        except si.ShapeInferenceError:
            shapes = None
        total = 0
        for name, fn in passes:
            n = fn(model, shapes)
            rep.count(name, n)
            total += n
        rep.rounds += 1
        if total == 0:
            break
    rep.nodes_after = len(model.graph.nodes)
    return rep
