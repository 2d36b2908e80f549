"""Symbolic shape inference over ONNX graphs, without running them.

Counterpart of the reference's ``onnx-runtime-shape-inference`` crate (src/lib.rs:1-60, dim_expr.rs, shape_data.rs,
registry.rs, report.rs), built around the same four ideas and nothing of its code:

* a registry of per-operator rules keyed by ``domain::op`` (an unregistered operator leaves its outputs unresolved
  instead of failing);
* dimension arithmetic on :class:`Dim`, an integer polynomial in named symbols (``batch * 4``, ``past + seq``,
  exact division, the ``-1`` of a Reshape cancelled against the input's element count);
* shape-data propagation: the element values of small integer tensors are carried through
  ``Shape -> Slice / Gather -> Concat / Unsqueeze -> Reshape / Expand`` chains, which is what lets transformer graphs
  resolve with symbolic batch and sequence lengths;
* merge policies: ``permissive`` prefers the more specific of two dimensions and goes on, ``strict`` makes a
  disagreement between two concrete dimensions an error.

``infer(model)`` returns an :class:`InferenceReport`: the element type and shape of every value it could resolve, the
names it could not, and the number of fresh symbols it had to mint (data-dependent extents such as ``NonZero``).
The graph executor is dynamic and does not need this pass; the ``validate`` command, the decoder recogniser's error
messages and memory planning for static graphs do.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import onnx_pb as pb


class ShapeInferenceError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------------------------------
# dimension arithmetic
# ---------------------------------------------------------------------------------------------------------------------
class Dim:
    """Integer polynomial over named symbols: ``{monomial: coefficient}`` with a monomial a sorted tuple of names."""

    __slots__ = ("terms",)

    def __init__(self, terms=None):
        self.terms = {m: c for m, c in (terms or {}).items() if c != 0}

    @staticmethod
    def of(v) -> "Dim":
        if isinstance(v, Dim):
            return v
        if isinstance(v, (int, np.integer)):
            return Dim({(): int(v)})
        if isinstance(v, str):
            return Dim({(v,): 1})
        raise TypeError(f"not a dimension: {v!r}")

    @property
    def is_const(self) -> bool:
        return all(m == () for m in self.terms)

    def const(self) -> int:
        return self.terms.get((), 0)

    def __add__(self, o):
        o = Dim.of(o)
        t = dict(self.terms)
        for m, c in o.terms.items():
            t[m] = t.get(m, 0) + c
        return Dim(t)

    __radd__ = __add__

    def __neg__(self):
        return Dim({m: -c for m, c in self.terms.items()})

    def __sub__(self, o):
        return self + (-Dim.of(o))

    def __rsub__(self, o):
        return Dim.of(o) - self

    def __mul__(self, o):
        o = Dim.of(o)
        t: dict = {}
        for m1, c1 in self.terms.items():
            for m2, c2 in o.terms.items():
                m = tuple(sorted(m1 + m2))
                t[m] = t.get(m, 0) + c1 * c2
        return Dim(t)

    __rmul__ = __mul__

    def exact_div(self, o):
        """``self / o`` when it is exact (an integer divisor of every coefficient, or a single monomial contained in every
        term); ``None`` otherwise."""
        o = Dim.of(o)
        if len(o.terms) != 1:
            return self if (self - o).terms == {} and False else (Dim.of(1) if self == o else None)
        (dm, dc), = o.terms.items()
        out = {}
        for m, c in self.terms.items():
            if c % dc:
                return None
            rest = list(m)
            for s in dm:
                if s not in rest:
                    return None
                rest.remove(s)
            out[tuple(rest)] = c // dc
        return Dim(out)

    def __eq__(self, o):
        try:
            return self.terms == Dim.of(o).terms
        except TypeError:
            return NotImplemented

    def __hash__(self):
        return hash(tuple(sorted(self.terms.items())))

    def lower(self):
        """int for a constant, the name for a bare symbol, otherwise a canonical expression string."""
        if self.is_const:
            return self.const()
        if len(self.terms) == 1:
            (m, c), = self.terms.items()
            if c == 1 and len(m) == 1:
                return m[0]
        parts = []
        for m, c in sorted(self.terms.items(), key=lambda kv: (len(kv[0]), kv[0])):
            body = "*".join(m)
            parts.append(str(c) if not m else (body if c == 1 else f"{c}*{body}"))
        return " + ".join(parts).replace("+ -", "- ")

    def __repr__(self):
        return f"Dim({self.lower()!r})"


def _d(v):
    return None if v is None else Dim.of(v)


@dataclass
class TensorType:
    dtype: int | None = None
    shape: list | None = None          # list of Dim | None (unknown extent); None = unknown rank

    @property
    def resolved(self) -> bool:
        return self.dtype is not None and self.shape is not None and all(d is not None for d in self.shape)

    def lowered(self):
        return None if self.shape is None else [None if d is None else d.lower() for d in self.shape]


@dataclass
class InferenceReport:
    types: dict = field(default_factory=dict)        # value name -> TensorType
    unresolved: list = field(default_factory=list)
    unregistered: dict = field(default_factory=dict)  # "domain::op" -> node count
    fresh_symbols: int = 0

    @property
    def fully_resolved(self) -> bool:
        return not self.unresolved

    def shape(self, name):
        t = self.types.get(name)
        return None if t is None else t.lowered()

    def dtype(self, name):
        t = self.types.get(name)
        return None if t is None else t.dtype


# ---------------------------------------------------------------------------------------------------------------------
# context and registry
# ---------------------------------------------------------------------------------------------------------------------
RULES: dict = {}


def rule(*names):
    def deco(fn):
        for n in names:
            RULES[n] = fn
        return fn
    return deco


class _Ctx:
    def __init__(self, policy):
        self.types: dict = {}
        self.data: dict = {}          # value name -> list of Dim | None (elements of a small integer tensor), or Dim for a scalar
        self.consts: dict = {}        # value name -> numpy array (initializers and Constant nodes)
        self.policy = policy
        self.fresh = 0

    def fresh_symbol(self, hint="n"):
        self.fresh += 1
        return Dim.of(f"_{hint}{self.fresh}")

    def type(self, name):
        return self.types.get(name) if name else None

    def shape(self, name):
        t = self.type(name)
        return None if t is None or t.shape is None else list(t.shape)

    def dtype(self, name):
        t = self.type(name)
        return None if t is None else t.dtype

    def values(self, name):
        """Elements of a small integer tensor as a list of Dim (None for unknown elements), or None when not tracked."""
        if not name:
            return None
        if name in self.data:
            v = self.data[name]
            return list(v) if isinstance(v, list) else [v]
        c = self.consts.get(name)
        if c is not None and c.size <= 64 and (np.issubdtype(c.dtype, np.integer) or c.dtype == np.bool_):
            return [Dim.of(int(x)) for x in c.reshape(-1)]
        return None

    def ints(self, name):
        v = self.values(name)
        if v is None or any(x is None or not x.is_const for x in v):
            return None
        return [x.const() for x in v]

    def merge(self, a, b, where=""):
        if a is None:
            return b
        if b is None:
            return a
        if a == b:
            return a
        if a.is_const and b.is_const:
            if self.policy == "strict":
                raise ShapeInferenceError(f"{where}: dimension {a.const()} disagrees with {b.const()}")
            return a
        return a if a.is_const else (b if b.is_const else a)


def _broadcast(ctx, shapes, where):
    shapes = [s for s in shapes]
    if any(s is None for s in shapes):
        return None
    rank = max(len(s) for s in shapes)
    out = []
    for i in range(rank):
        dim = Dim.of(1)
        unknown = False
        for s in shapes:
            j = i - (rank - len(s))
            if j < 0:
                continue
            d = s[j]
            if d is None:
                unknown = True
                continue
            if d == 1:
                continue
            if dim == 1:
                dim = d
            elif dim != d:
                if dim.is_const and d.is_const and ctx.policy == "strict":
                    raise ShapeInferenceError(f"{where}: cannot broadcast {dim.const()} with {d.const()}")
                dim = dim if dim.is_const else d
        out.append(None if (unknown and dim == 1) else dim)
    return out


def _norm_axis(a, rank):
    return a + rank if a < 0 else a


def _prod(dims):
    p = Dim.of(1)
    for d in dims:
        if d is None:
            return None
        p = p * d
    return p


# ---------------------------------------------------------------------------------------------------------------------
# rules.  A rule gets (ctx, node) and returns a list of TensorType (one per output) or None to leave them unresolved;
# it may record shape data with ctx.data[output] = [...].
# ---------------------------------------------------------------------------------------------------------------------
_UNARY = ("Abs Neg Exp Log Sqrt Reciprocal Relu Sigmoid Tanh Erf Floor Ceil Round Sign Sin Cos Tan Asin Acos Atan Sinh Cosh "
          "Asinh Acosh Atanh Softplus Softsign Elu Selu Celu LeakyRelu ThresholdedRelu HardSigmoid HardSwish Mish Gelu "
          "Identity Dropout Clip Softmax LogSoftmax Hardmax Not BitwiseNot Swish Silu QuickGelu FastGelu BiasGelu Trilu CumSum "
          "LRN MeanVarianceNormalization InstanceNormalization LpNormalization Shrink IsNaN IsInf").split()


@rule(*_UNARY, "com.microsoft::Gelu", "com.microsoft::FastGelu", "com.microsoft::QuickGelu", "com.microsoft::BiasGelu")
def _same(ctx, n):
    t = ctx.type(n.inputs[0])
    if t is None:
        return None
    dt = pb.BOOL if n.op_type in ("Not", "IsNaN", "IsInf") else t.dtype
    if n.op_type == "Identity" and ctx.values(n.inputs[0]) is not None:
        ctx.data[n.outputs[0]] = ctx.values(n.inputs[0])
    outs = [TensorType(dt, t.shape)]
    if n.op_type == "Dropout" and len(n.outputs) > 1:
        outs.append(TensorType(pb.BOOL, t.shape))
    return outs


_BINARY = "Add Sub Mul Div Pow Mod Min Max Mean Sum And Or Xor BitwiseAnd BitwiseOr BitwiseXor BitShift PRelu".split()
_COMPARE = "Equal Less Greater LessOrEqual GreaterOrEqual".split()


@rule(*_BINARY, *_COMPARE)
def _binary(ctx, n):
    shapes = [ctx.shape(x) for x in n.inputs if x]
    out = _broadcast(ctx, shapes, n.op_type)
    dt = pb.BOOL if n.op_type in _COMPARE else ctx.dtype(n.inputs[0])
    if n.op_type in ("Add", "Sub", "Mul", "Div") and len(n.inputs) == 2:
        a, b = ctx.values(n.inputs[0]), ctx.values(n.inputs[1])
        if a is not None and b is not None and (len(a) == len(b) or len(a) == 1 or len(b) == 1):
            m = max(len(a), len(b))
            a, b = a * (m // len(a)), b * (m // len(b))
            vals = []
            for x, y in zip(a, b):
                if x is None or y is None:
                    vals.append(None)
                elif n.op_type == "Add":
                    vals.append(x + y)
                elif n.op_type == "Sub":
                    vals.append(x - y)
                elif n.op_type == "Mul":
                    vals.append(x * y)
                else:
                    q = x.exact_div(y)
                    if q is None and x.is_const and y.is_const and y.const() != 0:
                        q = Dim.of(int(x.const() / y.const()))          # ONNX integer division truncates toward zero
                    vals.append(q)
            ctx.data[n.outputs[0]] = vals
    return [TensorType(dt, out)]


@rule("Where")
def _where(ctx, n):
    return [TensorType(ctx.dtype(n.inputs[1]), _broadcast(ctx, [ctx.shape(x) for x in n.inputs], "Where"))]


@rule("Cast", "CastLike")
def _cast(ctx, n):
    t = ctx.type(n.inputs[0])
    if t is None:
        return None
    to = int(n.attrs["to"]) if n.op_type == "Cast" else ctx.dtype(n.inputs[1])
    if ctx.values(n.inputs[0]) is not None and to in (pb.INT64, pb.INT32):
        ctx.data[n.outputs[0]] = ctx.values(n.inputs[0])
    return [TensorType(to, t.shape)]


@rule("Constant")
def _constant(ctx, n):
    a = n.attrs
    if "value" in a:
        t = a["value"]
        arr = t.numpy()
        if arr is not None:
            ctx.consts[n.outputs[0]] = np.asarray(arr).reshape(tuple(t.dims))
        return [TensorType(t.data_type, [Dim.of(d) for d in t.dims])]
    for key, dt, scalar in (("value_int", pb.INT64, True), ("value_float", pb.FLOAT, True), ("value_ints", pb.INT64, False),
                            ("value_floats", pb.FLOAT, False)):
        if key in a:
            arr = np.asarray(a[key], dtype=np.int64 if dt == pb.INT64 else np.float32)
            ctx.consts[n.outputs[0]] = arr
            return [TensorType(dt, [] if scalar else [Dim.of(arr.size)])]
    return None


@rule("Shape")
def _shape(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return [TensorType(pb.INT64, [None])]
    start, end = int(n.attrs.get("start", 0)), n.attrs.get("end")
    rank = len(s)
    start = max(0, min(rank, _norm_axis(start, rank)))
    end = rank if end is None else max(0, min(rank, _norm_axis(int(end), rank)))
    ctx.data[n.outputs[0]] = s[start:end]
    return [TensorType(pb.INT64, [Dim.of(max(0, end - start))])]


@rule("Size")
def _size(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is not None and _prod(s) is not None:
        ctx.data[n.outputs[0]] = [_prod(s)]
    return [TensorType(pb.INT64, [])]


@rule("Reshape")
def _reshape(ctx, n):
    src, target = ctx.shape(n.inputs[0]), ctx.values(n.inputs[1])
    dt = ctx.dtype(n.inputs[0])
    if target is None:
        ts = ctx.shape(n.inputs[1])
        if ts is not None and len(ts) == 1 and ts[0] is not None and ts[0].is_const:
            return [TensorType(dt, [None] * ts[0].const())]
        return [TensorType(dt, None)]
    allowzero = int(n.attrs.get("allowzero", 0))
    out = []
    for i, v in enumerate(target):
        if v is not None and v == 0 and not allowzero:
            out.append(src[i] if src is not None and i < len(src) else None)
        else:
            out.append(v)
    minus = [i for i, v in enumerate(out) if v is not None and v == -1]
    if minus:
        known = _prod([v for i, v in enumerate(out) if i != minus[0]])
        total = _prod(src) if src is not None else None
        out[minus[0]] = None
        if known is not None and total is not None:
            q = total.exact_div(known)
            out[minus[0]] = q if q is not None else ctx.fresh_symbol("reshape")
    if ctx.values(n.inputs[0]) is not None and all(v is not None and v.is_const for v in out) and len(out) <= 1:
        ctx.data[n.outputs[0]] = ctx.values(n.inputs[0])
    return [TensorType(dt, out)]


@rule("Flatten")
def _flatten(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return [TensorType(ctx.dtype(n.inputs[0]), [None, None])]
    ax = _norm_axis(int(n.attrs.get("axis", 1)), len(s))
    return [TensorType(ctx.dtype(n.inputs[0]), [_prod(s[:ax]), _prod(s[ax:])])]


@rule("Transpose")
def _transpose(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    perm = list(n.attrs.get("perm", reversed(range(len(s)))))
    return [TensorType(ctx.dtype(n.inputs[0]), [s[p] for p in perm])]


def _axes_of(ctx, n, idx=1):
    if "axes" in n.attrs:
        return [int(a) for a in n.attrs["axes"]]
    if len(n.inputs) > idx and n.inputs[idx]:
        return ctx.ints(n.inputs[idx])
    return None


@rule("Unsqueeze")
def _unsqueeze(ctx, n):
    s, axes = ctx.shape(n.inputs[0]), _axes_of(ctx, n)
    if s is None or axes is None:
        return None
    rank = len(s) + len(axes)
    axes = sorted(_norm_axis(a, rank) for a in axes)
    out = list(s)
    for a in axes:
        out.insert(a, Dim.of(1))
    v = ctx.values(n.inputs[0])
    if v is not None and len(s) <= 1:
        ctx.data[n.outputs[0]] = v
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("Squeeze")
def _squeeze(ctx, n):
    s, axes = ctx.shape(n.inputs[0]), _axes_of(ctx, n)
    if s is None:
        return None
    if axes is None:
        if len(n.inputs) > 1 and n.inputs[1]:
            return None
        out = [d for d in s if not (d is not None and d == 1)]
    else:
        drop = {_norm_axis(a, len(s)) for a in axes}
        out = [d for i, d in enumerate(s) if i not in drop]
    v = ctx.values(n.inputs[0])
    if v is not None:
        ctx.data[n.outputs[0]] = v
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("Concat")
def _concat(ctx, n):
    shapes = [ctx.shape(x) for x in n.inputs]
    dt = ctx.dtype(n.inputs[0])
    vals = [ctx.values(x) for x in n.inputs]
    if all(v is not None for v in vals) and all(s is not None and len(s) <= 1 for s in shapes):
        ctx.data[n.outputs[0]] = [e for v in vals for e in v]
    known = [s for s in shapes if s is not None]
    if not known:
        return [TensorType(dt, None)]
    rank = len(known[0])
    ax = _norm_axis(int(n.attrs.get("axis", 0)), rank)
    out = [None] * rank
    for i in range(rank):
        if i == ax:
            tot = Dim.of(0)
            for s in shapes:
                if s is None or s[i] is None:
                    tot = None
                    break
                tot = tot + s[i]
            out[i] = tot
        else:
            d = None
            for s in known:
                d = ctx.merge(d, s[i], f"Concat axis {i}")
            out[i] = d
    return [TensorType(dt, out)]


@rule("Split")
def _split(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    ax = _norm_axis(int(n.attrs.get("axis", 0)), len(s))
    sizes = [int(x) for x in n.attrs["split"]] if "split" in n.attrs else (ctx.ints(n.inputs[1]) if len(n.inputs) > 1 and n.inputs[1] else None)
    k = len(n.outputs)
    outs = []
    for i in range(k):
        o = list(s)
        if sizes is not None:
            o[ax] = Dim.of(sizes[i])
        elif s[ax] is not None and s[ax].is_const:
            total = s[ax].const()
            chunk = -(-total // k)
            o[ax] = Dim.of(max(0, min(chunk, total - i * chunk)))
        else:
            o[ax] = s[ax].exact_div(k) if s[ax] is not None else None
        outs.append(TensorType(ctx.dtype(n.inputs[0]), o))
    return outs


@rule("Slice")
def _slice(ctx, n):
    s = ctx.shape(n.inputs[0])
    dt = ctx.dtype(n.inputs[0])
    if s is None:
        return None
    if "starts" in n.attrs:
        starts, ends = [int(x) for x in n.attrs["starts"]], [int(x) for x in n.attrs["ends"]]
        axes = [int(x) for x in n.attrs.get("axes", range(len(starts)))]
        steps = [1] * len(starts)
    else:
        starts, ends = ctx.values(n.inputs[1]), ctx.values(n.inputs[2])
        axes = ctx.ints(n.inputs[3]) if len(n.inputs) > 3 and n.inputs[3] else None
        steps = ctx.ints(n.inputs[4]) if len(n.inputs) > 4 and n.inputs[4] else None
        if starts is None or ends is None:
            return [TensorType(dt, [None] * len(s))]
        axes = list(range(len(starts))) if axes is None else axes
        steps = [1] * len(starts) if steps is None else steps
    out = list(s)
    data = ctx.values(n.inputs[0])
    for st, en, ax, step in zip(starts, ends, axes, steps):
        ax = _norm_axis(ax, len(s))
        dim = s[ax]
        st_c = st if isinstance(st, int) else (st.const() if st is not None and st.is_const else None)
        en_c = en if isinstance(en, int) else (en.const() if en is not None and en.is_const else None)
        if dim is not None and dim.is_const and st_c is not None and en_c is not None:
            ln = len(range(*slice(st_c, en_c, step).indices(dim.const())))
            out[ax] = Dim.of(ln)
            if data is not None and len(s) == 1:
                data = data[slice(st_c, en_c, step)]
        elif st_c is not None and en_c is not None and step == 1 and st_c >= 0 and en_c >= 0 and en_c < (1 << 30):
            out[ax] = Dim.of(max(0, en_c - st_c))          # a window that lies inside the (symbolic) extent is assumed
            data = None
        elif st_c is not None and st_c >= 0 and step == 1 and en_c is not None and en_c >= (1 << 30) and dim is not None:
            out[ax] = dim - st_c
            data = None
        elif step == 1 and st is not None and en is not None and not isinstance(st, int) and not isinstance(en, int) and st_c is not None and st_c >= 0:
            out[ax] = en - st                               # symbolic end (for instance a sequence length taken from a Shape)
            data = None
        else:
            out[ax] = None
            data = None
    if data is not None and len(s) == 1:
        ctx.data[n.outputs[0]] = data
    return [TensorType(dt, out)]


@rule("Gather")
def _gather(ctx, n):
    s, idx = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[1])
    dt = ctx.dtype(n.inputs[0])
    if s is None or idx is None:
        return [TensorType(dt, None)]
    ax = _norm_axis(int(n.attrs.get("axis", 0)), len(s))
    data, iv = ctx.values(n.inputs[0]), ctx.ints(n.inputs[1])
    if data is not None and iv is not None and len(s) == 1:
        ctx.data[n.outputs[0]] = [data[i] for i in iv]
    return [TensorType(dt, s[:ax] + idx + s[ax + 1:])]


@rule("GatherElements", "ScatterElements", "ScatterND", "Scatter")
def _like_first_or_index(ctx, n):
    if n.op_type == "GatherElements":
        return [TensorType(ctx.dtype(n.inputs[0]), ctx.shape(n.inputs[1]))]
    return [TensorType(ctx.dtype(n.inputs[0]), ctx.shape(n.inputs[0]))]


@rule("GatherND")
def _gather_nd(ctx, n):
    s, idx = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[1])
    if s is None or idx is None or idx[-1] is None or not idx[-1].is_const:
        return [TensorType(ctx.dtype(n.inputs[0]), None)]
    b = int(n.attrs.get("batch_dims", 0))
    return [TensorType(ctx.dtype(n.inputs[0]), idx[:-1] + s[b + idx[-1].const():])]


@rule("Expand")
def _expand(ctx, n):
    s, target = ctx.shape(n.inputs[0]), ctx.values(n.inputs[1])
    if target is None:
        return [TensorType(ctx.dtype(n.inputs[0]), None)]
    return [TensorType(ctx.dtype(n.inputs[0]), _broadcast(ctx, [s, target], "Expand"))]


@rule("Tile")
def _tile(ctx, n):
    s, reps = ctx.shape(n.inputs[0]), ctx.values(n.inputs[1])
    if s is None:
        return None
    if reps is None:
        return [TensorType(ctx.dtype(n.inputs[0]), [None] * len(s))]
    return [TensorType(ctx.dtype(n.inputs[0]), [None if (d is None or r is None) else d * r for d, r in zip(s, reps)])]


@rule("ConstantOfShape")
def _constant_of_shape(ctx, n):
    v = n.attrs.get("value")
    dt = v.data_type if v is not None else pb.FLOAT
    target = ctx.values(n.inputs[0])
    if target is None:
        ts = ctx.shape(n.inputs[0])
        rank = ts[0].const() if ts and ts[0] is not None and ts[0].is_const else None
        return [TensorType(dt, None if rank is None else [None] * rank)]
    return [TensorType(dt, target)]


@rule("Range")
def _range(ctx, n):
    a, b, c = (ctx.values(x) for x in n.inputs)
    dt = ctx.dtype(n.inputs[0])
    if a and b and c and all(v[0] is not None for v in (a, b, c)):
        start, limit, delta = a[0], b[0], c[0]
        if start.is_const and limit.is_const and delta.is_const and delta.const() != 0:
            return [TensorType(dt, [Dim.of(max(0, -(-(limit.const() - start.const()) // delta.const())))])]
        if delta == 1:
            return [TensorType(dt, [limit - start])]
    return [TensorType(dt, [ctx.fresh_symbol("range")])]


@rule("MatMul", "MatMulInteger", "QLinearMatMul")
def _matmul(ctx, n):
    ia, ib = (0, 3) if n.op_type == "QLinearMatMul" else (0, 1)
    a, b = ctx.shape(n.inputs[ia]), ctx.shape(n.inputs[ib])
    dt = pb.INT32 if n.op_type == "MatMulInteger" else (ctx.dtype(n.inputs[7]) if n.op_type == "QLinearMatMul" else ctx.dtype(n.inputs[0]))
    if a is None or b is None:
        return [TensorType(dt, None)]
    if len(a) == 1 and len(b) == 1:
        return [TensorType(dt, [])]
    if len(a) == 1:
        return [TensorType(dt, b[:-2] + b[-1:])]
    if len(b) == 1:
        return [TensorType(dt, a[:-1])]
    batch = _broadcast(ctx, [a[:-2], b[:-2]], "MatMul")
    return [TensorType(dt, batch + [a[-2], b[-1]])]


@rule("Gemm", "com.microsoft::FusedGemm")
def _gemm(ctx, n):
    a, b = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[1])
    if a is None or b is None:
        return [TensorType(ctx.dtype(n.inputs[0]), [None, None])]
    m = a[1] if int(n.attrs.get("transA", 0)) else a[0]
    nn = b[0] if int(n.attrs.get("transB", 0)) else b[1]
    return [TensorType(ctx.dtype(n.inputs[0]), [m, nn])]


@rule("com.microsoft::MatMulNBits")
def _matmul_nbits(ctx, n):
    a = ctx.shape(n.inputs[0])
    if a is None:
        return None
    return [TensorType(ctx.dtype(n.inputs[0]), a[:-1] + [Dim.of(int(n.attrs["N"]))])]


def _spatial(ctx, n, x, kernel, out_channels):
    """Output extents of a convolution / pooling window over the trailing spatial axes of ``x``."""
    nd = len(kernel)
    strides = [int(v) for v in n.attrs.get("strides", [1] * nd)]
    dil = [int(v) for v in n.attrs.get("dilations", [1] * nd)]
    pads = [int(v) for v in n.attrs.get("pads", [0] * (2 * nd))]
    auto = n.attrs.get("auto_pad", "NOTSET")
    auto = auto.decode() if isinstance(auto, bytes) else auto
    ceil_mode = int(n.attrs.get("ceil_mode", 0))
    out = [x[0], out_channels]
    for i in range(nd):
        d = x[2 + i]
        if d is None or not d.is_const:
            same = auto in ("SAME_UPPER", "SAME_LOWER")
            out.append(d if (same and strides[i] == 1) or (d is not None and kernel[i] == 1 and strides[i] == 1 and pads[i] + pads[nd + i] == 0) else None)
            continue
        size = d.const()
        if auto in ("SAME_UPPER", "SAME_LOWER"):
            out.append(Dim.of(-(-size // strides[i])))
            continue
        pad = 0 if auto == "VALID" else pads[i] + pads[nd + i]
        eff = dil[i] * (kernel[i] - 1) + 1
        num = size + pad - eff
        o = (-(-num // strides[i]) if ceil_mode else num // strides[i]) + 1
        if ceil_mode and (o - 1) * strides[i] >= size + pads[i]:
            o -= 1
        out.append(Dim.of(max(0, o)))
    return out


@rule("Conv", "ConvInteger", "QLinearConv")
def _conv(ctx, n):
    wi = 3 if n.op_type == "QLinearConv" else 1
    x, w = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[wi])
    dt = pb.INT32 if n.op_type == "ConvInteger" else ctx.dtype(n.inputs[0])
    if x is None or w is None:
        return [TensorType(dt, None)]
    kernel = [int(v) for v in n.attrs["kernel_shape"]] if "kernel_shape" in n.attrs else \
        [d.const() if d is not None and d.is_const else None for d in w[2:]]
    if any(k is None for k in kernel):
        return [TensorType(dt, [x[0], w[0]] + [None] * (len(x) - 2))]
    return [TensorType(dt, _spatial(ctx, n, x, kernel, w[0]))]


@rule("ConvTranspose")
def _conv_transpose(ctx, n):
    x, w = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[1])
    if x is None or w is None:
        return None
    nd = len(x) - 2
    group = int(n.attrs.get("group", 1))
    kernel = [int(v) for v in n.attrs["kernel_shape"]] if "kernel_shape" in n.attrs else [d.const() if d is not None and d.is_const else None for d in w[2:]]
    strides = [int(v) for v in n.attrs.get("strides", [1] * nd)]
    dil = [int(v) for v in n.attrs.get("dilations", [1] * nd)]
    pads = [int(v) for v in n.attrs.get("pads", [0] * (2 * nd))]
    opad = [int(v) for v in n.attrs.get("output_padding", [0] * nd)]
    out = [x[0], None if w[1] is None else w[1] * group]
    if "output_shape" in n.attrs:
        return [TensorType(ctx.dtype(n.inputs[0]), out + [Dim.of(int(v)) for v in n.attrs["output_shape"]])]
    for i in range(nd):
        d = x[2 + i]
        if d is None or kernel[i] is None:
            out.append(None)
        else:
            out.append((d - 1) * strides[i] + (opad[i] + (kernel[i] - 1) * dil[i] + 1 - pads[i] - pads[nd + i]))
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("MaxPool", "AveragePool", "LpPool")
def _pool(ctx, n):
    x = ctx.shape(n.inputs[0])
    if x is None:
        return None
    kernel = [int(v) for v in n.attrs["kernel_shape"]]
    outs = [TensorType(ctx.dtype(n.inputs[0]), _spatial(ctx, n, x, kernel, x[1]))]
    if len(n.outputs) > 1:
        outs.append(TensorType(pb.INT64, outs[0].shape))
    return outs


@rule("GlobalAveragePool", "GlobalMaxPool", "GlobalLpPool")
def _global_pool(ctx, n):
    x = ctx.shape(n.inputs[0])
    if x is None:
        return None
    return [TensorType(ctx.dtype(n.inputs[0]), x[:2] + [Dim.of(1)] * (len(x) - 2))]


_REDUCE = "ReduceSum ReduceMean ReduceMax ReduceMin ReduceProd ReduceL1 ReduceL2 ReduceLogSum ReduceLogSumExp ReduceSumSquare".split()


@rule(*_REDUCE)
def _reduce(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    keep = int(n.attrs.get("keepdims", 1))
    axes = _axes_of(ctx, n)
    if axes is None:
        if len(n.inputs) > 1 and n.inputs[1]:
            return [TensorType(ctx.dtype(n.inputs[0]), [None] * len(s) if keep else None)]
        if int(n.attrs.get("noop_with_empty_axes", 0)):
            return [TensorType(ctx.dtype(n.inputs[0]), s)]
        axes = list(range(len(s)))
    axes = {_norm_axis(a, len(s)) for a in axes}
    out = [Dim.of(1) if i in axes else d for i, d in enumerate(s) if keep or i not in axes]
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("ArgMax", "ArgMin")
def _argmax(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    ax = _norm_axis(int(n.attrs.get("axis", 0)), len(s))
    keep = int(n.attrs.get("keepdims", 1))
    return [TensorType(pb.INT64, [Dim.of(1) if i == ax else d for i, d in enumerate(s) if keep or i != ax])]


@rule("TopK")
def _topk(ctx, n):
    s, k = ctx.shape(n.inputs[0]), ctx.values(n.inputs[1]) if len(n.inputs) > 1 else [Dim.of(int(n.attrs["k"]))]
    if s is None:
        return None
    ax = _norm_axis(int(n.attrs.get("axis", -1)), len(s))
    out = list(s)
    out[ax] = k[0] if k else None
    return [TensorType(ctx.dtype(n.inputs[0]), out), TensorType(pb.INT64, out)]


@rule("LayerNormalization", "SimplifiedLayerNormalization", "com.microsoft::SimplifiedLayerNormalization", "RMSNormalization",
      "com.microsoft::SkipLayerNormalization", "com.microsoft::SkipSimplifiedLayerNormalization", "GroupNormalization",
      "BatchNormalization")
def _norm(ctx, n):
    t = ctx.type(n.inputs[0])
    if t is None or t.shape is None:
        return None
    outs = [TensorType(t.dtype, t.shape)]
    if n.op_type == "BatchNormalization":
        c = [t.shape[1]] if len(t.shape) > 1 else None
        outs += [TensorType(t.dtype, c)] * (len(n.outputs) - 1)
        return outs
    skip = n.op_type.startswith("Skip")
    ax = _norm_axis(int(n.attrs.get("axis", -1)), len(t.shape))
    stat = t.shape[:ax] + [Dim.of(1)] * (len(t.shape) - ax)
    for i in range(1, len(n.outputs)):
        last = skip and i == len(n.outputs) - 1 and i == 3
        outs.append(TensorType(t.dtype if last else pb.FLOAT, t.shape if last else stat))
    return outs


@rule("Pad")
def _pad(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    pads = [int(v) for v in n.attrs["pads"]] if "pads" in n.attrs else ctx.ints(n.inputs[1])
    if pads is None:
        return [TensorType(ctx.dtype(n.inputs[0]), [None] * len(s))]
    axes = ctx.ints(n.inputs[3]) if len(n.inputs) > 3 and n.inputs[3] else list(range(len(s)))
    out = list(s)
    k = len(axes)
    for j, ax in enumerate(axes):
        ax = _norm_axis(ax, len(s))
        out[ax] = None if s[ax] is None else s[ax] + pads[j] + pads[k + j]
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("Resize", "Upsample")
def _resize(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None:
        return None
    sizes = ctx.values(n.inputs[3]) if len(n.inputs) > 3 and n.inputs[3] else None
    scales_name = n.inputs[2] if n.op_type == "Resize" and len(n.inputs) > 2 else (n.inputs[1] if n.op_type == "Upsample" and len(n.inputs) > 1 else "")
    scales = ctx.consts.get(scales_name) if scales_name else None
    axes = [int(a) for a in n.attrs["axes"]] if "axes" in n.attrs else None
    out = list(s)
    if sizes is not None:
        for j, v in enumerate(sizes):
            out[_norm_axis(axes[j], len(s)) if axes else j] = v
    elif scales is not None and scales.size:
        for j, sc in enumerate(np.asarray(scales).reshape(-1)):
            i = _norm_axis(axes[j], len(s)) if axes else j
            out[i] = Dim.of(int(np.floor(s[i].const() * float(sc)))) if s[i] is not None and s[i].is_const else (s[i] if float(sc) == 1.0 else None)
    else:
        out = [None] * len(s)
    return [TensorType(ctx.dtype(n.inputs[0]), out)]


@rule("OneHot")
def _one_hot(ctx, n):
    s, depth = ctx.shape(n.inputs[0]), ctx.values(n.inputs[1])
    if s is None:
        return None
    ax = int(n.attrs.get("axis", -1))
    ax = ax + len(s) + 1 if ax < 0 else ax
    out = list(s)
    out.insert(ax, depth[0] if depth else None)
    return [TensorType(ctx.dtype(n.inputs[2]), out)]


@rule("NonZero")
def _nonzero(ctx, n):
    s = ctx.shape(n.inputs[0])
    return [TensorType(pb.INT64, [None if s is None else Dim.of(len(s)), ctx.fresh_symbol("nonzero")])]


@rule("Einsum")
def _einsum(ctx, n):
    eq = n.attrs["equation"]
    eq = (eq.decode() if isinstance(eq, bytes) else eq).replace(" ", "")
    if "->" not in eq or "..." in eq:
        return None
    lhs, rhs = eq.split("->")
    sizes: dict = {}
    for term, name in zip(lhs.split(","), n.inputs):
        s = ctx.shape(name)
        if s is None or len(s) != len(term):
            return None
        for ch, d in zip(term, s):
            sizes[ch] = ctx.merge(sizes.get(ch), d, f"Einsum index {ch}")
    return [TensorType(ctx.dtype(n.inputs[0]), [sizes.get(ch) for ch in rhs])]


@rule("DequantizeLinear")
def _dequant(ctx, n):
    return [TensorType(ctx.dtype(n.inputs[1]) or pb.FLOAT, ctx.shape(n.inputs[0]))]


@rule("QuantizeLinear")
def _quant(ctx, n):
    dt = ctx.dtype(n.inputs[2]) if len(n.inputs) > 2 and n.inputs[2] else pb.UINT8
    return [TensorType(dt, ctx.shape(n.inputs[0]))]


@rule("DynamicQuantizeLinear")
def _dyn_quant(ctx, n):
    return [TensorType(pb.UINT8, ctx.shape(n.inputs[0])), TensorType(pb.FLOAT, []), TensorType(pb.UINT8, [])]


@rule("RotaryEmbedding", "com.microsoft::RotaryEmbedding")
def _rotary(ctx, n):
    return [TensorType(ctx.dtype(n.inputs[0]), ctx.shape(n.inputs[0]))]


@rule("com.microsoft::GroupQueryAttention")
def _gqa(ctx, n):
    q, past = ctx.shape(n.inputs[0]), ctx.shape(n.inputs[3]) if len(n.inputs) > 3 else None
    dt = ctx.dtype(n.inputs[0])
    if q is None:
        return None
    heads, kv_heads = int(n.attrs["num_heads"]), int(n.attrs["kv_num_heads"])
    packed = len(n.inputs) < 2 or not n.inputs[1]
    hidden = q[-1]
    if packed and hidden is not None:
        hidden = hidden.exact_div(heads + 2 * kv_heads)
        hidden = None if hidden is None else hidden * heads
    out = [TensorType(dt, q[:-1] + [hidden])]
    head_dim = None if hidden is None else hidden.exact_div(heads)
    if past is not None:
        total = None if past[2] is None or q[1] is None else past[2] + q[1]
        present = [past[0], past[1], total, past[3]]
    else:
        present = [q[0], Dim.of(kv_heads), None, head_dim]
    out += [TensorType(dt, present)] * (len(n.outputs) - 1)
    return out


@rule("Attention")
def _attention23(ctx, n):
    q, k, v = (ctx.shape(x) for x in n.inputs[:3])
    dt = ctx.dtype(n.inputs[0])
    if q is None or v is None:
        return None
    if len(q) == 4:
        y = q[:3] + [v[3]]
    else:
        qh, kvh = int(n.attrs["q_num_heads"]), int(n.attrs["kv_num_heads"])
        vd = None if v[2] is None else v[2].exact_div(kvh)
        y = q[:2] + [None if vd is None else vd * qh]
    outs = [TensorType(dt, y)]
    past_k = ctx.shape(n.inputs[4]) if len(n.inputs) > 4 and n.inputs[4] else None
    for i in range(1, len(n.outputs)):
        src = k if i == 1 else v
        if i > 2 or src is None or len(src) != 4:
            outs.append(TensorType(dt, None))
            continue
        total = src[2] if past_k is None else (None if past_k[2] is None or src[2] is None else past_k[2] + src[2])
        outs.append(TensorType(dt, [src[0], src[1], total, src[3]]))
    return outs


@rule("DepthToSpace", "SpaceToDepth")
def _depth_space(ctx, n):
    s = ctx.shape(n.inputs[0])
    if s is None or len(s) != 4:
        return None
    b = int(n.attrs["blocksize"])
    if n.op_type == "DepthToSpace":
        c = None if s[1] is None else s[1].exact_div(b * b)
        return [TensorType(ctx.dtype(n.inputs[0]), [s[0], c, None if s[2] is None else s[2] * b, None if s[3] is None else s[3] * b])]
    return [TensorType(ctx.dtype(n.inputs[0]), [s[0], None if s[1] is None else s[1] * (b * b), None if s[2] is None else s[2].exact_div(b),
                                                None if s[3] is None else s[3].exact_div(b)])]


@rule("EyeLike", "Bernoulli", "RandomNormalLike", "RandomUniformLike")
def _like(ctx, n):
    dt = int(n.attrs["dtype"]) if "dtype" in n.attrs else ctx.dtype(n.inputs[0])
    return [TensorType(dt, ctx.shape(n.inputs[0]))]


@rule("RandomNormal", "RandomUniform")
def _random(ctx, n):
    return [TensorType(int(n.attrs.get("dtype", pb.FLOAT)), [Dim.of(int(v)) for v in n.attrs["shape"]])]


@rule("Compress", "Unique")
def _data_dependent(ctx, n):
    s = ctx.shape(n.inputs[0])
    if n.op_type == "Compress" and s is not None and "axis" in n.attrs:
        out = list(s)
        out[_norm_axis(int(n.attrs["axis"]), len(s))] = ctx.fresh_symbol("compress")
        return [TensorType(ctx.dtype(n.inputs[0]), out)]
    first = TensorType(ctx.dtype(n.inputs[0]), [ctx.fresh_symbol(n.op_type.lower())])
    return [first] + [TensorType(pb.INT64, [None])] * (len(n.outputs) - 1)


# ---------------------------------------------------------------------------------------------------------------------
# driver
# ---------------------------------------------------------------------------------------------------------------------
def _from_value_info(vi) -> TensorType:
    shape = None
    if vi.shape is not None:
        shape = []
        for d in vi.shape:
            shape.append(Dim.of(d) if isinstance(d, (int, np.integer)) and d >= 0 else (Dim.of(d) if isinstance(d, str) and d else None))
    return TensorType(vi.elem_type, shape)


def _toposort(graph):
    produced = {o: n for n in graph.nodes for o in n.outputs if o}
    order, state = [], {}
    for root in graph.nodes:
        stack = [(root, iter([produced[i] for i in root.inputs if i in produced]))]
        if state.get(id(root)):
            continue
        state[id(root)] = 1
        while stack:
            node, it = stack[-1]
            nxt = next(it, None)
            if nxt is None:
                order.append(node)
                state[id(node)] = 2
                stack.pop()
            elif not state.get(id(nxt)):
                state[id(nxt)] = 1
                stack.append((nxt, iter([produced[i] for i in nxt.inputs if i in produced])))
    return order


def infer(model, input_shapes: dict | None = None, policy: str = "permissive") -> InferenceReport:
    """Infer the type and shape of every value of ``model.graph``.

    ``input_shapes`` overrides or completes the declared input shapes (``{name: [dims]}``, a dim an int, a symbol name or
    None).  ``policy``: ``"permissive"`` (default) or ``"strict"``."""
    if policy not in ("permissive", "strict"):
        raise ValueError("policy must be 'permissive' or 'strict'")
    g = model.graph
    ctx = _Ctx(policy)
    for name, t in g.initializers.items():
        ctx.types[name] = TensorType(t.data_type, [Dim.of(int(d)) for d in t.dims])
        arr = t.numpy()
        if arr is not None and int(np.prod(t.dims, dtype=np.int64)) <= 64:
            ctx.consts[name] = np.asarray(arr).reshape(tuple(int(d) for d in t.dims))
    for vi in g.inputs:
        if vi.name in g.initializers:
            continue
        tt = _from_value_info(vi)
        if input_shapes and vi.name in input_shapes:
            tt.shape = [_d(d) for d in input_shapes[vi.name]]
        ctx.types[vi.name] = tt
    report = InferenceReport()
    for n in _toposort(g):
        key = f"{n.domain}::{n.op_type}" if n.domain not in ("", "ai.onnx") else n.op_type
        fn = RULES.get(key) or (RULES.get(n.op_type) if n.domain in ("", "ai.onnx") else None)
        outs = None
        if fn is None:
            report.unregistered[key] = report.unregistered.get(key, 0) + 1
        else:
            try:
                outs = fn(ctx, n)
            except ShapeInferenceError:
                raise
            except (KeyError, IndexError, TypeError, AttributeError, ValueError):
                outs = None                      # malformed or unusual node: leave its outputs unresolved
        for i, name in enumerate(n.outputs):
            if not name:
                continue
            ctx.types[name] = outs[i] if outs is not None and i < len(outs) and outs[i] is not None else TensorType()
    declared = {vo.name: _from_value_info(vo) for vo in g.outputs}
    for name, want in declared.items():
        got = ctx.types.get(name)
        if got is None:
            ctx.types[name] = want
            continue
        if got.dtype is None:
            got.dtype = want.dtype
        if got.shape is None:
            got.shape = want.shape
        elif want.shape is not None and len(want.shape) == len(got.shape):
            got.shape = [ctx.merge(a, b, f"output {name} axis {i}") for i, (a, b) in enumerate(zip(got.shape, want.shape))]
        elif want.shape is not None and policy == "strict":
            raise ShapeInferenceError(f"output {name}: inferred rank {len(got.shape)} but the graph declares rank {len(want.shape)}")
    report.types = ctx.types
    report.unresolved = sorted(name for name, t in ctx.types.items() if not t.resolved and name not in g.initializers)
    report.fresh_symbols = ctx.fresh
    return report
