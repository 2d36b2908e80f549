"""Well-formedness checker for ONNX models, over this package's own graph objects.

Counterpart of the reference's model checker and operator-schema registry (crates/onnx-runtime-onnx-std: a schema per
operator -- arity, attribute names and kinds -- and a checker that walks a model before anything executes it).  A loader
that accepts anything turns a malformed file into a confusing failure deep inside a kernel; this pass reports every
problem it finds, each with the node it belongs to, before the graph is run or lowered:

* structure    values defined exactly once (SSA), every node input defined before its use (topological order), subgraph
               bodies checked in a scope chained over the enclosing graph, graph outputs produced, no empty or clashing names;
* operator set every node's domain has an opset import; default-domain operators are known to the schema table;
* schema       input / output counts inside the operator's range, required attributes present, attribute kinds as declared;
* tensors      initializer payload size equal to the product of its dimensions times the element size.

``check_model`` returns a list of :class:`Problem`; ``severity`` is ``error`` (the model cannot run as written) or
``warning`` (legal but suspicious: an initializer nothing reads, an operator the table does not know).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import onnx_pb as pb

I, F, S, T, G, IS, FS, SS = "int", "float", "string", "tensor", "graph", "ints", "floats", "strings"
INF = 1 << 30


@dataclass
class Problem:
    severity: str
    where: str
    message: str

    def __str__(self):
        return f"{self.severity}: {self.where}: {self.message}"


def _s(min_in, max_in, min_out=1, max_out=1, attrs=None, required=()):
    return (min_in, max_in, min_out, max_out, attrs or {}, tuple(required))


_UNARY = ("Abs Neg Exp Log Sqrt Reciprocal Relu Sigmoid Tanh Erf Floor Ceil Round Sign Sin Cos Tan Asin Acos Atan Sinh Cosh Asinh Acosh "
          "Atanh Softplus Softsign Identity Not BitwiseNot Mish IsNaN Size Shape NonZero GlobalAveragePool GlobalMaxPool Det Swish").split()
_BINARY = "Add Sub Mul Div Pow Equal Less Greater LessOrEqual GreaterOrEqual And Or Xor BitwiseAnd BitwiseOr BitwiseXor PRelu MatMul".split()
_VARIADIC = "Min Max Mean Sum".split()
_REDUCE = "ReduceSum ReduceMean ReduceMax ReduceMin ReduceProd ReduceL1 ReduceL2 ReduceLogSum ReduceLogSumExp ReduceSumSquare".split()

SCHEMAS: dict = {n: _s(1, 1) for n in _UNARY}
SCHEMAS.update({n: _s(2, 2) for n in _BINARY})
SCHEMAS.update({n: _s(1, INF) for n in _VARIADIC})
SCHEMAS.update({n: _s(1, 2, attrs={"axes": IS, "keepdims": I, "noop_with_empty_axes": I}) for n in _REDUCE})
SCHEMAS.update({
    "Shape": _s(1, 1, attrs={"start": I, "end": I}),
    "Mod": _s(2, 2, attrs={"fmod": I}), "BitShift": _s(2, 2, attrs={"direction": S}, required=("direction",)),
    "Elu": _s(1, 1, attrs={"alpha": F}), "Selu": _s(1, 1, attrs={"alpha": F, "gamma": F}), "Celu": _s(1, 1, attrs={"alpha": F}),
    "LeakyRelu": _s(1, 1, attrs={"alpha": F}), "ThresholdedRelu": _s(1, 1, attrs={"alpha": F}), "HardSigmoid": _s(1, 1, attrs={"alpha": F, "beta": F}),
    "HardSwish": _s(1, 1), "Gelu": _s(1, 1, attrs={"approximate": S}), "Shrink": _s(1, 1, attrs={"bias": F, "lambd": F}),
    "IsInf": _s(1, 1, attrs={"detect_negative": I, "detect_positive": I}),
    "Softmax": _s(1, 1, attrs={"axis": I}), "LogSoftmax": _s(1, 1, attrs={"axis": I}), "Hardmax": _s(1, 1, attrs={"axis": I}),
    "Clip": _s(1, 3, attrs={"min": F, "max": F}), "Cast": _s(1, 1, attrs={"to": I, "saturate": I}, required=("to",)), "CastLike": _s(2, 2, attrs={"saturate": I}),
    "Where": _s(3, 3), "Dropout": _s(1, 3, 1, 2, attrs={"seed": I, "ratio": F}),
    "Constant": _s(0, 0, attrs={"value": T, "value_int": I, "value_float": F, "value_ints": IS, "value_floats": FS, "value_string": S,
                               "value_strings": SS, "sparse_value": T}),
    "ConstantOfShape": _s(1, 1, attrs={"value": T}), "Range": _s(3, 3), "EyeLike": _s(1, 1, attrs={"dtype": I, "k": I}),
    "Reshape": _s(2, 2, attrs={"allowzero": I}), "Flatten": _s(1, 1, attrs={"axis": I}), "Transpose": _s(1, 1, attrs={"perm": IS}),
    "Squeeze": _s(1, 2, attrs={"axes": IS}), "Unsqueeze": _s(1, 2, attrs={"axes": IS}), "Expand": _s(2, 2), "Tile": _s(2, 2),
    "Concat": _s(1, INF, attrs={"axis": I}, required=("axis",)), "Split": _s(1, 2, 1, INF, attrs={"axis": I, "split": IS, "num_outputs": I}),
    "Slice": _s(1, 5, attrs={"starts": IS, "ends": IS, "axes": IS}), "Gather": _s(2, 2, attrs={"axis": I}), "GatherElements": _s(2, 2, attrs={"axis": I}),
    "GatherND": _s(2, 2, attrs={"batch_dims": I}), "ScatterElements": _s(3, 3, attrs={"axis": I, "reduction": S}),
    "ScatterND": _s(3, 3, attrs={"reduction": S}), "Pad": _s(1, 4, attrs={"mode": S, "pads": IS, "value": F}),
    "Trilu": _s(1, 2, attrs={"upper": I}), "CumSum": _s(2, 2, attrs={"exclusive": I, "reverse": I}), "OneHot": _s(3, 3, attrs={"axis": I}),
    "DepthToSpace": _s(1, 1, attrs={"blocksize": I, "mode": S}, required=("blocksize",)), "SpaceToDepth": _s(1, 1, attrs={"blocksize": I}, required=("blocksize",)),
    "ArgMax": _s(1, 1, attrs={"axis": I, "keepdims": I, "select_last_index": I}), "ArgMin": _s(1, 1, attrs={"axis": I, "keepdims": I, "select_last_index": I}),
    "TopK": _s(1, 2, 2, 2, attrs={"axis": I, "largest": I, "sorted": I, "k": I}), "Unique": _s(1, 1, 1, 4, attrs={"axis": I, "sorted": I}),
    "Compress": _s(2, 2, attrs={"axis": I}), "NonMaxSuppression": _s(2, 5, attrs={"center_point_box": I}),
    "Gemm": _s(2, 3, attrs={"alpha": F, "beta": F, "transA": I, "transB": I}), "MatMulInteger": _s(2, 4), "QLinearMatMul": _s(8, 8),
    "Einsum": _s(1, INF, attrs={"equation": S}, required=("equation",)),
    "Conv": _s(2, 3, attrs={"auto_pad": S, "dilations": IS, "group": I, "kernel_shape": IS, "pads": IS, "strides": IS}),
    "ConvTranspose": _s(2, 3, attrs={"auto_pad": S, "dilations": IS, "group": I, "kernel_shape": IS, "pads": IS, "strides": IS, "output_padding": IS,
                                      "output_shape": IS}),
    "ConvInteger": _s(2, 4, attrs={"auto_pad": S, "dilations": IS, "group": I, "kernel_shape": IS, "pads": IS, "strides": IS}),
    "MaxPool": _s(1, 1, 1, 2, attrs={"auto_pad": S, "ceil_mode": I, "dilations": IS, "kernel_shape": IS, "pads": IS, "strides": IS, "storage_order": I},
                  required=("kernel_shape",)),
    "AveragePool": _s(1, 1, attrs={"auto_pad": S, "ceil_mode": I, "count_include_pad": I, "dilations": IS, "kernel_shape": IS, "pads": IS, "strides": IS},
                      required=("kernel_shape",)),
    "LpPool": _s(1, 1, attrs={"auto_pad": S, "ceil_mode": I, "dilations": IS, "kernel_shape": IS, "p": I, "pads": IS, "strides": IS}, required=("kernel_shape",)),
    "GlobalLpPool": _s(1, 1, attrs={"p": I}),
    "Resize": _s(1, 4, attrs={"antialias": I, "axes": IS, "coordinate_transformation_mode": S, "cubic_coeff_a": F, "exclude_outside": I,
                              "extrapolation_value": F, "keep_aspect_ratio_policy": S, "mode": S, "nearest_mode": S}),
    "GridSample": _s(2, 2, attrs={"align_corners": I, "mode": S, "padding_mode": S}),
    "BatchNormalization": _s(5, 5, 1, 5, attrs={"epsilon": F, "momentum": F, "training_mode": I, "spatial": I}),
    "InstanceNormalization": _s(3, 3, attrs={"epsilon": F}), "LayerNormalization": _s(2, 3, 1, 3, attrs={"axis": I, "epsilon": F, "stash_type": I}),
    "GroupNormalization": _s(3, 3, attrs={"epsilon": F, "num_groups": I, "stash_type": I}, required=("num_groups",)),
    "RMSNormalization": _s(2, 2, attrs={"axis": I, "epsilon": F, "stash_type": I}), "LRN": _s(1, 1, attrs={"alpha": F, "beta": F, "bias": F, "size": I}, required=("size",)),
    "LpNormalization": _s(1, 1, attrs={"axis": I, "p": I}), "MeanVarianceNormalization": _s(1, 1, attrs={"axes": IS}),
    "QuantizeLinear": _s(2, 3, attrs={"axis": I, "saturate": I, "block_size": I, "output_dtype": I, "precision": I}),
    "DequantizeLinear": _s(2, 3, attrs={"axis": I, "block_size": I, "output_dtype": I}), "DynamicQuantizeLinear": _s(1, 1, 3, 3),
    "RotaryEmbedding": _s(3, 4, attrs={"interleaved": I, "num_heads": I, "rotary_embedding_dim": I}),
    "Attention": _s(3, 7, 1, 4, attrs={"is_causal": I, "kv_num_heads": I, "q_num_heads": I, "qk_matmul_output_mode": I, "scale": F, "softcap": F,
                                       "softmax_precision": I}),
    "If": _s(1, 1, 0, INF, attrs={"then_branch": G, "else_branch": G}, required=("then_branch", "else_branch")),
    "Loop": _s(2, INF, 0, INF, attrs={"body": G}, required=("body",)),
    "Scan": _s(1, INF, 0, INF, attrs={"body": G, "num_scan_inputs": I, "scan_input_axes": IS, "scan_input_directions": IS, "scan_output_axes": IS,
                                       "scan_output_directions": IS}, required=("body", "num_scan_inputs")),
    "RandomNormal": _s(0, 0, attrs={"dtype": I, "mean": F, "scale": F, "seed": F, "shape": IS}, required=("shape",)),
    "RandomUniform": _s(0, 0, attrs={"dtype": I, "high": F, "low": F, "seed": F, "shape": IS}, required=("shape",)),
    "RandomNormalLike": _s(1, 1, attrs={"dtype": I, "mean": F, "scale": F, "seed": F}), "RandomUniformLike": _s(1, 1, attrs={"dtype": I, "high": F, "low": F, "seed": F}),
    "Bernoulli": _s(1, 1, attrs={"dtype": I, "seed": F}), "Multinomial": _s(1, 1, attrs={"dtype": I, "sample_size": I, "seed": F}),
    "DFT": _s(1, 3, attrs={"axis": I, "inverse": I, "onesided": I}), "STFT": _s(2, 4, attrs={"onesided": I}),
    "HannWindow": _s(1, 1, attrs={"output_datatype": I, "periodic": I}), "HammingWindow": _s(1, 1, attrs={"output_datatype": I, "periodic": I}),
    "BlackmanWindow": _s(1, 1, attrs={"output_datatype": I, "periodic": I}), "MelWeightMatrix": _s(5, 5, attrs={"output_datatype": I}),
    "Col2Im": _s(3, 3, attrs={"dilations": IS, "pads": IS, "strides": IS}), "CenterCropPad": _s(2, 2, attrs={"axes": IS}),
    "AffineGrid": _s(2, 2, attrs={"align_corners": I}), "Upsample": _s(1, 2, attrs={"mode": S, "scales": FS}),
    "TensorScatter": _s(2, 3, attrs={"axis": I, "mode": S}),
})

_KIND_OK = {
    I: lambda v: isinstance(v, (int, np.integer)) and not isinstance(v, bool),
    F: lambda v: isinstance(v, (float, int, np.floating, np.integer)) and not isinstance(v, bool),
    S: lambda v: isinstance(v, (str, bytes)),
    T: lambda v: isinstance(v, pb.Tensor),
    G: lambda v: isinstance(v, pb.Graph),
    IS: lambda v: isinstance(v, (list, tuple)) and all(isinstance(x, (int, np.integer)) for x in v),
    FS: lambda v: isinstance(v, (list, tuple)) and all(isinstance(x, (float, int, np.floating, np.integer)) for x in v),
    SS: lambda v: isinstance(v, (list, tuple)) and all(isinstance(x, (str, bytes)) for x in v),
}


def _check_graph(g, opsets, outer: set, problems: list, path: str, known_domains_only: bool):
    defined = set(outer)
    names_in = [vi.name for vi in g.inputs]
    for name in names_in:
        if not name:
            problems.append(Problem("error", path, "a graph input has an empty name"))
    dup = {n for n in names_in if names_in.count(n) > 1}
    for n in sorted(dup):
        problems.append(Problem("error", path, f"graph input '{n}' is declared twice"))
    defined |= set(names_in)
    for name, t in g.initializers.items():
        defined.add(name)
        arr = t.numpy()
        if arr is not None and t.data_type in pb._ITEM:
            want = int(np.prod([int(d) for d in t.dims], dtype=np.int64)) * pb._ITEM[t.data_type]
            have = int(np.asarray(arr).nbytes)
            if have != want:
                problems.append(Problem("error", f"{path}: initializer '{name}'", f"{have} bytes of data for dims {tuple(int(d) for d in t.dims)} "
                                        f"of element size {pb._ITEM[t.data_type]} ({want} bytes expected)"))
    produced_by: dict = {}
    all_outputs = {o for n in g.nodes for o in n.outputs if o}
    used = set()
    for idx, n in enumerate(g.nodes):
        where = f"{path}: node {idx} '{n.name or (n.outputs[0] if n.outputs else '')}' ({(n.domain + '::') if n.domain else ''}{n.op_type})"
        dom = n.domain or ""
        if dom not in opsets and not (dom == "" and "ai.onnx" in opsets):
            problems.append(Problem("error", where, f"domain '{dom or 'ai.onnx'}' has no opset import; the model imports {sorted(opsets) or 'nothing'}"))
        for i in n.inputs:
            if not i:
                continue
            used.add(i)
            if i not in defined:
                if i in all_outputs:
                    problems.append(Problem("warning", where, f"input '{i}' is produced by a later node: the node list is not in topological "
                                            "order (the executor sorts it; other runtimes may refuse)"))
                else:
                    problems.append(Problem("error", where, f"input '{i}' is not defined anywhere (no graph input, initializer or node output of that name)"))
        for o in n.outputs:
            if not o:
                continue
            if o in produced_by or o in names_in or o in g.initializers:
                problems.append(Problem("error", where, f"output '{o}' is already defined" + (f" by node '{produced_by[o]}'" if o in produced_by else
                                                                                           " as a graph input or initializer") + " (values are assigned once)"))
            produced_by[o] = n.name or o
        if not any(n.outputs):
            problems.append(Problem("error", where, "the node has no output"))
        if dom in ("", "ai.onnx"):
            sch = SCHEMAS.get(n.op_type)
            if sch is None:
                if known_domains_only:
                    problems.append(Problem("warning", where, "operator is not in the schema table: arity and attributes were not checked"))
            else:
                min_in, max_in, min_out, max_out, attrs, required = sch
                n_in = len(n.inputs)
                while n_in > 0 and not n.inputs[n_in - 1]:
                    n_in -= 1                           # trailing optional inputs left empty
                if not (min_in <= n_in <= max_in):
                    rng = f"{min_in}" if min_in == max_in else (f"at least {min_in}" if max_in >= INF else f"{min_in} to {max_in}")
                    problems.append(Problem("error", where, f"{n_in} input(s) given, the operator takes {rng}"))
                n_out = len([o for o in n.outputs if o])
                if not (min_out <= n_out <= max_out) and not (n_out == 0):
                    rng = f"{min_out}" if min_out == max_out else (f"at least {min_out}" if max_out >= INF else f"{min_out} to {max_out}")
                    problems.append(Problem("error", where, f"{n_out} output(s) given, the operator produces {rng}"))
                for r in required:
                    if r not in n.attrs:
                        problems.append(Problem("error", where, f"required attribute '{r}' is missing"))
                for k, v in n.attrs.items():
                    kind = attrs.get(k)
                    if kind is None:
                        problems.append(Problem("warning", where, f"attribute '{k}' is not one the operator declares"))
                    elif not _KIND_OK[kind](v) and not (kind in (IS, FS, SS) and isinstance(v, (list, tuple)) and len(v) == 0):
                        problems.append(Problem("error", where, f"attribute '{k}' should be of kind {kind}, found {type(v).__name__}"))
        for k, v in n.attrs.items():
            if isinstance(v, pb.Graph):
                _check_graph(v, opsets, defined | set(produced_by), problems, f"{where} / {k}", known_domains_only)
                used |= _free_names(v)
        defined |= {o for o in n.outputs if o}
    cyc = _cycle(g, all_outputs)
    if cyc:
        problems.append(Problem("error", path, "the nodes form a cycle through " + " -> ".join(f"'{c}'" for c in cyc)))
    for vo in g.outputs:
        if vo.name not in defined:
            problems.append(Problem("error", path, f"graph output '{vo.name}' is not produced by any node"))
        used.add(vo.name)
    for name in g.initializers:
        if name not in used and name not in names_in:
            problems.append(Problem("warning", f"{path}: initializer '{name}'", "nothing reads it"))


def _cycle(g, all_outputs) -> list:
    """Value names along one dependency cycle of the graph's own nodes (Kahn's algorithm leaves exactly the cyclic part), or []."""
    producer = {o: k for k, n in enumerate(g.nodes) for o in n.outputs if o}
    deps = [{producer[i] for i in n.inputs if i in all_outputs and i in producer} for n in g.nodes]
    users: list = [[] for _ in g.nodes]
    for k, d in enumerate(deps):
        for j in d:
            users[j].append(k)
    left = [len(d) for d in deps]
    ready = [k for k, c in enumerate(left) if c == 0]
    done = 0
    while ready:
        k = ready.pop()
        done += 1
        for u in users[k]:
            left[u] -= 1
            if left[u] == 0:
                ready.append(u)
    if done == len(g.nodes):
        return []
    stuck = {k for k, c in enumerate(left) if c > 0}
    k = min(stuck)
    seen, walk = {}, []
    while k not in seen:
        seen[k] = len(walk)
        walk.append(k)
        k = min(j for j in deps[k] if j in stuck)
    loop = walk[seen[k]:]
    return [next(o for o in g.nodes[j].outputs if o) for j in loop] + [next(o for o in g.nodes[loop[0]].outputs if o)]


def _free_names(graph) -> set:
    bound = {vi.name for vi in graph.inputs} | set(graph.initializers)
    free = set()
    for n in graph.nodes:
        free |= {i for i in n.inputs if i and i not in bound}
        for v in n.attrs.values():
            if isinstance(v, pb.Graph):
                free |= _free_names(v) - bound
        bound |= {o for o in n.outputs if o}
    return free


def check_model(model, warn_unknown_ops: bool = False) -> list:
    """Every problem found in ``model`` (a parsed :class:`onnx_pb.Model`); an empty list means it is well-formed."""
    problems: list = []
    opsets = dict(model.opsets or {})
    if not opsets:
        problems.append(Problem("error", "model", "no opset import: the operator set version is unknown"))
        opsets = {"": 0}
    for dom, ver in opsets.items():
        if not isinstance(ver, (int, np.integer)) or ver < 0:
            problems.append(Problem("error", "model", f"opset import for domain '{dom or 'ai.onnx'}' has version {ver!r}"))
    if model.ir_version is not None and int(model.ir_version) < 3:
        problems.append(Problem("warning", "model", f"ir_version {model.ir_version} predates initializers as optional inputs"))
    _check_graph(model.graph, opsets, set(), problems, f"graph '{model.graph.name}'", warn_unknown_ops)
    return problems


def errors(problems) -> list:
    return [p for p in problems if p.severity == "error"]
