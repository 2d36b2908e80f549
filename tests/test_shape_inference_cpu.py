"""Symbolic shape inference: dimension arithmetic, shape-data chains, operator rules against executed shapes."""
import glob
import os

import numpy as np
import pytest

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package import shape_inference as si
from onnx_genai_b200.package.shape_inference import Dim

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


def test_dimension_arithmetic():
    b, s = Dim.of("batch"), Dim.of("seq")
    assert (b * 4 + s - s).lower() == "4*batch"
    assert ((b * s * 64).exact_div(b * 64)) == s
    assert (b * 6).exact_div(4) is None and (b * 6).exact_div(3) == b * 2
    assert (s + 3 - 3) == "seq" and (Dim.of(7) * 3).lower() == 21
    assert (b * s + 2 * b).lower() in ("2*batch + batch*seq",)
    assert hash(b * s) == hash(s * b)


def _node(op, ins, outs, domain="", **attrs):
    return pb.Node(op_type=op, inputs=list(ins), outputs=list(outs), domain=domain, attrs=attrs)


def _const(name, values, dtype=np.int64):
    arr = np.asarray(values, dtype=dtype)
    return pb.Tensor(name=name, dims=tuple(arr.shape), data_type=pb.INT64 if dtype == np.int64 else pb.FLOAT, array=arr)


def test_transformer_reshape_chain_resolves_with_symbolic_batch_and_sequence():
    """x [batch, seq, 64] -> Shape -> Gather / Slice -> Concat -> Reshape to [batch, seq, 4, 16] -> Transpose; then the
    inverse Reshape with -1, whose extent cancels back to 64."""
    g = pb.Graph(name="t")
    g.inputs = [pb.ValueInfo("x", pb.FLOAT, ("batch", "seq", 64))]
    g.initializers = {"i0": _const("i0", [0]), "i1": _const("i1", [1]), "i2": _const("i2", [2]), "hd": _const("hd", [4, 16]),
                      "zero": _const("zero", 0), "back": _const("back", [0, 0, -1])}
    g.nodes = [
        _node("Shape", ["x"], ["shp"]),
        _node("Slice", ["shp", "i0", "i2"], ["bs"]),
        _node("Concat", ["bs", "hd"], ["target"], axis=0),
        _node("Reshape", ["x", "target"], ["split"]),
        _node("Transpose", ["split"], ["heads"], perm=[0, 2, 1, 3]),
        _node("Transpose", ["heads"], ["unheads"], perm=[0, 2, 1, 3]),
        _node("Reshape", ["unheads", "back"], ["merged"]),
        _node("Gather", ["shp", "zero"], ["b_scalar"], axis=0),
        _node("Unsqueeze", ["b_scalar", "i0"], ["b_vec"]),
        _node("MatMul", ["heads", "heads_t"], ["scores"]),
        _node("Transpose", ["heads"], ["heads_t"], perm=[0, 1, 3, 2]),
        _node("Softmax", ["scores"], ["probs"], axis=-1),
        _node("ReduceSum", ["probs", "i1"], ["summed"], keepdims=0),
    ]
    g.outputs = [pb.ValueInfo("merged", pb.FLOAT, (None, None, None)), pb.ValueInfo("summed", pb.FLOAT, None)]
    r = si.infer(pb.Model(graph=g))
    assert r.shape("split") == ["batch", "seq", 4, 16]
    assert r.shape("heads") == ["batch", 4, "seq", 16]
    assert r.shape("merged") == ["batch", "seq", 64]
    assert r.shape("scores") == ["batch", 4, "seq", "seq"] and r.shape("summed") == ["batch", "seq", "seq"]
    assert r.shape("b_vec") == [1] and r.fully_resolved, r.unresolved
    assert r.fresh_symbols == 0
    concrete = si.infer(pb.Model(graph=g), input_shapes={"x": [2, 5, 64]})
    assert concrete.shape("merged") == [2, 5, 64] and concrete.shape("scores") == [2, 4, 5, 5]


def test_unregistered_operators_and_policies():
    g = pb.Graph(name="t")
    g.inputs = [pb.ValueInfo("x", pb.FLOAT, (2, 3)), pb.ValueInfo("y", pb.FLOAT, (4, 3))]
    g.nodes = [_node("FancyOp", ["x"], ["z"], domain="vendor"), _node("Relu", ["z"], ["w"]), _node("Add", ["x", "y"], ["bad"]),
               _node("NonZero", ["x"], ["nz"])]
    g.outputs = [pb.ValueInfo("w", pb.FLOAT, None)]
    r = si.infer(pb.Model(graph=g))
    assert r.unregistered == {"vendor::FancyOp": 1} and "z" in r.unresolved and "w" in r.unresolved
    assert r.shape("nz")[0] == 2 and isinstance(r.shape("nz")[1], str) and r.fresh_symbols == 1
    with pytest.raises(si.ShapeInferenceError, match="broadcast"):
        si.infer(pb.Model(graph=g), policy="strict")


def _random_feeds(g, rng):
    feeds = {}
    for vi in g.inputs:
        if vi.name in g.initializers:
            continue
        npdt = np.dtype(pb._NP[vi.elem_type])
        if vi.name == "cumulative_sequence_length":
            feeds[vi.name] = np.asarray([0, 8][: vi.shape[0]], dtype=npdt)
        elif np.issubdtype(npdt, np.floating):
            feeds[vi.name] = rng.standard_normal(vi.shape).astype(npdt)
        elif npdt == np.bool_:
            feeds[vi.name] = rng.integers(0, 2, vi.shape).astype(bool)
        else:
            feeds[vi.name] = rng.integers(0, 2, vi.shape).astype(npdt)
    return feeds


def test_inferred_shapes_agree_with_executed_shapes_on_the_upstream_operator_fixtures():
    """Every value the pass resolves to concrete extents must have exactly those extents when the graph is run."""
    from onnx_genai_b200.package.graph_executor import GraphExecutor
    from onnx_genai_b200.package.onnx_text import load_any

    paths = sorted(glob.glob(os.path.join(REF, "crates", "onnx-runtime-ep-cpu-plugin", "tests", "fixtures", "*", "model.onnx.textproto")))
    if not paths:
        pytest.skip("upstream fixtures not available")
    rng = np.random.default_rng(0)
    checked = resolved_outputs = graphs = 0
    for path in paths:
        model = load_any(path)
        g = model.graph
        if any(not all(isinstance(d, int) for d in vi.shape) for vi in g.inputs if vi.name not in g.initializers):
            continue
        report = si.infer(model)
        names = [o for n in g.nodes for o in n.outputs if o]
        ex = GraphExecutor(model, "cpu")
        out = ex.run(_random_feeds(g, rng), outputs=names)
        graphs += 1
        for name in names:
            shape = report.shape(name)
            if shape is None or name not in out or not hasattr(out[name], "shape"):
                continue
            assert len(shape) == out[name].dim(), (path, name, shape, tuple(out[name].shape))
            for want, got in zip(shape, out[name].shape):
                if isinstance(want, int):
                    assert want == got, (path, name, shape, tuple(out[name].shape))
                    checked += 1
        resolved_outputs += sum(1 for vo in g.outputs if report.types[vo.name].resolved)
    assert graphs >= 10 and checked > 100 and resolved_outputs >= graphs // 2, (graphs, checked, resolved_outputs)


def test_exported_decoder_resolves_fully(tmp_path):
    from onnx_genai_b200.bench.config_bench import _export
    from onnx_genai_b200.package.onnx_pb import load_model

    _export("tiny-llama", str(tmp_path), "fp32", layers=2)
    model = load_model(str(tmp_path / "decoder.onnx"))
    r = si.infer(model)
    assert not r.unregistered, r.unregistered
    logits = r.shape("logits")
    assert logits is not None and logits[-1] == 32000 and logits[0] is not None and logits[1] is not None
    present = r.shape("present.0.key")
    assert present is not None and present[1] == 2 and present[3] == 32 and isinstance(present[2], str) and "+" in present[2]
    assert r.fully_resolved, r.unresolved[:10]
