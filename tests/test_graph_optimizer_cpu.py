"""Graph rewrites: every pass on a graph built for it, then the whole pipeline on the upstream fixtures, always comparing
the outputs of the rewritten graph with those of the original on the same inputs."""
import copy
import glob
import math
import os

import numpy as np
import pytest

from onnx_genai_b200.package import graph_optimizer as opt
from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package.graph_executor import GraphExecutor

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


def _t(name, arr, dt=None):
    arr = np.asarray(arr)
    if dt is None:
        dt = pb.INT64 if arr.dtype.kind == "i" else pb.FLOAT
    arr = arr.astype(np.int64 if dt == pb.INT64 else np.float32)
    return pb.Tensor(name=name, dims=tuple(arr.shape), data_type=dt, array=arr)


def _n(op, ins, outs, domain="", **attrs):
    return pb.Node(op_type=op, inputs=list(ins), outputs=list(outs), domain=domain, attrs=attrs)


def _model():
    rng = np.random.default_rng(1)
    g = pb.Graph(name="m")
    g.inputs = [pb.ValueInfo("x", pb.FLOAT, (6, 16))]
    init = {"w": rng.standard_normal((16, 16)) * 0.3, "b": rng.standard_normal(16), "gamma": rng.standard_normal(16), "beta": rng.standard_normal(16),
            "sqrt2": math.sqrt(2.0), "one": 1.0, "half": 0.5, "two": 2.0, "eps": 1e-5, "three": np.asarray([3], dtype=np.int64),
            "four": np.asarray([4], dtype=np.int64), "axm1": np.asarray([-1], dtype=np.int64), "unused": np.zeros(5)}
    g.initializers = {k: _t(k, v) for k, v in init.items()}
    g.nodes = [
        _n("Identity", ["x"], ["x1"]),
        _n("MatMul", ["x1", "w"], ["mm"]), _n("Add", ["mm", "b"], ["lin"]), _n("Relu", ["lin"], ["h"]),
        # erf GELU
        _n("Div", ["h", "sqrt2"], ["g1"]), _n("Erf", ["g1"], ["g2"]), _n("Add", ["g2", "one"], ["g3"]), _n("Mul", ["h", "g3"], ["g4"]),
        _n("Mul", ["g4", "half"], ["gelu"]),
        # layer norm
        _n("ReduceMean", ["gelu", "axm1"], ["mu"], keepdims=1), _n("Sub", ["gelu", "mu"], ["cen"]), _n("Pow", ["cen", "two"], ["sq"]),
        _n("ReduceMean", ["sq", "axm1"], ["var"], keepdims=1), _n("Add", ["var", "eps"], ["ve"]), _n("Sqrt", ["ve"], ["sd"]),
        _n("Div", ["cen", "sd"], ["nrm"]), _n("Mul", ["nrm", "gamma"], ["sc"]), _n("Add", ["sc", "beta"], ["ln"]),
        # shape arithmetic on constants, a no-op reshape, two transposes, a dead branch
        _n("Shape", ["ln"], ["shp"]), _n("Mul", ["three", "four"], ["twelve"]), _n("Cast", ["ln"], ["ln_f"], to=pb.FLOAT),
        _n("Reshape", ["ln_f", "shp"], ["same"]), _n("Transpose", ["same"], ["t1"], perm=[1, 0]), _n("Transpose", ["t1"], ["t2"], perm=[1, 0]),
        _n("Transpose", ["t2"], ["y"], perm=[1, 0]),
        _n("Exp", ["x"], ["dead1"]), _n("Neg", ["dead1"], ["dead2"]),
    ]
    g.outputs = [pb.ValueInfo("y", pb.FLOAT, (16, 6))]
    return pb.Model(graph=g)


def test_every_pass_fires_and_the_graph_computes_the_same():
    model = _model()
    x = np.random.default_rng(0).standard_normal((6, 16)).astype(np.float32)
    want = GraphExecutor(copy.deepcopy(model), "cpu").run({"x": x})["y"].numpy()
    rep = opt.optimize(model)
    ops = [n.op_type for n in model.graph.nodes]
    assert sorted(ops) == sorted(["FusedGemm", "Gelu", "LayerNormalization", "Transpose"]), ops
    assert rep.nodes_before == 27 and rep.nodes_after == 4 and rep.rounds >= 2
    for name in ("fold_constants", "eliminate_identities", "merge_transposes", "fuse_patterns", "eliminate_dead_nodes"):
        assert rep.changes.get(name, 0) > 0, (name, rep.changes)
    assert "unused" not in model.graph.initializers and "twelve" not in model.graph.initializers
    got = GraphExecutor(model, "cpu").run({"x": x})["y"].numpy()
    assert np.allclose(got, want, atol=1e-5)
    assert [vo.name for vo in model.graph.outputs] == ["y"] and [vi.name for vi in model.graph.inputs] == ["x"]


def test_patterns_are_left_alone_when_an_intermediate_is_read_elsewhere():
    model = _model()
    model.graph.outputs.append(pb.ValueInfo("g3", pb.FLOAT, (6, 16)))       # the inside of the GELU chain is an output
    model.graph.outputs.append(pb.ValueInfo("cen", pb.FLOAT, (6, 16)))      # and so is the centred value of the layer norm
    x = np.random.default_rng(0).standard_normal((6, 16)).astype(np.float32)
    want = GraphExecutor(copy.deepcopy(model), "cpu").run({"x": x})
    opt.optimize(model)
    ops = [n.op_type for n in model.graph.nodes]
    assert "Gelu" not in ops and "LayerNormalization" not in ops and "Erf" in ops
    got = GraphExecutor(model, "cpu").run({"x": x})
    for k in ("y", "g3", "cen"):
        assert np.allclose(got[k].numpy(), want[k].numpy(), atol=1e-5)


def test_optimized_upstream_fixtures_compute_what_the_originals_compute():
    from onnx_genai_b200.package.onnx_text import load_any

    paths = sorted(glob.glob(os.path.join(REF, "crates", "onnx-runtime-ep-cpu-plugin", "tests", "fixtures", "*", "model.onnx.textproto")))
    paths += sorted(glob.glob(os.path.join(REF, "tests", "fixtures", "tiny-llm*", "*.onnx.textproto")))
    if not paths:
        pytest.skip("upstream fixtures not available")
    rng = np.random.default_rng(0)
    ran = removed = 0
    for path in paths:
        model = load_any(path)
        g = model.graph
        if any(not all(isinstance(d, int) for d in vi.shape) for vi in g.inputs if vi.name not in g.initializers):
            continue
        if any(n.op_type.startswith("Random") or n.op_type in ("Bernoulli", "Multinomial") for n in g.nodes):
            continue
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
        want = GraphExecutor(copy.deepcopy(model), "cpu").run(feeds)
        rep = opt.optimize(model)
        got = GraphExecutor(model, "cpu").run(feeds)
        for vo in g.outputs:
            a, b = want[vo.name], got[vo.name]
            assert tuple(a.shape) == tuple(b.shape), (path, vo.name)
            assert np.allclose(a.float().numpy(), b.float().numpy(), atol=1e-5, equal_nan=True), (path, vo.name, rep.changes)
        ran += 1
        removed += rep.nodes_before - rep.nodes_after
    assert ran >= 10, ran
