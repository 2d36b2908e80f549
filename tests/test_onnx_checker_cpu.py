"""Model checker: every upstream text fixture is well-formed, and each kind of malformation is named with its node."""
import copy
import glob
import os

import numpy as np
import pytest

from onnx_genai_b200.package import onnx_checker as ck
from onnx_genai_b200.package import onnx_pb as pb

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


def _n(op, ins, outs, domain="", **attrs):
    return pb.Node(op_type=op, inputs=list(ins), outputs=list(outs), domain=domain, attrs=attrs, name=outs[0] + "_node")


def _good():
    g = pb.Graph(name="g")
    g.inputs = [pb.ValueInfo("x", pb.FLOAT, (2, 4))]
    w = np.ones((4, 4), dtype=np.float32)
    g.initializers = {"w": pb.Tensor(name="w", dims=(4, 4), data_type=pb.FLOAT, array=w)}
    g.nodes = [_n("MatMul", ["x", "w"], ["y"]), _n("Relu", ["y"], ["z"]), _n("Concat", ["z", "y"], ["out"], axis=1)]
    g.outputs = [pb.ValueInfo("out", pb.FLOAT, (2, 8))]
    return pb.Model(graph=g, opsets={"": 21})


def test_a_well_formed_model_has_no_problems():
    assert ck.check_model(_good()) == []


@pytest.mark.parametrize("mutate,needle", [
    (lambda m: m.graph.nodes[0].inputs.__setitem__(0, "z"), "the nodes form a cycle through 'y' -> 'z' -> 'y'"),
    (lambda m: m.graph.nodes[1].inputs.__setitem__(0, "ghost"), "'ghost' is not defined anywhere"),
    (lambda m: m.graph.nodes[1].outputs.__setitem__(0, "y"), "output 'y' is already defined"),
    (lambda m: m.graph.nodes[2].attrs.pop("axis"), "required attribute 'axis' is missing"),
    (lambda m: m.graph.nodes[2].attrs.__setitem__("axis", "one"), "attribute 'axis' should be of kind int"),
    (lambda m: m.graph.nodes[1].inputs.append("y"), "2 input(s) given, the operator takes 1"),
    (lambda m: m.graph.nodes.append(_n("Gelu", ["z"], ["q"], domain="com.microsoft")), "domain 'com.microsoft' has no opset import"),
    (lambda m: m.graph.outputs.append(pb.ValueInfo("nope", pb.FLOAT, (1,))), "graph output 'nope' is not produced"),
    (lambda m: setattr(m.graph.initializers["w"], "dims", (4, 5)), "64 bytes of data for dims (4, 5)"),
    (lambda m: m.opsets.clear(), "no opset import"),
])
def test_each_malformation_is_reported_with_its_place(mutate, needle):
    m = _good()
    mutate(m)
    text = "\n".join(str(p) for p in ck.errors(ck.check_model(m)))
    assert needle in text, text


def test_an_unsorted_node_list_is_a_warning_because_the_executor_sorts_it():
    m = _good()
    m.graph.nodes.reverse()
    ps = ck.check_model(m)
    assert ck.errors(ps) == [] and any("not in topological order" in str(p) for p in ps)


def test_warnings_do_not_count_as_errors_and_subgraphs_see_the_outer_scope():
    m = _good()
    m.graph.initializers["spare"] = pb.Tensor(name="spare", dims=(1,), data_type=pb.FLOAT, array=np.zeros(1, dtype=np.float32))
    m.graph.nodes[1].attrs["fancy"] = 3
    body = pb.Graph(name="then", nodes=[_n("Add", ["z", "y"], ["t"])], outputs=[pb.ValueInfo("t", pb.FLOAT, (2, 4))])
    other = pb.Graph(name="else", nodes=[_n("Sub", ["z", "missing"], ["e"])], outputs=[pb.ValueInfo("e", pb.FLOAT, (2, 4))])
    m.graph.inputs.append(pb.ValueInfo("c", pb.BOOL, ()))
    m.graph.nodes.append(_n("If", ["c"], ["branch"], then_branch=body, else_branch=other))
    ps = ck.check_model(m)
    warn = [str(p) for p in ps if p.severity == "warning"]
    assert any("'spare'" in w and "nothing reads it" in w for w in warn) and any("attribute 'fancy'" in w for w in warn)
    errs = [str(p) for p in ck.errors(ps)]
    assert len(errs) == 1 and "else_branch" in errs[0] and "'missing' is not defined" in errs[0]      # z and y come from the outer graph


def test_every_upstream_text_fixture_is_well_formed():
    from onnx_genai_b200.package.onnx_text import TextFormatError, load_any

    paths = sorted(glob.glob(os.path.join(REF, "**", "*.onnx.textproto"), recursive=True))
    if not paths:
        pytest.skip("upstream fixtures not available")
    checked = 0
    for path in paths:
        try:
            model = load_any(path)
        except TextFormatError:
            continue                                    # a placeholder file of a packaging fixture, not a model
        errs = ck.errors(ck.check_model(model))
        assert errs == [], (path, [str(e) for e in errs][:3])
        checked += 1
    assert checked >= 100
