"""The static memory plan of interpreted graphs (package/memory_plan.py) and the executor's lifetime-based release."""
import glob
import os

import numpy as np
import pytest
import torch

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package import onnx_text
from onnx_genai_b200.package.graph_executor import GraphExecutor
from onnx_genai_b200.package.memory_plan import lifetimes, plan_memory

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))

CHAIN = """
ir_version: 8
opset_import { domain: "" version: 17 }
graph {
  name: "chain"
  input { name: "x" type { tensor_type { elem_type: 1 shape { dim { dim_param: "n" } dim { dim_value: 64 } } } } }
  output { name: "y" type { tensor_type { elem_type: 1 shape { dim { dim_param: "n" } dim { dim_value: 64 } } } } }
  node { op_type: "Relu" input: "x" output: "a" }
  node { op_type: "Sigmoid" input: "a" output: "b" }
  node { op_type: "Reshape" input: "b" input: "shape" output: "b_view" }
  node { op_type: "Tanh" input: "b" output: "c" }
  node { op_type: "Neg" input: "c" output: "d" }
  node { op_type: "Reshape" input: "b_view" input: "shape2" output: "b_back" }
  node { op_type: "Add" input: "d" input: "b_back" output: "e" }
  node { op_type: "Mul" input: "e" input: "a" output: "y" }
  initializer { name: "shape" data_type: 7 dims: 2 int64_data: 64 int64_data: -1 }
  initializer { name: "shape2" data_type: 7 dims: 2 int64_data: -1 int64_data: 64 }
}
"""


def test_lifetimes_views_and_the_arena_on_a_small_chain():
    model = onnx_text.parse_model_text(CHAIN)
    plan = plan_memory(model, symbols={"n": 100}, alignment=1)
    row = 100 * 64 * 4
    v = plan.values
    assert v["b_view"].alias_of == "b" and v["b_back"].alias_of == "b" and v["b_view"].bytes == 0
    assert v["b"].dies == v["b_back"].dies                      # the view read by Add keeps b alive until then
    assert v["a"].dies == len(plan.order) - 1 and v["y"].dies == len(plan.order)
    assert plan.naive_bytes == 6 * row                          # a b c d e y
    assert plan.lower_bound_bytes == 4 * row                    # at Add: a, b (through its view), d, e
    assert plan.arena_bytes == plan.lower_bound_bytes and plan.efficiency == 1.0
    plan.check()
    unbound = plan_memory(model)                                # n left symbolic: nothing can be sized, nothing is guessed
    assert unbound.arena_bytes == 0 and set(unbound.unsized) >= {"a", "b", "c"}


def test_executor_release_holds_the_live_set_and_computes_the_same(tmp_path):
    model = onnx_text.parse_model_text(CHAIN)
    x = torch.randn(100, 64)
    keep = GraphExecutor(model).run({"x": x})["y"]
    ex = GraphExecutor(model, release=True)
    got = ex.run({"x": x})["y"]
    assert torch.equal(got, keep)
    row = 100 * 64 * 4
    assert ex.peak_live_bytes == 4 * row                        # the plan's lower bound, measured on real storages
    order, born, last = lifetimes(model, ex.order)
    assert last["c"] == born["d"] and last["y"] == len(order)


def test_upstream_graphs_plan_within_a_few_percent_of_the_bound_and_release_changes_nothing():
    paths = sorted(glob.glob(os.path.join(REF, "crates", "onnx-runtime-ep-cpu-plugin", "tests", "fixtures", "*", "model.onnx.textproto")))
    if not paths:
        pytest.skip("upstream fixtures not available")
    planned = 0
    for path in paths:
        model = onnx_text.load_model_text(path)
        try:
            ex = GraphExecutor(model, release=True)
        except Exception:
            continue
        feeds, shapes = {}, {}
        rng = np.random.default_rng(0)
        ok = True
        for vi in model.graph.inputs:
            if vi.name in model.graph.initializers:
                continue
            dims = [d if isinstance(d, int) and d > 0 else 3 for d in (vi.shape or [])]
            shapes[vi.name] = dims
            np_dtype = pb._NP.get(vi.elem_type)
            if np_dtype is None:
                ok = False
                break
            feeds[vi.name] = (rng.standard_normal(dims).astype(np_dtype) if np.issubdtype(np_dtype, np.floating)
                              else rng.integers(0, 2, size=dims).astype(np_dtype))
        if not ok:
            continue
        plan = plan_memory(model, input_shapes=shapes)
        plan.check()
        if plan.arena_bytes:
            planned += 1
            assert plan.lower_bound_bytes <= plan.arena_bytes <= plan.naive_bytes
            assert plan.efficiency > 0.6, (path, plan.summary())
        try:
            want = GraphExecutor(model).run(feeds)
        except Exception:
            continue                                            # the fixture needs particular input values: not this test's subject
        got = ex.run(feeds)
        for name in want:
            a, b = want[name], got[name]
            assert a.shape == b.shape and torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float())), (path, name)
    assert planned >= 5
