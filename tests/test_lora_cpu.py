"""Per-row low-rank parameter overlays: weight formats, heterogeneous batches, the adapter cache, the workflow binding."""
import json
import os

import numpy as np
import pytest
import torch
import yaml

from onnx_genai_b200.engine.lora import AdapterError, AdapterStore, parameter_overlay_adapter
from onnx_genai_b200.engine.workflow_runtime import WorkflowRuntimeError, WorkflowSession
from onnx_genai_b200.package import onnx_pb as pb

FIXTURES = os.path.join(os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference")),
                        "tests", "fixtures", "onnx_genai_workflows")
N_IN, N_OUT, RANK = 6, 4, 2


def _package(tmp_path, rng):
    w = rng.standard_normal((N_IN, N_OUT)).astype(np.float32)
    g = pb.Graph(name="g", nodes=[pb.Node("MatMul", ["x", "proj"], ["y"], name="proj")],
                 initializers={"proj": pb.Tensor(name="proj", dims=w.shape, data_type=pb.FLOAT, array=w)},
                 inputs=[pb.ValueInfo("x", pb.FLOAT, ("b", N_IN))], outputs=[pb.ValueInfo("y", pb.FLOAT, ("b", N_OUT))])
    pb.save_model(pb.Model(graph=g), str(tmp_path / "model.onnx"), external_data=False)
    adapters = {}
    for name in ("one", "two", "three"):
        a, b = rng.standard_normal((RANK, N_IN)).astype(np.float32), rng.standard_normal((RANK, N_OUT)).astype(np.float32)
        adapters[name] = (a, b)
        os.makedirs(tmp_path / "adapters" / name)
        if name == "three":      # the same content in the PEFT layout: lora_A [rank, in], lora_B [out, rank]
            from safetensors.torch import save_file

            save_file({"base_model.model.layers.0.proj.lora_A.weight": torch.from_numpy(a),
                       "base_model.model.layers.0.proj.lora_B.weight": torch.from_numpy(b.T.copy())}, str(tmp_path / "adapters" / name / "adapter_model.safetensors"))
        else:
            (tmp_path / "adapters" / name / "adapter.json").write_text(json.dumps({"targets": {"proj": {"a": a.reshape(-1).tolist(), "b": b.reshape(-1).tolist()}}}))
    tensor = lambda dtype, shape: {"contract": {"dtype": dtype, "rank": len(shape), "shape": shape, "batch_layout": {"kind": "request_aligned", "axis": 0}}}
    doc = {"pipeline": {"workflow": {
        "inputs": {"x": {**tensor("float32", ["batch", N_IN]), "source": {"kind": "application"}, "required": True},
                   "sel.segments": {**tensor("int64", ["batch", 2]), "source": {"kind": "request"}},
                   "sel.counts": {**tensor("int64", ["batch"]), "source": {"kind": "request"}},
                   "sel.scales": {**tensor("float32", ["batch", 2]), "source": {"kind": "request"}}},
        "outputs": {"y": tensor("float32", ["batch", N_OUT])},
        "components": {"decoder": {"implementation": {"kind": "onnx", "artifact": "model.onnx"}},
                       "overlay": {"implementation": {"kind": "adapter", "abi": "onnx-genai.parameter-overlay", "version": "1"},
                                   "ports": {"inputs": {"input": {"dtype": "float32", "rank": 2}}, "outputs": {"output": {"dtype": "float32", "rank": 2}}},
                                   "contract": {"parameters": {"action": "apply", "component": "decoder", "parameter": "proj"}}}},
        "steps": [{"kind": "invoke", "component": "overlay", "inputs": {"input": "x"}, "outputs": {"output": "adapted"}},
                  {"kind": "emit", "value": "adapted", "output": "y", "mode": "replace"}]}},
        "adapters": {"target_manifest": {"targets": [{"id": "proj", "component": "decoder", "initializer": "proj", "input_features": N_IN,
                                                       "output_features": N_OUT, "rank": RANK, "alpha": 4.0}]},
                     "selection": {"segments": "sel.segments", "adapter_counts": "sel.counts", "scales": "sel.scales", "max_adapters": 2},
                     "cache": {"max_entries": 2},
                     "artifacts": {name: {"index": i, "rank": RANK, "alpha": 4.0,
                                          "weights": [{"location": f"adapters/{name}/" + ("adapter_model.safetensors" if name == "three" else "adapter.json"),
                                                       "format": "hf_peft" if name == "three" else "json", "scale_encoding": "alpha_over_rank"}],
                                          "bindings": [{"target": "proj", "weight_key": "proj"}]} for i, name in enumerate(("one", "two", "three"))}}}
    (tmp_path / "inference_metadata.yaml").write_text(yaml.safe_dump(doc, sort_keys=False))
    return w, adapters


def test_heterogeneous_rows_formats_cache_and_errors(tmp_path):
    rng = np.random.default_rng(0)
    w, ad = _package(tmp_path, rng)
    sess = WorkflowSession.from_package(str(tmp_path))
    x = torch.from_numpy(rng.standard_normal((4, N_IN)).astype(np.float32))
    seg = torch.tensor([[0, -1], [-1, -1], [2, 1], [1, -1]])
    counts, scales = torch.tensor([1, 0, 2, 1]), torch.tensor([[1.0, 0.0], [0.0, 0.0], [0.5, 2.0], [1.0, 0.0]])
    got = sess.run({"x": x, "sel.segments": seg, "sel.counts": counts, "sel.scales": scales})["y"]
    names = ["one", "two", "three"]
    want = x @ torch.from_numpy(w)
    for row in range(4):
        for j in range(int(counts[row])):
            a, b = ad[names[int(seg[row, j])]]
            want[row] += float(scales[row, j]) * (4.0 / RANK) * (x[row] @ torch.from_numpy(a).T) @ torch.from_numpy(b)
    assert torch.allclose(got, want, atol=1e-5)
    store = sess.components["overlay"].store
    assert store.loads == 3 and store.evictions == 1 and len(store.cache) == 2          # three adapters through a cache of two
    # the selection is positional: the same rows alone, or reordered, give the same rows
    alone = sess.run({"x": x[2:3], "sel.segments": seg[2:3], "sel.counts": counts[2:3], "sel.scales": scales[2:3]})["y"]
    assert torch.allclose(alone[0], want[2], atol=1e-5)
    # no selection supplied: the base projection
    assert torch.allclose(sess.run({"x": x})["y"], x @ torch.from_numpy(w), atol=1e-6)
    with pytest.raises(AdapterError, match="adapter index 7 is not in the package"):
        sess.run({"x": x[:1], "sel.segments": torch.tensor([[7, -1]]), "sel.counts": torch.tensor([1]), "sel.scales": torch.ones(1, 2)})
    with pytest.raises(AdapterError, match="slot 1 is empty"):
        sess.run({"x": x[:1], "sel.segments": torch.tensor([[0, -1]]), "sel.counts": torch.tensor([2]), "sel.scales": torch.ones(1, 2)})
    os.remove(tmp_path / "adapters" / "one" / "adapter.json")
    store.cache.clear()
    with pytest.raises(AdapterError, match="no readable weights: adapters/one/adapter.json does not exist"):
        sess.run({"x": x[:1], "sel.segments": torch.tensor([[0, -1]]), "sel.counts": torch.tensor([1]), "sel.scales": torch.ones(1, 2)})


def test_binding_errors_name_the_problem(tmp_path):
    _package(tmp_path, np.random.default_rng(1))
    doc = yaml.safe_load((tmp_path / "inference_metadata.yaml").read_text())
    doc["pipeline"]["workflow"]["components"]["overlay"]["contract"]["parameters"]["parameter"] = "gate"
    (tmp_path / "inference_metadata.yaml").write_text(yaml.safe_dump(doc, sort_keys=False))
    with pytest.raises(WorkflowRuntimeError, match="overlays parameter 'gate', which the adapter target manifest does not list"):
        WorkflowSession.from_package(str(tmp_path))


@pytest.mark.skipif(not os.path.isdir(FIXTURES), reason="the upstream workflow fixtures are not available on this machine")
def test_upstream_adapter_package_gives_the_upstream_numbers():
    sess = WorkflowSession.from_package(os.path.join(FIXTURES, "adapter"))
    idx = {a["name"]: i for i, a in sess.components["overlay"].store.by_index.items()}
    x = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    out = sess.run({"activations": x, "request.active": torch.tensor([True, True, True]),
                    "request.adapter_segments": torch.tensor([[idx["red"], -1], [-1, -1], [idx["red"], idx["blue"]]]),
                    "request.adapter_counts": torch.tensor([1, 0, 2]), "request.adapter_scales": torch.tensor([[1.0, 0.0], [0.0, 0.0], [0.5, 1.0]])})
    assert out["result"].tolist() == [[2.0, 4.0], [3.0, 4.0], [25.5, 35.0]]
    out = sess.run({"activations": x[:1], "request.active": torch.tensor([False]), "request.adapter_segments": torch.tensor([[idx["blue"], -1]]),
                    "request.adapter_counts": torch.tensor([1]), "request.adapter_scales": torch.ones(1, 2)})
    assert out["result"].tolist() == [[1.0, 2.0]]                      # an inactive row keeps the base projection
