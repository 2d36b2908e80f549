"""Protobuf text format reader for ONNX models."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package.graph_executor import GraphExecutor
from onnx_genai_b200.package.onnx_text import TextFormatError, load_any, parse_model_text, parse_text

TEXT = r'''
# a two-node graph: y = relu(x @ w + b), w as raw bytes, b as float_data
ir_version: 10
producer_name: "hand"
opset_import { domain: "" version: 21 }
metadata_props { key: "note" value: "text \"quoted\"" }
graph {
  name: "tiny"
  node { input: "x" input: "w" output: "xw" op_type: "MatMul" name: "mm" }
  node {
    input: "xw" input: "b" output: "s" op_type: "Add"
  }
  node { input: "s" output: "y" op_type: "LeakyRelu" attribute { name: "alpha" f: 0.5 type: FLOAT } }
  node { output: "c" op_type: "Constant" attribute { name: "value_ints" ints: [1, 2, 3] type: INTS } }
  initializer {
    dims: 2 dims: 2 data_type: 1 name: "w"
    raw_data: "\000\000\200?\000\000\000@\000\000@@\000\000\200@"
  }
  initializer { dims: 2 data_type: FLOAT float_data: -10.0 float_data: 0.5 name: "b" }
  input { name: "x" type { tensor_type { elem_type: 1 shape { dim { dim_param: "n" } dim { dim_value: 2 } } } } }
  output { name: "y" type { tensor_type { elem_type: 1 } } }
  output { name: "c" type { tensor_type { elem_type: 7 } } }
}
'''


def test_text_model_parses_and_runs():
    m = parse_model_text(TEXT)
    assert m.ir_version == 10 and m.producer_name == "hand" and m.opsets == {"": 21} and m.metadata == {"note": 'text "quoted"'}
    g = m.graph
    assert [n.op_type for n in g.nodes] == ["MatMul", "Add", "LeakyRelu", "Constant"] and g.nodes[2].attrs == {"alpha": 0.5}
    assert g.nodes[3].attrs["value_ints"] == [1, 2, 3]
    assert g.initializers["w"].array.tolist() == [[1.0, 2.0], [3.0, 4.0]] and g.inputs[0].shape == ("n", 2)
    out = GraphExecutor(m).run({"x": torch.tensor([[1.0, 1.0]])})
    assert out["y"].tolist() == [[-3.0, 6.5]] and out["c"].tolist() == [1, 2, 3]


def test_text_and_binary_forms_agree(tmp_path):
    m = parse_model_text(TEXT)
    path = str(tmp_path / "m.onnx")
    pb.save_model(m, path, external_data=False)
    (tmp_path / "m.onnx.textproto").write_text(TEXT)
    a, b = load_any(path), load_any(str(tmp_path / "m.onnx.textproto"))
    x = torch.randn(3, 2)
    assert torch.equal(GraphExecutor(a).run({"x": x})["y"], GraphExecutor(b).run({"x": x})["y"])


def test_text_syntax_corners_and_errors():
    msg = parse_text('a: 1 a: 2 b { c: "x" "y" d: [1.5, -2e1] } e: < f: true > g: 0x10 h: -inf i: SOME_ENUM j: \'\\x41\\102\'')
    assert msg["a"] == [1, 2] and msg["b"][0]["c"] == [b"xy"] and msg["b"][0]["d"] == [1.5, -20.0]
    assert msg["e"][0]["f"] == [True] and msg["g"] == [16] and msg["h"] == [float("-inf")] and msg["i"] == ["SOME_ENUM"] and msg["j"] == [b"AB"]
    with pytest.raises(TextFormatError, match="closing brace is missing"):
        parse_text("a { b: 1")
    with pytest.raises(TextFormatError, match="no `graph"):
        parse_model_text("ir_version: 3")
    with pytest.raises(TextFormatError, match="unknown tensor data type"):
        parse_model_text('graph { initializer { data_type: QUATERNION name: "q" } }')


def test_external_tensor_data_is_resolved_against_the_file(tmp_path):
    np.arange(6, dtype=np.float32).tofile(tmp_path / "w.bin")
    text = """graph { node { input: "x" input: "w" output: "y" op_type: "Add" }
      initializer { dims: 2 data_type: 1 name: "w" data_location: EXTERNAL
        external_data { key: "location" value: "w.bin" } external_data { key: "offset" value: "8" } }
      input { name: "x" type { tensor_type { elem_type: 1 } } } output { name: "y" type { tensor_type { elem_type: 1 } } } }"""
    (tmp_path / "m.onnx.textproto").write_text(text)
    m = load_any(str(tmp_path / "m.onnx.textproto"))
    assert m.graph.initializers["w"].array.tolist() == [2.0, 3.0]
    with pytest.raises(TextFormatError, match="without a directory"):
        parse_model_text(text)
