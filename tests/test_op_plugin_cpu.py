"""Operator plugin ABI: the host loader against a well-behaved plugin and against the ways a plugin can be wrong."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.utils.op_plugin import OpPlugin, OpPluginError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "examples", "plugins", "example_ops.c")
pytestmark = pytest.mark.skipif(shutil.which("gcc") is None, reason="building the example plugin needs gcc")


def build(tmp_path, name, *defines):
    out = str(tmp_path / f"lib{name}.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-I", os.path.join(ROOT, "csrc"), *defines, SRC, "-o", out], check=True)
    return out


def test_plugin_kernels_run_inside_a_graph_and_replace_a_builtin(tmp_path):
    from onnx_genai_b200.package.graph_executor import OPS, GraphExecutor

    path = build(tmp_path, "example_ops")
    plug = OpPlugin(path)
    assert plug.name == "example-ops" and plug.capabilities == 0x3
    assert [(d, o, v) for _, d, o, v in plug.kernels] == [("example.ops", "ScaledClip", 1), ("", "Relu", 6)]
    builtin_relu = OPS["Relu"]
    assert plug.register() == ["example.ops::ScaledClip", "Relu"]
    try:
        g = pb.Graph(name="g")
        g.inputs = [pb.ValueInfo("x", pb.FLOAT, (3, 5))]
        g.nodes = [pb.Node("ScaledClip", ["x"], ["a"], domain="example.ops", attrs={"alpha": 2.0, "lo": -0.5, "hi": 1.5}),
                   pb.Node("Relu", ["a"], ["b"]), pb.Node("ScaledClip", ["b"], ["y"], domain="example.ops", attrs={"alpha": 0.5})]
        g.outputs = [pb.ValueInfo("y", pb.FLOAT, (3, 5))]
        x = np.random.default_rng(0).standard_normal((3, 5)).astype(np.float32)
        ex = GraphExecutor(pb.Model(graph=g, opsets={"": 21, "example.ops": 1}), "cpu")
        y = ex.run({"x": x})["y"].numpy()
        want = np.clip(0.5 * np.maximum(np.clip(2.0 * x, -0.5, 1.5), 0), -1.0, 1.0)
        assert np.allclose(y, want, atol=1e-6)
        ex.run({"x": x})
        calls = ctypes.CDLL(path).example_ops_relu_calls
        calls.restype = ctypes.c_long
        assert calls() == 2                                   # the built-in Relu was not used
        with pytest.raises(OpPluginError, match="lo exceeds hi"):
            plug.kernel("example.ops", "ScaledClip", {"lo": 2.0, "hi": 1.0})
        with pytest.raises(OpPluginError, match="float32 only") as e:
            plug.kernel("example.ops", "ScaledClip")([torch.zeros(4, dtype=torch.int64)])
        assert e.value.code == 2
        with pytest.raises(OpPluginError, match="no kernel for example.ops::Nope"):
            plug.kernel("example.ops", "Nope")
    finally:
        plug.close()
    assert OPS["Relu"] is builtin_relu and "example.ops::ScaledClip" not in OPS


@pytest.mark.parametrize("define,message", [
    ("-DOGB_OP_WRONG_MAJOR", "version negotiation failed: host speaks 1.0, plugin answers 2.0"),
    ("-DOGB_OP_UNKNOWN_CAP", "capability bits this host does not know (0x100)"),
    ("-DOGB_OP_SHORT_VTABLE", "provider is 24 bytes"),
    ("-DOGB_OP_NO_OVERRIDE_CAP", "did not ask for the override capability"),
])
def test_misbehaving_plugins_are_refused_at_load(tmp_path, define, message):
    with pytest.raises(OpPluginError) as e:
        OpPlugin(build(tmp_path, "bad", define))
    assert message in str(e.value)


def test_a_failing_kernel_is_a_status_not_a_crash_and_unload_waits_for_kernels(tmp_path):
    plug = OpPlugin(build(tmp_path, "failing", "-DOGB_OP_FAILING_KERNEL"))
    k = plug.kernel("example.ops", "ScaledClip", {"alpha": 1.0})
    with pytest.raises(OpPluginError, match=r"internal error\): .*device lost \(injected\)") as e:
        k([torch.ones(2, 2)])
    assert e.value.code == 4
    err = ctypes.create_string_buffer(128)
    assert plug.lib.ogb_ophost_unload(plug.handle, err, len(err)) == 1 and b"still alive" in err.value
    plug.close()
    with pytest.raises(OpPluginError, match="cannot load"):
        OpPlugin(str(tmp_path / "missing.so"))
