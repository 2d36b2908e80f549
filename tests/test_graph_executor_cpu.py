"""Generic ONNX graph execution over torch: small graphs built with the package's own protobuf writer."""
import math
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package.graph_executor import GraphExecutionError, GraphExecutor, as_component

REF = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


def T(name, arr):
    arr = np.asarray(arr)
    dt = {np.dtype("float32"): pb.FLOAT, np.dtype("int64"): pb.INT64, np.dtype("bool"): pb.BOOL, np.dtype("uint8"): pb.UINT8}[arr.dtype]
    return pb.Tensor(name=name, dims=tuple(arr.shape), data_type=dt, array=arr)


def model(nodes, inits, inputs, outputs, tmp_path=None):
    g = pb.Graph(name="g", nodes=nodes, initializers={t.name: t for t in inits},
                 inputs=[pb.ValueInfo(n, dt, shape) for n, dt, shape in inputs], outputs=[pb.ValueInfo(n, pb.FLOAT, ()) for n in outputs])
    m = pb.Model(graph=g)
    if tmp_path is not None:                     # through the wire format and back
        path = str(tmp_path / "m.onnx")
        pb.save_model(m, path, external_data=False)
        return path
    return m


def N(op, ins, outs, domain="", **attrs):
    return pb.Node(op_type=op, inputs=list(ins), outputs=list(outs), name=outs[0], domain=domain, attrs=attrs)


def test_mlp_block_round_trips_through_the_wire_format(tmp_path):
    rng = np.random.default_rng(0)
    w1, b1 = rng.standard_normal((16, 8)).astype(np.float32), rng.standard_normal(16).astype(np.float32)
    w2 = rng.standard_normal((16, 4)).astype(np.float32)
    gam, bet = rng.standard_normal(16).astype(np.float32), rng.standard_normal(16).astype(np.float32)
    path = model([N("Gemm", ["x", "w1", "b1"], ["h"], transB=1, alpha=1.0, beta=1.0), N("Gelu", ["h"], ["a"], domain="com.microsoft"),
                  N("LayerNormalization", ["a", "gam", "bet"], ["n"], axis=-1, epsilon=1e-5), N("MatMul", ["n", "w2"], ["l"]),
                  N("Softmax", ["l"], ["p"], axis=-1)],
                 [T("w1", w1), T("b1", b1), T("w2", w2), T("gam", gam), T("bet", bet)], [("x", pb.FLOAT, ("b", 8))], ["p"], tmp_path)
    ex = GraphExecutor(path)
    x = torch.randn(5, 8)
    got = ex.run({"x": x})["p"]
    h = F.gelu(x @ torch.from_numpy(w1).T + torch.from_numpy(b1))
    want = torch.softmax(F.layer_norm(h, (16,), torch.from_numpy(gam), torch.from_numpy(bet), 1e-5) @ torch.from_numpy(w2), -1)
    assert torch.allclose(got, want, atol=1e-5) and ex.input_names == ["x"] and ex.output_names == ["p"]
    with pytest.raises(GraphExecutionError, match="missing graph input"):
        ex.run({})


def test_convolutional_stack():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((6, 3, 3, 3)).astype(np.float32) * 0.3
    b = rng.standard_normal(6).astype(np.float32)
    bn = [np.abs(rng.standard_normal(6)).astype(np.float32) + 0.5 for _ in range(4)]
    wt = rng.standard_normal((6, 2, 2, 2)).astype(np.float32) * 0.3
    m = model([N("Conv", ["x", "w", "b"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2]),
               N("BatchNormalization", ["c", "s", "bb", "mean", "var"], ["n"], epsilon=1e-5), N("Relu", ["n"], ["r"]),
               N("MaxPool", ["r"], ["p"], kernel_shape=[2, 2], strides=[2, 2]),
               N("ConvTranspose", ["p", "wt"], ["u"], kernel_shape=[2, 2], strides=[2, 2]),
               N("Resize", ["u", "", "scales"], ["z"], mode="nearest"),
               N("GroupNormalization", ["z", "gs", "gb"], ["gn"], num_groups=1, epsilon=1e-5),
               N("GlobalAveragePool", ["gn"], ["g"]), N("Flatten", ["g"], ["f"], axis=1)],
              [T("w", w), T("b", b), T("s", bn[0]), T("bb", bn[1]), T("mean", bn[2]), T("var", bn[3]), T("wt", wt),
               T("scales", np.asarray([1, 1, 2, 2], np.float32)), T("gs", np.ones(2, np.float32)), T("gb", np.zeros(2, np.float32))],
              [("x", pb.FLOAT, (1, 3, 16, 16))], ["f", "z"])
    x = torch.randn(2, 3, 16, 16)
    out = GraphExecutor(m).run({"x": x})
    tt = torch.from_numpy
    c = F.conv2d(x, tt(w), tt(b), stride=2, padding=1)
    r = F.relu(F.batch_norm(c, tt(bn[2]), tt(bn[3]), tt(bn[0]), tt(bn[1]), False, 0.0, 1e-5))
    u = F.conv_transpose2d(F.max_pool2d(r, 2, 2), tt(wt), stride=2)
    z = F.interpolate(u, scale_factor=2.0, mode="nearest")
    assert torch.allclose(out["z"], z, atol=1e-5) and out["z"].shape == (2, 2, 16, 16)
    assert torch.allclose(out["f"], F.group_norm(z, 1).mean((2, 3)), atol=1e-5)


def test_attention_shaped_graph_with_shape_ops():
    """Single-head attention written with the shape plumbing exporters emit: Shape / Gather / Unsqueeze / Concat / Reshape,
    Transpose, a causal mask from Trilu + Where, Slice with a negative step and Split."""
    d = 8
    rng = np.random.default_rng(2)
    wqkv = rng.standard_normal((d, 3 * d)).astype(np.float32) * 0.3
    nodes = [N("MatMul", ["x", "wqkv"], ["qkv"]), N("Split", ["qkv"], ["q", "k", "v"], axis=-1),
             N("Transpose", ["k"], ["kt"], perm=[0, 2, 1]), N("MatMul", ["q", "kt"], ["s0"]),
             N("Constant", [], ["scale"], value=T("", np.asarray(1.0 / math.sqrt(d), np.float32))), N("Mul", ["s0", "scale"], ["s"]),
             N("Shape", ["x"], ["shp"]), N("Gather", ["shp", "one"], ["t"], axis=0), N("Unsqueeze", ["t", "zero_ax"], ["t1"]),
             N("Concat", ["t1", "t1"], ["tt"], axis=0), N("ConstantOfShape", ["tt"], ["ones"], value=T("", np.asarray([1.0], np.float32))),
             N("Trilu", ["ones"], ["low"], upper=0), N("Cast", ["low"], ["mask"], to=pb.BOOL),
             N("Constant", [], ["neg"], value=T("", np.asarray(-1e9, np.float32))), N("Where", ["mask", "s", "neg"], ["sm"]),
             N("Softmax", ["sm"], ["p"], axis=-1), N("MatMul", ["p", "v"], ["o"]),
             N("Slice", ["o", "st", "en", "ax", "step"], ["rev"]), N("ReduceMean", ["rev"], ["m"], axes=[-1], keepdims=0)]
    m = model(nodes, [T("wqkv", wqkv), T("one", np.asarray(1, np.int64)), T("zero_ax", np.asarray([0], np.int64)),
                      T("st", np.asarray([-1], np.int64)), T("en", np.asarray([-(2 ** 62)], np.int64)), T("ax", np.asarray([1], np.int64)),
                      T("step", np.asarray([-1], np.int64))], [("x", pb.FLOAT, ("b", "t", d))], ["o", "rev", "m"])
    x = torch.randn(2, 5, d)
    out = GraphExecutor(m).run({"x": x})
    q, k, v = (x @ torch.from_numpy(wqkv)).split(d, -1)
    want = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert torch.allclose(out["o"], want, atol=1e-5)
    assert torch.allclose(out["rev"], want.flip(1), atol=1e-5) and torch.allclose(out["m"], want.flip(1).mean(-1), atol=1e-5)


def test_matmul_nbits_against_explicit_dequantisation():
    rng = np.random.default_rng(3)
    n, k, block = 6, 64, 32
    q = rng.integers(0, 16, size=(n, k)).astype(np.uint8)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).reshape(n, k // block, block // 2)
    scales = (rng.random((n, k // block)).astype(np.float32) + 0.1) * 0.1
    zp_q = rng.integers(0, 16, size=(n, k // block)).astype(np.uint8)
    zp = (zp_q[:, 0::2] | (zp_q[:, 1::2] << 4))
    m = model([N("MatMulNBits", ["x", "B", "s", "zp"], ["y"], domain="com.microsoft", K=k, N=n, bits=4, block_size=block)],
              [T("B", packed), T("s", scales.reshape(-1)), T("zp", zp.reshape(-1))], [("x", pb.FLOAT, ("m", k))], ["y"])
    x = torch.randn(3, k)
    got = GraphExecutor(m).run({"x": x})["y"]
    w = (q.reshape(n, k // block, block).astype(np.float32) - zp_q[..., None]) * scales[..., None]
    assert torch.allclose(got, x @ torch.from_numpy(w.reshape(n, k)).T, atol=1e-4)


def test_errors_name_the_operator_or_the_node():
    with pytest.raises(GraphExecutionError, match="outside the covered set: SequenceMap"):
        GraphExecutor(model([N("SequenceMap", ["x"], ["y"])], [], [("x", pb.FLOAT, (1,))], ["y"]))
    ex = GraphExecutor(model([N("MatMul", ["x", "w"], ["y"])], [T("w", np.zeros((3, 2), np.float32))], [("x", pb.FLOAT, ("b", 4))], ["y"]))
    with pytest.raises(GraphExecutionError, match=r"node 'y' \(MatMul\) failed on inputs \[\(2, 4\), \(3, 2\)\]"):
        ex.run({"x": torch.zeros(2, 4)})
    with pytest.raises(GraphExecutionError, match="never produced"):
        GraphExecutor(model([N("Relu", ["nowhere"], ["y"])], [], [("x", pb.FLOAT, (1,))], ["y"]))


def test_onnx_policy_graphs_as_workflow_components(tmp_path):
    """The imported ComfyUI document run with its policy components as ONNX graphs (Euler step, guidance, predicate)."""
    from onnx_genai_b200.engine.workflow_runtime import run_workflow
    from onnx_genai_b200.package.comfyui import import_comfyui
    from test_comfyui_cpu import GRAPH

    sig = np.linspace(1.0, 0.0, 21).astype(np.float32)
    one = T("one", np.asarray([1], np.int64))
    solver = model([N("Gather", ["schedule", "step"], ["s0"], axis=0), N("Add", ["step", "one"], ["nx"]), N("Gather", ["schedule", "nx"], ["s1"], axis=0),
                    N("Sub", ["s1", "s0"], ["dt"]), N("Reshape", ["dt", "shape"], ["dt4"]), N("Mul", ["dt4", "derivative"], ["upd"]),
                    N("Add", ["sample", "upd"], ["next_state"])], [one, T("shape", np.asarray([1, 1, 1, 1], np.int64))],
                   [("sample", pb.FLOAT, ()), ("step", pb.INT64, (1,)), ("schedule", pb.FLOAT, (21,)), ("derivative", pb.FLOAT, ())], ["next_state"])
    guidance = model([N("Sub", ["conditional", "unconditional"], ["d"]), N("Mul", ["d", "scale"], ["sd"]), N("Add", ["unconditional", "sd"], ["guided"])],
                     [], [("conditional", pb.FLOAT, ()), ("unconditional", pb.FLOAT, ()), ("scale", pb.FLOAT, (1,))], ["guided"])
    predicate = model([N("Not", ["done"], ["continue"])], [], [("done", pb.BOOL, (1,))], ["continue"])
    schedule = model([N("Identity", ["sig"], ["schedule"])], [T("sig", sig)], [], ["schedule"])
    comps = {"solver_step": as_component(solver), "guidance": as_component(guidance), "continue_predicate": as_component(predicate),
             "schedule": as_component(schedule),
             "text_encoder": lambda p: {"encoder_hidden_states": torch.as_tensor(p["input_ids"]).float() / 10.0},
             "denoiser": lambda p: {"noise_pred": torch.as_tensor(p["sample"]) * 0.5 + torch.as_tensor(p["encoder_hidden_states"]).mean()},
             "vae_decoder": lambda p: {"image": p["latent"][:, :3]}}
    noise = torch.randn(1, 4, 8, 8)
    pos, neg = np.array([[1, 2, 3]]), np.array([[4, 5, 6]])
    g = {k: ({**v, "inputs": {**v["inputs"], "width": 64, "height": 64, "batch_size": 1}} if v["class_type"] == "EmptyLatentImage" else v)
         for k, v in GRAPH.items()}
    out = run_workflow(import_comfyui(g), comps, {"request.positive_ids": pos, "request.negative_ids": neg, "request.noise": noise})
    x = noise.clone()
    cp, cn = float((pos / 10.0).mean()), float((neg / 10.0).mean())
    for i in range(20):
        d = (x * 0.5 + cn) + 8.0 * ((x * 0.5 + cp) - (x * 0.5 + cn))
        x = x + float(sig[i + 1] - sig[i]) * d
    assert torch.allclose(out["image"], x[:, :3], atol=1e-4)
    assert comps["solver_step"].executor.runs == 20


def test_run_workflow_cli_on_a_package_written_to_disk(tmp_path):
    """ComfyUI graph -> metadata document; every component an ONNX file written by this package's writer; run from the CLI."""
    import json as _json
    import struct
    import zlib

    import yaml

    from onnx_genai_b200 import cli
    from onnx_genai_b200.package.comfyui import import_comfyui
    from test_comfyui_cpu import GRAPH

    g = {k: ({**v, "inputs": {**v["inputs"], "width": 64, "height": 64, "batch_size": 1, }} if v["class_type"] == "EmptyLatentImage" else v)
         for k, v in GRAPH.items()}
    g["3"] = {**g["3"], "inputs": {**g["3"]["inputs"], "steps": 4}}
    doc = import_comfyui(g)
    pkg = tmp_path / "pkg"
    sig = np.linspace(1.0, 0.0, 5).astype(np.float32)
    one = T("one", np.asarray([1], np.int64))
    graphs = {
        "policies/solver_euler.onnx": model(
            [N("Gather", ["schedule", "step"], ["s0"], axis=0), N("Add", ["step", "one"], ["nx"]), N("Gather", ["schedule", "nx"], ["s1"], axis=0),
             N("Sub", ["s1", "s0"], ["dt"]), N("Reshape", ["dt", "shape"], ["dt4"]), N("Mul", ["dt4", "derivative"], ["upd"]),
             N("Add", ["sample", "upd"], ["next_state"])], [one, T("shape", np.asarray([1, 1, 1, 1], np.int64))],
            [("sample", pb.FLOAT, ()), ("step", pb.INT64, (1,)), ("schedule", pb.FLOAT, (5,)), ("derivative", pb.FLOAT, ())], ["next_state"]),
        "policies/classifier_free_guidance.onnx": model(
            [N("Sub", ["conditional", "unconditional"], ["d"]), N("Mul", ["d", "scale"], ["sd"]), N("Add", ["unconditional", "sd"], ["guided"])],
            [], [("conditional", pb.FLOAT, ()), ("unconditional", pb.FLOAT, ()), ("scale", pb.FLOAT, (1,))], ["guided"]),
        "policies/continue.onnx": model([N("Not", ["done"], ["continue"])], [], [("done", pb.BOOL, (1,))], ["continue"]),
        "policies/schedule_karras.onnx": model([N("Identity", ["sig"], ["schedule"])], [T("sig", sig)], [], ["schedule"]),
        "sd15/text_encoder.onnx": model([N("Cast", ["input_ids"], ["f"], to=pb.FLOAT), N("ReduceMean", ["f"], ["m"], axes=[1], keepdims=1),
                                         N("Mul", ["m", "tenth"], ["encoder_hidden_states"])], [T("tenth", np.asarray(0.1, np.float32))],
                                        [("input_ids", pb.INT64, ("b", "s"))], ["encoder_hidden_states"]),
        "sd15/unet.onnx": model([N("Mul", ["sample", "half"], ["h"]), N("ReduceMean", ["encoder_hidden_states"], ["c"], keepdims=0),
                                 N("Add", ["h", "c"], ["noise_pred"])], [T("half", np.asarray(0.5, np.float32))],
                                [("sample", pb.FLOAT, ()), ("step", pb.INT64, (1,)), ("schedule", pb.FLOAT, (5,)),
                                 ("encoder_hidden_states", pb.FLOAT, ())], ["noise_pred"]),
        "sd15/vae_decoder.onnx": model([N("Slice", ["latent", "s", "e", "ax"], ["rgb"]), N("Resize", ["rgb", "", "scales"], ["big"], mode="nearest"),
                                        N("Tanh", ["big"], ["image"])],
                                       [T("s", np.asarray([0], np.int64)), T("e", np.asarray([3], np.int64)), T("ax", np.asarray([1], np.int64)),
                                        T("scales", np.asarray([1, 1, 8, 8], np.float32))], [("latent", pb.FLOAT, ())], ["image"]),
    }
    for rel, m in graphs.items():
        path = pkg / rel
        path.parent.mkdir(parents=True, exist_ok=True)
        pb.save_model(m, str(path), external_data=False)
    (pkg / "inference_metadata.yaml").write_text(yaml.safe_dump(doc, sort_keys=False))
    noise = np.random.default_rng(0).standard_normal((1, 4, 8, 8)).astype(np.float32)
    np.save(tmp_path / "noise.npy", noise)
    out_dir = tmp_path / "out"
    import io
    import contextlib

    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        rc = cli.main(["run-workflow", str(pkg), "--input", "request.positive_ids=ids:1,2,3", "--input", "request.negative_ids=ids:4,5,6",
                       "--input", f"request.noise={tmp_path / 'noise.npy'}", "--out", str(out_dir)])
    assert rc == 0
    rep = _json.loads(buf.getvalue().strip().splitlines()[-1])
    assert rep["outputs"] == {"image": [1, 3, 64, 64]} and rep["iterations"] == 4 and rep["invocations"]["denoiser"] == 8
    x = noise.copy()
    for i in range(4):
        d = (x * 0.5 + 0.5) + 8.0 * ((x * 0.5 + 0.2) - (x * 0.5 + 0.5))
        x = x + (sig[i + 1] - sig[i]) * d
    want = np.tanh(np.repeat(np.repeat(x[:, :3], 8, 2), 8, 3))
    assert np.allclose(np.load(out_dir / "image.npy"), want, atol=1e-4)
    png = (out_dir / "image.png").read_bytes()
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and struct.unpack(">II", png[16:24]) == (64, 64)
    idat = png[png.index(b"IDAT") + 4: png.index(b"IEND") - 8]
    assert len(zlib.decompress(idat)) == 64 * (64 * 3 + 1)
    # a missing input and a missing artifact are reported, not raised
    assert cli.main(["run-workflow", str(pkg), "--input", "request.positive_ids=ids:1"]) == 1
    (pkg / "sd15" / "unet.onnx").unlink()
    assert cli.main(["run-workflow", str(pkg)]) == 1


def test_tensor_scatter_linear_and_circular():
    cache = np.zeros((2, 1, 5, 2), np.float32)
    upd = np.arange(2 * 1 * 2 * 2, dtype=np.float32).reshape(2, 1, 2, 2) + 1
    for mode, idx, rows in (("linear", [1, 3], ([1, 2], [3, 4])), ("circular", [4, 0], ([4, 0], [0, 1]))):
        m = model([N("TensorScatter", ["c", "u", "i"], ["o"], axis=-2, mode=mode)], [T("i", np.asarray(idx, np.int64))],
                  [("c", pb.FLOAT, (2, 1, 5, 2)), ("u", pb.FLOAT, (2, 1, 2, 2))], ["o"])
        out = GraphExecutor(m).run({"c": cache, "u": upd})["o"]
        want = torch.zeros(2, 1, 5, 2)
        for b in range(2):
            for j, pos in enumerate(rows[b]):
                want[b, 0, pos] = torch.from_numpy(upd[b, 0, j])
        assert torch.equal(out, want), mode
    m = model([N("TensorScatter", ["c", "u", "i"], ["o"])], [T("i", np.asarray([4, 0], np.int64))],
              [("c", pb.FLOAT, (2, 1, 5, 2)), ("u", pb.FLOAT, (2, 1, 2, 2))], ["o"])
    with pytest.raises(GraphExecutionError, match="into a cache of length 5"):
        GraphExecutor(m).run({"c": cache, "u": upd})


def test_if_and_loop_with_captured_outer_values(tmp_path):
    """If picks a branch; Loop carries state, emits a scan output and stops on its condition; bodies read outer values."""
    vi = lambda n, dt=pb.FLOAT, shape=(): pb.ValueInfo(n, dt, shape)
    then_g = pb.Graph(name="then", nodes=[N("Mul", ["x", "two"], ["t_out"])], outputs=[vi("t_out")])            # captures x and two
    else_g = pb.Graph(name="else", nodes=[N("Neg", ["x"], ["e_out"])], outputs=[vi("e_out")])
    # body: acc <- acc + y * step ; keep going while acc < limit ; scan output = acc
    body = pb.Graph(name="body", inputs=[vi("i", pb.INT64), vi("c", pb.BOOL), vi("acc")],
                    nodes=[N("Mul", ["y", "step"], ["inc"]), N("Add", ["acc", "inc"], ["acc_next"]), N("Less", ["acc_next", "limit"], ["c_next"]),
                           N("Identity", ["acc_next"], ["trace"])],
                    outputs=[vi("c_next", pb.BOOL), vi("acc_next"), vi("trace")])
    m = model([N("Greater", ["s", "zero"], ["pos"]), N("If", ["pos"], ["y"], then_branch=then_g, else_branch=else_g),
               N("Loop", ["trips", "go", "zero"], ["final", "history"], body=body)],
              [T("two", np.asarray(2.0, np.float32)), T("zero", np.asarray(0.0, np.float32)), T("step", np.asarray(0.5, np.float32)),
               T("limit", np.asarray(7.0, np.float32)), T("trips", np.asarray(10, np.int64)), T("go", np.asarray(True))],
              [("x", pb.FLOAT, ()), ("s", pb.FLOAT, ())], ["y", "final", "history"], tmp_path)          # through the binary codec
    ex = GraphExecutor(m)
    out = ex.run({"x": torch.tensor(3.0), "s": torch.tensor(1.0)})
    assert float(out["y"]) == 6.0                                     # then-branch: x * 2
    assert out["history"].tolist() == [3.0, 6.0, 9.0] and float(out["final"]) == 9.0      # stops once acc >= 7
    out = ex.run({"x": torch.tensor(3.0), "s": torch.tensor(-1.0)})
    assert float(out["y"]) == -3.0 and out["history"].tolist() == [-1.5 * k for k in range(1, 11)]     # never reaches the limit: trip count ends it
    bad_body = pb.Graph(name="b", inputs=[vi("i", pb.INT64)], nodes=[N("Identity", ["i"], ["o"])], outputs=[vi("o", pb.INT64)])
    bad = model([N("Loop", ["trips", "", "x"], ["r"], body=bad_body)], [T("trips", np.asarray(2, np.int64))], [("x", pb.FLOAT, ())], ["r"])
    with pytest.raises(GraphExecutionError, match="Loop body takes 1 inputs"):
        GraphExecutor(bad).run({"x": torch.tensor(1.0)})
    nested_unknown = pb.Graph(name="t", nodes=[N("Sort", ["x"], ["o"])], outputs=[vi("o")])
    with pytest.raises(GraphExecutionError, match="outside the covered set: Sort"):
        GraphExecutor(model([N("If", ["c"], ["y"], then_branch=nested_unknown, else_branch=else_g)], [], [("x", pb.FLOAT, ()), ("c", pb.BOOL, ())], ["y"]))


def test_moe_and_qmoe_against_a_dense_statement():
    rng = np.random.default_rng(7)
    experts, hid, inter, k, t, block = 4, 16, 16, 2, 5, 16          # every input width is one quantisation block
    x = rng.standard_normal((t, hid)).astype(np.float32)
    router = rng.standard_normal((t, experts)).astype(np.float32)
    pack = lambda q: (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)      # least significant nibble first along the input axis
    q1 = rng.integers(0, 16, size=(experts, 2 * inter, hid)).astype(np.uint8)
    s1 = (rng.random((experts, 2 * inter, 1)).astype(np.float32) + 0.5) * 0.05
    q2 = rng.integers(0, 16, size=(experts, hid, inter)).astype(np.uint8)
    s2 = (rng.random((experts, hid, 1)).astype(np.float32) + 0.5) * 0.05
    w1 = (q1.astype(np.float32) - 8.0) * s1
    w2 = (q2.astype(np.float32) - 8.0) * s2
    m = model([N("QMoE", ["x", "r", "w1", "s1", "", "w2", "s2"], ["y"], domain="com.microsoft", k=k, activation_type="swiglu", swiglu_fusion=1,
                 expert_weight_bits=4, block_size=block, normalize_routing_weights=1, quant_type="int")],
              [T("w1", pack(q1)), T("s1", s1), T("w2", pack(q2)), T("s2", s2)], [("x", pb.FLOAT, (t, hid)), ("r", pb.FLOAT, (t, experts))], ["y"])
    got = GraphExecutor(m).run({"x": x, "r": router})["y"]
    want = np.zeros((t, hid), np.float32)
    for row in range(t):
        top = sorted(range(experts), key=lambda e: (-router[row, e], e))[:k]
        ex = np.exp(router[row] - router[row].max())
        for e in top:
            h = w1[e] @ x[row]
            g, l = h[0::2], h[1::2]
            act = g * (1 / (1 + np.exp(-g))) * l
            want[row] += ex[e] / ex[top].sum() * (w2[e] @ act)
    assert torch.allclose(got, torch.from_numpy(want), atol=1e-4)
    # float MoE, relu, weights over all experts (no renormalisation)
    f1, f2 = rng.standard_normal((experts, inter, hid)).astype(np.float32) * 0.2, rng.standard_normal((experts, hid, inter)).astype(np.float32) * 0.2
    m = model([N("MoE", ["x", "r", "f1", "", "f2"], ["y"], domain="com.microsoft", k=1, activation_type="relu")], [T("f1", f1), T("f2", f2)],
              [("x", pb.FLOAT, (t, hid)), ("r", pb.FLOAT, (t, experts))], ["y"])
    got = GraphExecutor(m).run({"x": x, "r": router})["y"]
    want = np.zeros((t, hid), np.float32)
    for row in range(t):
        e = int(np.argmax(router[row]))
        p = np.exp(router[row] - router[row].max())
        want[row] = p[e] / p.sum() * (f2[e] @ np.maximum(f1[e] @ x[row], 0))
    assert torch.allclose(got, torch.from_numpy(want), atol=1e-5)


def test_block_quantized_matmul_mxfp4_and_iq4_nl():
    """Layout facts of the two covered formats, then the operator against a dense product with the decoded weight."""
    import struct

    from onnx_genai_b200.package.graph_executor import OPS, GraphExecutionError, decode_weight_blocks, encode_mxfp4

    # mxfp4: scale byte first; byte j = element j (low nibble) and element j+16 (high nibble); code 8|m is -m
    blk = torch.zeros(1, 1, 17, dtype=torch.uint8)
    blk[0, 0, 0] = 128                               # 2^(128-127) = 2
    blk[0, 0, 1] = 0x27                              # element 0 = code 7 (6.0), element 16 = code 2 (1.0)
    blk[0, 0, 2] = 0x0B                              # element 1 = code 11 (-1.5)
    w = decode_weight_blocks(blk, "mxfp4")[0]
    assert w[0] == 12.0 and w[16] == 2.0 and w[1] == -3.0 and float(w.abs().sum()) == 17.0
    blk[0, 0, 0] = 255                               # a NaN scale poisons non-zero codes only
    w = decode_weight_blocks(blk, "mxfp4")[0]
    assert torch.isnan(w[0]) and w[2] == 0.0
    # iq4_nl: fp16 scale, then the same nibble order over the non-linear table
    raw = bytearray(18)
    raw[0:2] = struct.pack("<e", 0.5)
    raw[2] = 0xF0                                    # element 0 = table[0] = -127, element 16 = table[15] = 113
    w = decode_weight_blocks(torch.tensor(list(raw), dtype=torch.uint8).reshape(1, 1, 18), "iq4_nl")[0]
    assert w[0] == -63.5 and w[16] == 56.5

    torch.manual_seed(0)
    dense = torch.randn(5, 70)                       # K = 70: the third block is partial
    packed = encode_mxfp4(dense)
    assert tuple(packed.shape) == (5, 3, 17)
    deq = decode_weight_blocks(packed, "mxfp4")[:, :70]
    assert float((deq - dense).abs().max()) <= 0.5 * float(dense.abs().max()) / 3      # half the widest code gap (4 -> 6) at scale amax/6
    assert torch.equal(decode_weight_blocks(encode_mxfp4(deq), "mxfp4")[:, :70], deq)    # representable values survive a second trip
    x, bias = torch.randn(2, 3, 70), torch.randn(5)
    y = OPS["BlockQuantizedMatMul"]([x, packed, bias], {"K": 70, "N": 5, "format": "mxfp4", "block_layout_version": 1})
    assert torch.allclose(y, x @ deq.T + bias, atol=1e-5) and tuple(y.shape) == (2, 3, 5)
    with pytest.raises(GraphExecutionError, match="iq2_xxs"):
        OPS["BlockQuantizedMatMul"]([x, packed, None], {"K": 70, "N": 5, "format": "iq2_xxs"})
    with pytest.raises(GraphExecutionError, match="block_layout_version"):
        OPS["BlockQuantizedMatMul"]([x, packed, None], {"K": 70, "N": 5, "format": "mxfp4", "block_layout_version": 2})


def test_block_quantized_matmul_iq4_xs_superblocks():
    """iq4_xs: the pinned vector of the reference's unit test (d = 0.5, every 6-bit sub-scale 37, every code byte 0x98 ->
    sixteen 2.5 then sixteen 32.5 per sub-block), then random super-blocks against a scalar statement of the layout."""
    import struct

    from onnx_genai_b200.package.graph_executor import _IQ4_NL, OPS, decode_weight_blocks

    raw = bytearray(struct.pack("<e", 0.5)) + bytearray(struct.pack("<H", 0xAAAA)) + bytearray([0x55] * 4) + bytearray([0x98] * 128)
    w = decode_weight_blocks(torch.tensor(list(raw), dtype=torch.uint8).reshape(1, 1, 136), "iq4_xs")[0]
    assert w.tolist() == ([2.5] * 16 + [32.5] * 16) * 8

    g = torch.Generator().manual_seed(3)
    packed = torch.randint(0, 256, (3, 2, 136), dtype=torch.uint8, generator=g)
    packed[..., 0:2] = torch.tensor(list(struct.pack("<e", 0.03125)), dtype=torch.uint8)      # a finite fp16 scale
    got = decode_weight_blocks(packed, "iq4_xs")
    want = torch.zeros(3, 512)
    for n in range(3):
        for blk in range(2):
            b = packed[n, blk].tolist()
            d = struct.unpack("<e", bytes(b[0:2]))[0]
            high = b[2] | (b[3] << 8)
            for ib in range(8):
                ls = ((b[4 + ib // 2] >> (4 * (ib % 2))) & 0xF) | (((high >> (2 * ib)) & 3) << 4)
                dl = d * (ls - 32)
                qs = b[8 + 16 * ib: 8 + 16 * ib + 16]
                for j in range(16):
                    want[n, blk * 256 + ib * 32 + j] = dl * _IQ4_NL[qs[j] & 0xF]
                    want[n, blk * 256 + ib * 32 + j + 16] = dl * _IQ4_NL[qs[j] >> 4]
    assert torch.allclose(got, want, rtol=0, atol=1e-6)
    x = torch.randn(4, 300)                            # K = 300: the second super-block is partial
    y = OPS["BlockQuantizedMatMul"]([x, packed, None], {"K": 300, "N": 3, "format": "iq4_xs", "block_layout_version": 1})
    assert torch.allclose(y, x @ want[:, :300].T, atol=1e-4)


def test_contrib_attention_variants_nonzero_prelu():
    from onnx_genai_b200.package.graph_executor import OPS

    torch.manual_seed(1)
    b, s, past, h, d = 2, 3, 4, 4, 8
    q, k, v = torch.randn(b, s, h * d), torch.randn(b, s, h * d), torch.randn(b, s, h * d)
    pk, pv = torch.randn(b, h, past, d), torch.randn(b, h, past, d)
    bias = torch.randn(3 * h * d)
    pad = torch.ones(b, past + s, dtype=torch.int32)
    pad[1, :2] = 0
    out, nk, nv = OPS["MultiHeadAttention"]([q, k, v, bias, pad, None, pk, pv], {"num_heads": h, "unidirectional": 1})
    bq, bk, bv = bias.split(h * d)
    heads = lambda x: x.reshape(b, s, h, d).transpose(1, 2)
    kk, vv = torch.cat([pk, heads(k + bk)], 2), torch.cat([pv, heads(v + bv)], 2)
    assert torch.equal(nk, kk) and torch.equal(nv, vv)
    for bi in range(b):
        for hi in range(h):
            for si in range(s):
                sc = (heads(q + bq)[bi, hi, si] @ kk[bi, hi].T) / d ** 0.5
                sc[past + si + 1:] = float("-inf")
                if bi == 1:
                    sc[:2] = -10000.0
                want = torch.softmax(sc, -1) @ vv[bi, hi]
                assert torch.allclose(out[bi, si, hi * d:(hi + 1) * d], want, atol=1e-5)

    # packed rows: two sequences of 3 and 5 tokens equal two separate unpadded calls
    t = 8
    q, k, v = torch.randn(t, h * d), torch.randn(t, h * d), torch.randn(t, h * d)
    cu = torch.tensor([0, 3, 8], dtype=torch.int32)
    packed = OPS["PackedMultiHeadAttention"]([q, k, v, None, torch.zeros(2, 5, dtype=torch.int32), cu], {"num_heads": h})
    for lo, hi in ((0, 3), (3, 8)):
        want = OPS["MultiHeadAttention"]([q[None, lo:hi], k[None, lo:hi], v[None, lo:hi]], {"num_heads": h})[0][0]
        assert torch.allclose(packed[lo:hi], want, atol=1e-5)

    nz = OPS["NonZero"]([torch.tensor([[0.0, 2.0], [3.0, 0.0]])], {})
    assert nz.dtype == torch.int64 and nz.tolist() == [[0, 1], [1, 0]]
    assert OPS["PRelu"]([torch.tensor([[-2.0, 4.0], [-1.0, -3.0]]), torch.tensor([0.5, 0.1])], {}).tolist() == [[-1.0, 4.0], [-0.5, pytest.approx(-0.3)]]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "crates", "onnx-runtime-ep-cpu-plugin", "tests", "fixtures")),
                    reason="the upstream operator fixtures are not available on this machine")
def test_every_upstream_operator_fixture_runs():
    """The reference's provider-plugin fixtures are single-operator or few-operator graphs with declared static shapes;
    each must execute here on random inputs of those shapes and give outputs of the declared shapes."""
    import glob

    from onnx_genai_b200.package import onnx_pb as pb
    from onnx_genai_b200.package.graph_executor import GraphExecutor
    from onnx_genai_b200.package.onnx_text import load_any

    ran = 0
    rng = np.random.default_rng(0)
    for path in sorted(glob.glob(os.path.join(REF, "crates", "onnx-runtime-ep-cpu-plugin", "tests", "fixtures", "*", "model.onnx.textproto"))):
        model = load_any(path)
        g = model.graph
        if any(not all(isinstance(d, int) for d in vi.shape) for vi in g.inputs if vi.name not in g.initializers):
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
        out = GraphExecutor(model, "cpu").run(feeds)
        for vo in g.outputs:
            if vo.shape and all(isinstance(d, int) for d in vo.shape) and "nonzero" not in path:
                assert tuple(out[vo.name].shape) == tuple(vo.shape), (path, vo.name, tuple(out[vo.name].shape), vo.shape)
        ran += 1
    assert ran >= 10, ran


def test_index_share_equals_dense_masked_attention_and_validates_indices():
    from onnx_genai_b200.package.graph_executor import OPS

    torch.manual_seed(2)
    b, n, nkv, sq, past, h, kk = 2, 4, 2, 3, 5, 8, 4
    q, k, v = torch.randn(b, n, sq, h), torch.randn(b, nkv, sq, h), torch.randn(b, nkv, sq, h)
    pk, pv = torch.randn(b, nkv, past, h), torch.randn(b, nkv, past, h)
    total = past + sq
    sel = torch.full((b, 1, sq, kk), -1, dtype=torch.int64)
    for bi in range(b):
        for si in range(sq):
            m = 2 + (bi + si) % 3                                                 # rows of different fill
            sel[bi, 0, si, :m] = torch.sort(torch.randperm(past + si + 1)[:m]).values
    bias = torch.zeros(1, 1, sq, total).masked_fill(~torch.ones(sq, total, dtype=torch.bool).tril(past), float("-inf"))
    out, nk, nv = OPS["IndexShare"]([q, k, v, pk, pv, sel, bias], {"num_heads": n, "kv_num_heads": nkv})
    assert torch.equal(nk, torch.cat([pk, k], 2)) and torch.equal(nv, torch.cat([pv, v], 2))
    dense = torch.full((b, 1, sq, total), float("-inf"))
    for bi in range(b):
        for si in range(sq):
            dense[bi, 0, si, sel[bi, 0, si][sel[bi, 0, si] >= 0]] = 0.0
    kf, vf = nk.repeat_interleave(n // nkv, 1), nv.repeat_interleave(n // nkv, 1)
    want = torch.softmax(q @ kf.transpose(-1, -2) / h ** 0.5 + dense + bias, -1) @ vf
    assert torch.allclose(out, want, atol=1e-5)
    # a row whose selected positions are all masked by the bias gives zeros, not NaN
    dead = bias.clone()
    dead[..., 0, :] = float("-inf")
    out2 = OPS["IndexShare"]([q, k, v, pk, pv, sel, dead], {"num_heads": n, "kv_num_heads": nkv})[0]
    assert float(out2[:, :, 0].abs().max()) == 0.0 and torch.allclose(out2[:, :, 1:], want[:, :, 1:], atol=1e-5)

    def bad(row, match):
        s2 = sel.clone()
        s2[0, 0, 0] = torch.tensor(row)
        with pytest.raises(GraphExecutionError, match=match):
            OPS["IndexShare"]([q, k, v, pk, pv, s2, None], {"num_heads": n, "kv_num_heads": nkv})

    bad([1, 1, 2, -1], "strictly increasing")
    bad([3, 2, -1, -1], "strictly increasing")
    bad([0, -1, 2, -1], "pad the end")
    bad([-1, -1, -1, -1], "empty")
    bad([0, 1, total, -1], "outside")

    # ties go to the lower index, largest or smallest
    vals, idx = OPS["TopK"]([torch.tensor([[0.0, 2.0, 0.0, 2.0, 1.0]]), torch.tensor([3])], {})
    assert idx.tolist() == [[1, 3, 4]] and vals.tolist() == [[2.0, 2.0, 1.0]]
    assert OPS["TopK"]([torch.tensor([[0.0, 2.0, 0.0, 2.0, 1.0]]), torch.tensor([2])], {"largest": 0})[1].tolist() == [[0, 2]]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "tests", "fixtures", "tiny-fp8-kv")),
                    reason="the upstream fp8 cache fixtures are not available on this machine")
def test_fp8_cache_graphs_keep_their_element_type():
    """The reference probes a runtime for one-byte KV support with two graphs over FLOAT8E4M3FN tensors
    (crates/onnx-genai-ort/tests/fp8_kv_capability.rs): a scatter of new rows into a cache and an identity."""
    from onnx_genai_b200.package.onnx_text import load_any

    d = os.path.join(REF, "tests", "fixtures", "tiny-fp8-kv")
    cache = torch.zeros(2, 4, 8).to(torch.float8_e4m3fn)
    new = (torch.arange(16).reshape(2, 1, 8).float() / 4).to(torch.float8_e4m3fn)
    out = GraphExecutor(load_any(os.path.join(d, "scatter.onnx.textproto")), "cpu").run(
        {"key_cache": cache, "write_indices": torch.tensor([[[0, 2]], [[1, 1]]]), "new_key": new})["updated_key_cache"]
    assert out.dtype == torch.float8_e4m3fn
    want = torch.zeros(2, 4, 8)
    want[0, 2], want[1, 1] = new[0, 0].float(), new[1, 0].float()
    assert torch.equal(out.float(), want)
    same = GraphExecutor(load_any(os.path.join(d, "identity.onnx.textproto")), "cpu").run({"key_cache": out})["updated_key_cache"]
    assert same.dtype == torch.float8_e4m3fn and torch.equal(same.float(), want)
