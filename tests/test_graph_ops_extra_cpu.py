"""The long tail of graph operators, each against a direct statement of its definition."""
import math

import numpy as np
import pytest
import torch

from onnx_genai_b200.package.graph_executor import OPS, GraphExecutionError


def test_elementwise_activations_and_reductions():
    x = torch.tensor([[-1.5, -0.25, 0.0, 0.4, 2.0]])
    unit = torch.tensor([-0.9, -0.2, 0.0, 0.5, 0.8])
    for name, fn in (("Acos", np.arccos), ("Asin", np.arcsin), ("Atan", np.arctan), ("Atanh", np.arctanh), ("Asinh", np.arcsinh),
                     ("Sinh", np.sinh), ("Cosh", np.cosh), ("Tan", np.tan)):
        assert np.allclose(OPS[name]([unit], {}).numpy(), fn(unit.numpy()), atol=1e-6), name
    assert np.allclose(OPS["Acosh"]([unit + 2], {}).numpy(), np.arccosh(unit.numpy() + 2), atol=1e-6)
    assert torch.allclose(OPS["Softsign"]([x], {}), x / (1 + x.abs()))
    assert torch.allclose(OPS["Silu"]([x], {}), x * torch.sigmoid(x))
    assert torch.allclose(OPS["Celu"]([x], {"alpha": 2.0}), torch.clamp(x, min=0) + torch.clamp(2.0 * (torch.exp(x / 2.0) - 1), max=0))
    selu = OPS["Selu"]([x], {})
    assert selu[0, 4] == pytest.approx(2.0 * 1.0507009873554805) and selu[0, 0] == pytest.approx(1.0507009873554805 * 1.6732632423543772 * (math.exp(-1.5) - 1))
    assert OPS["ThresholdedRelu"]([x], {"alpha": 0.4}).tolist() == [[0.0, 0.0, 0.0, 0.0, 2.0]]
    assert OPS["Hardmax"]([torch.tensor([[1.0, 3.0, 3.0], [2.0, 0.0, 1.0]])], {}).tolist() == [[0.0, 1.0, 0.0], [1.0, 0.0, 0.0]]
    m = torch.tensor([[3.0, -4.0], [1.0, 2.0]])
    assert OPS["LpNormalization"]([m], {"axis": 1, "p": 2})[0].tolist() == pytest.approx([0.6, -0.8])
    assert OPS["LpNormalization"]([m], {"axis": 0, "p": 1})[:, 0].tolist() == pytest.approx([0.75, 0.25])
    assert OPS["ReduceL1"]([m, torch.tensor([1])], {"keepdims": 0}).tolist() == [7.0, 3.0]
    assert OPS["ReduceLogSum"]([m.abs(), torch.tensor([1])], {"keepdims": 0}).tolist() == pytest.approx([math.log(7.0), math.log(3.0)])
    assert OPS["ReduceLogSumExp"]([m], {"keepdims": 0}).item() == pytest.approx(math.log(sum(math.exp(v) for v in (3, -4, 1, 2))))
    img = torch.arange(16.0).reshape(1, 1, 4, 4) - 8
    assert OPS["GlobalLpPool"]([img], {"p": 2}).reshape(-1).item() == pytest.approx(float(img.pow(2).sum().sqrt()))
    lp = OPS["LpPool"]([img], {"kernel_shape": [2, 2], "strides": [2, 2], "p": 2})
    assert tuple(lp.shape) == (1, 1, 2, 2) and lp[0, 0, 0, 0].item() == pytest.approx(math.sqrt(64 + 49 + 16 + 9))
    assert OPS["EyeLike"]([torch.zeros(2, 3)], {"k": 1}).tolist() == [[0.0, 1.0, 0.0], [0.0, 0.0, 1.0]]
    seq = torch.tensor([1.0, 2.0, 3.0, 4.0])
    assert OPS["CumProd"]([seq, torch.tensor(0)], {}).tolist() == [1.0, 2.0, 6.0, 24.0]
    assert OPS["CumProd"]([seq, torch.tensor(0)], {"exclusive": 1}).tolist() == [1.0, 1.0, 2.0, 6.0]
    assert OPS["CumProd"]([seq, torch.tensor(0)], {"reverse": 1}).tolist() == [24.0, 24.0, 12.0, 4.0]
    assert OPS["Compress"]([m, torch.tensor([False, True])], {"axis": 1}).tolist() == [[-4.0], [2.0]]
    assert OPS["Compress"]([m, torch.tensor([True, False, True])], {}).tolist() == [3.0, 1.0]
    assert torch.allclose(OPS["FusedMatMulBias"]([m, m, torch.tensor([1.0, 2.0])], {}), m @ m + torch.tensor([1.0, 2.0]))
    assert torch.allclose(OPS["FusedGemm"]([m, m, torch.tensor([1.0, -50.0])], {"activation": "LeakyRelu", "activation_alpha": 0.5, "transB": 1}),
                          torch.nn.functional.leaky_relu(m @ m.T + torch.tensor([1.0, -50.0]), 0.5))
    with pytest.raises(GraphExecutionError, match="Bogus"):
        OPS["FusedGemm"]([m, m], {"activation": "Bogus"})


def test_unique_in_both_orders_and_along_an_axis():
    x = torch.tensor([2.0, 1.0, 1.0, 3.0, 4.0, 3.0])
    vals, first, inverse, counts = OPS["Unique"]([x], {})
    assert vals.tolist() == [1.0, 2.0, 3.0, 4.0] and first.tolist() == [1, 0, 3, 4] and inverse.tolist() == [1, 0, 0, 2, 3, 2] and counts.tolist() == [2, 1, 2, 1]
    vals, first, inverse, counts = OPS["Unique"]([x], {"sorted": 0})
    assert vals.tolist() == [2.0, 1.0, 3.0, 4.0] and first.tolist() == [0, 1, 3, 4] and inverse.tolist() == [0, 1, 1, 2, 3, 2] and counts.tolist() == [1, 2, 2, 1]
    rows = torch.tensor([[1, 0], [1, 0], [0, 2]])
    vals, first, inverse, counts = OPS["Unique"]([rows], {"axis": 0})
    assert vals.tolist() == [[0, 2], [1, 0]] and first.tolist() == [2, 0] and inverse.tolist() == [1, 1, 0] and counts.tolist() == [1, 2]


def test_linear_quantisation_round_trips():
    x = torch.tensor([[-1.0, 0.0, 0.26, 2.5, 100.0], [0.5, 1.5, 2.5, -2.5, -100.0]])
    q = OPS["QuantizeLinear"]([x, torch.tensor(0.5), torch.tensor(3, dtype=torch.uint8)], {})
    assert q.dtype == torch.uint8 and q.tolist() == [[1, 3, 4, 8, 203], [4, 6, 8, 0, 0]]           # half rounds to even; saturates
    d = OPS["DequantizeLinear"]([q, torch.tensor(0.5), torch.tensor(3, dtype=torch.uint8)], {})
    assert d.tolist() == [[-1.0, 0.0, 0.5, 2.5, 100.0], [0.5, 1.5, 2.5, -1.5, -1.5]]
    # one scale per row (axis 0), signed
    q = OPS["QuantizeLinear"]([x, torch.tensor([1.0, 0.5]), torch.tensor([0, 0], dtype=torch.int8)], {"axis": 0})
    assert q.tolist() == [[-1, 0, 0, 2, 100], [1, 3, 5, -5, -128]]
    # blocks of two along axis 1
    w = torch.tensor([[1, 2, 3, 4]], dtype=torch.int8)
    d = OPS["DequantizeLinear"]([w, torch.tensor([[1.0, 10.0]]), None], {"axis": 1, "block_size": 2})
    assert d.tolist() == [[1.0, 2.0, 30.0, 40.0]]
    y, scale, zp = OPS["DynamicQuantizeLinear"]([torch.tensor([0.0, 2.0, -1.0, 5.1])], {})
    assert scale.item() == pytest.approx(6.1 / 255) and zp.item() == round(1.0 / (6.1 / 255)) and y.dtype == torch.uint8
    assert torch.allclose((y.float() - zp.float()) * scale, torch.tensor([0.0, 2.0, -1.0, 5.1]), atol=scale.item())
    a = torch.tensor([[10, 20]], dtype=torch.uint8)
    b = torch.tensor([[1, 2], [3, 4]], dtype=torch.uint8)
    out = OPS["QLinearMatMul"]([a, torch.tensor(0.5), torch.tensor(0, dtype=torch.uint8), b, torch.tensor(2.0), torch.tensor(1, dtype=torch.uint8),
                                torch.tensor(1.0), torch.tensor(5, dtype=torch.uint8)], {})
    assert out.tolist() == [[5 + 40, 5 + 70]]                                          # (5, 10) @ ((0, 2), (4, 6)) = (40, 70), then the zero point


def test_windows_and_fourier_transform():
    n = 8
    k = np.arange(n)
    assert np.allclose(OPS["HannWindow"]([torch.tensor(n)], {}).numpy(), 0.5 - 0.5 * np.cos(2 * np.pi * k / n), atol=1e-6)
    assert np.allclose(OPS["HannWindow"]([torch.tensor(n)], {"periodic": 0}).numpy(), np.hanning(n), atol=1e-6)
    assert np.allclose(OPS["HammingWindow"]([torch.tensor(n)], {"periodic": 0}).numpy(), 25 / 46 - 21 / 46 * np.cos(2 * np.pi * k / (n - 1)), atol=1e-6)
    assert np.allclose(OPS["BlackmanWindow"]([torch.tensor(n)], {"periodic": 0}).numpy(), np.blackman(n), atol=1e-6)
    sig = torch.randn(2, 16, 1, generator=torch.Generator().manual_seed(0))
    full = OPS["DFT"]([sig], {})
    want = np.fft.fft(sig[..., 0].numpy(), axis=1)
    assert np.allclose(full[..., 0].numpy(), want.real, atol=1e-5) and np.allclose(full[..., 1].numpy(), want.imag, atol=1e-5)
    half = OPS["DFT"]([sig, None, torch.tensor(1)], {"onesided": 1})
    assert tuple(half.shape) == (2, 9, 2) and torch.allclose(half, full[:, :9], atol=1e-6)
    back = OPS["DFT"]([full], {"inverse": 1})
    assert torch.allclose(back[..., 0], sig[..., 0], atol=1e-5) and float(back[..., 1].abs().max()) < 1e-5
    padded = OPS["DFT"]([sig, torch.tensor(32)], {})
    assert tuple(padded.shape) == (2, 32, 2)
    with pytest.raises(GraphExecutionError, match="imaginary axis"):
        OPS["DFT"]([sig, None, torch.tensor(-1)], {})


def test_image_operators():
    img = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3, 4, 5)
    theta = torch.tensor([[[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]]]).repeat(2, 1, 1)
    grid = OPS["AffineGrid"]([theta, torch.tensor([2, 3, 4, 5])], {"align_corners": 1})
    assert torch.allclose(OPS["GridSample"]([img, grid], {"align_corners": 1}), img, atol=1e-4)        # the identity map samples the image itself
    flipped = OPS["GridSample"]([img, grid * torch.tensor([-1.0, 1.0])], {"align_corners": 1, "mode": "nearest"})
    assert torch.equal(flipped, img.flip(-1))
    crop = OPS["CenterCropPad"]([img, torch.tensor([2, 7])], {"axes": [2, 3]})
    assert tuple(crop.shape) == (2, 3, 2, 7) and torch.equal(crop[..., 1:6], img[:, :, 1:3]) and float(crop[..., 0].abs().max()) == 0.0
    cols = torch.nn.functional.unfold(img, (2, 2), stride=(2, 1))
    folded = OPS["Col2Im"]([cols, torch.tensor([4, 5]), torch.tensor([2, 2])], {"strides": [2, 1]})
    assert torch.equal(folded, torch.nn.functional.fold(cols, (4, 5), (2, 2), stride=(2, 1)))
    boxes = torch.tensor([[[0.0, 0.0, 1.0, 1.0], [0.0, 0.1, 1.0, 1.1], [0.0, -0.1, 1.0, 0.9], [0.0, 10.0, 1.0, 11.0], [0.0, 10.1, 1.0, 11.1], [0.0, 100.0, 1.0, 101.0]]])
    scores = torch.tensor([[[0.9, 0.75, 0.6, 0.95, 0.5, 0.3]]])
    keep = OPS["NonMaxSuppression"]([boxes, scores, torch.tensor([3]), torch.tensor([0.5]), torch.tensor([0.0])], {})
    assert keep.tolist() == [[0, 0, 3], [0, 0, 0], [0, 0, 5]]
    keep = OPS["NonMaxSuppression"]([boxes, scores, torch.tensor([3]), torch.tensor([0.5]), torch.tensor([0.4])], {})
    assert keep.tolist() == [[0, 0, 3], [0, 0, 0]]
    assert OPS["NonMaxSuppression"]([boxes, scores], {}).shape == (0, 3)


def test_operator_table_covers_the_names_the_reference_cpu_provider_registers():
    """Every quoted operator name in the reference's kernel registry has an entry here, save the listed exceptions."""
    import os
    import re

    ref = os.environ.get("OGB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
    path = os.path.join(ref, "crates", "onnx-runtime-ep-cpu", "src", "kernels", "mod.rs")
    if not os.path.exists(path):
        pytest.skip("the reference kernel registry is not available on this machine")
    with open(path, encoding="utf-8") as f:
        src = f.read()
    body = src[src.index("macro_rules! register_operator_group"):]
    body = body[: body.index("#[cfg(test)]")] if "#[cfg(test)]" in body else body
    names = set(re.findall(r'"([A-Z][A-Za-z0-9]+)"', body))
    assert len(names) > 150
    have = set(OPS) | {k.split("::")[1] for k in OPS if "::" in k} | {"If", "Loop", "Scan", "Constant", "Split"}
    not_built = {"CompressedSparseAttention"}           # stateful compressed-cache attention
    not_operators = {"TotallyFakeOp"}                    # a name the registry's own tests look up and expect to miss
    assert names - have - not_operators == not_built
