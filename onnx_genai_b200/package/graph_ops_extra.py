"""The long tail of the graph executor's operator table.

Operators that models around a decoder use now and then -- inverse trigonometry, the rarer activations and reductions,
linear quantisation, window functions and the discrete Fourier transform of audio front ends, grid sampling, box
suppression -- kept apart from the core table so that file stays readable.  Importing this module adds them to
``graph_executor.OPS``.  The reference registers the same names on its CPU provider
(crates/onnx-runtime-ep-cpu/src/kernels/mod.rs, the ``register_*_ops`` groups).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import onnx_pb
from .graph_executor import _TORCH_DTYPE, OPS, GraphExecutionError, _opt, _reduce


def _scalar(t, default=None):
    return default if t is None else t.reshape(-1)[0].item()


# ---- quantisation -----------------------------------------------------------------------------------------------------
_QRANGE = {torch.uint8: (0, 255), torch.int8: (-128, 127), torch.int16: (-32768, 32767), torch.int32: (-2 ** 31, 2 ** 31 - 1)}


def _per_axis(t, x, axis, block):
    """Broadcast a scale / zero point against ``x``: a scalar, one value per slice of ``axis``, or one per block of it."""
    if t.numel() == 1:
        return t.reshape(())
    if t.dim() == 1:
        shape = [1] * x.dim()
        shape[axis % x.dim()] = -1
        return t.reshape(shape)
    if block:
        return t.repeat_interleave(block, dim=axis % x.dim()).narrow(axis % x.dim(), 0, x.shape[axis % x.dim()])
    return t


def _dequantize_linear(ins, attrs):
    x, scale, zp = ins[0], ins[1], _opt(ins, 2)
    axis, block = int(attrs.get("axis", 1)), int(attrs.get("block_size", 0))
    xf = x.float()
    if zp is not None:
        xf = xf - _per_axis(zp.float(), x, axis, block)
    return (xf * _per_axis(scale.float(), x, axis, block)).to(scale.dtype)


def _quantize_linear(ins, attrs):
    x, scale, zp = ins[0], ins[1], _opt(ins, 2)
    axis, block = int(attrs.get("axis", 1)), int(attrs.get("block_size", 0))
    out_dtype = zp.dtype if zp is not None else _TORCH_DTYPE.get(int(attrs.get("output_dtype", 0)) or onnx_pb.UINT8, torch.uint8)
    y = x.float() / _per_axis(scale.float(), x, axis, block)
    if out_dtype in _QRANGE:
        lo, hi = _QRANGE[out_dtype]
        y = torch.round(y)                                                  # half to even, as the operator says
        if zp is not None:
            y = y + _per_axis(zp.float(), x, axis, block)
        return y.clamp(lo, hi).to(out_dtype)
    return y.to(out_dtype)                                                   # float8 targets saturate in the cast


def _dynamic_quantize_linear(ins, attrs):
    x = ins[0].float()
    lo, hi = min(float(x.min()), 0.0), max(float(x.max()), 0.0)
    scale = (hi - lo) / 255.0 or 1.0
    zp = float(min(max(round(-lo / scale), 0), 255))
    y = (torch.round(x / scale) + zp).clamp(0, 255).to(torch.uint8)
    return [y, torch.tensor(scale, dtype=torch.float32, device=x.device), torch.tensor(int(zp), dtype=torch.uint8, device=x.device)]


def _qlinear_matmul(ins, attrs):
    a, a_s, a_z, b, b_s, b_z, y_s, y_z = ins[:8]
    af = (a.float() - a_z.float()) * a_s.float()
    bf = (b.float() - _per_axis(b_z.float(), b, -1, 0)) * _per_axis(b_s.float(), b, -1, 0)
    lo, hi = _QRANGE[y_z.dtype]
    return (torch.round(af @ bf / y_s.float()) + y_z.float()).clamp(lo, hi).to(y_z.dtype)


# ---- signal ------------------------------------------------------------------------------------------------------------
def _window(coeffs):
    def run(ins, attrs):
        n = int(_scalar(ins[0]))
        denom = n if int(attrs.get("periodic", 1)) else max(n - 1, 1)
        k = torch.arange(n, dtype=torch.float64, device=ins[0].device)
        w = sum(c * torch.cos(2 * math.pi * h * k / denom) for h, c in enumerate(coeffs))
        return w.to(_TORCH_DTYPE.get(int(attrs.get("output_datatype", onnx_pb.FLOAT)), torch.float32))
    return run


def _dft(ins, attrs):
    """DFT: the last axis holds 1 (real) or 2 (real, imaginary) values; opset 20 passes the axis as an input."""
    x = ins[0]
    length = _opt(ins, 1)
    axis_in = _opt(ins, 2)
    axis = int(_scalar(axis_in)) if axis_in is not None else int(attrs.get("axis", -2))
    axis = axis % x.dim()
    if axis == x.dim() - 1:
        raise GraphExecutionError("DFT cannot transform the real / imaginary axis")
    z = torch.complex(x[..., 0].double(), x[..., 1].double()) if x.shape[-1] == 2 else x[..., 0].double().to(torch.complex128)
    n = int(_scalar(length)) if length is not None else z.shape[axis]
    inverse, onesided = bool(attrs.get("inverse", 0)), bool(attrs.get("onesided", 0))
    if inverse and onesided:
        raise GraphExecutionError("DFT: inverse and onesided cannot both be set")
    out = torch.fft.ifft(z, n=n, dim=axis) if inverse else torch.fft.fft(z, n=n, dim=axis)
    if onesided:
        out = out.narrow(axis, 0, n // 2 + 1)
    return torch.view_as_real(out).to(x.dtype)


# ---- images -------------------------------------------------------------------------------------------------------------
def _grid_sample(ins, attrs):
    mode = {"linear": "bilinear", "cubic": "bicubic"}.get(attrs.get("mode", "linear"), attrs.get("mode", "linear"))
    return F.grid_sample(ins[0], ins[1].to(ins[0].dtype), mode=mode, padding_mode=attrs.get("padding_mode", "zeros"),
                         align_corners=bool(attrs.get("align_corners", 0)))


def _affine_grid(ins, attrs):
    return F.affine_grid(ins[0], [int(v) for v in ins[1].reshape(-1).tolist()], align_corners=bool(attrs.get("align_corners", 0)))


def _center_crop_pad(ins, attrs):
    x, shape = ins[0], [int(v) for v in ins[1].reshape(-1).tolist()]
    axes = [a % x.dim() for a in (attrs.get("axes") or range(x.dim()))]
    for axis, want in zip(axes, shape):
        have = x.shape[axis]
        if have > want:
            x = x.narrow(axis, (have - want) // 2, want)
        elif have < want:
            before = (want - have) // 2
            pad = [0, 0] * x.dim()
            pad[2 * (x.dim() - 1 - axis)], pad[2 * (x.dim() - 1 - axis) + 1] = before, want - have - before
            x = F.pad(x, pad)
    return x


def _lp_pool(ins, attrs):
    x, p = ins[0], float(attrs.get("p", 2))
    kernel = [int(k) for k in attrs["kernel_shape"]]
    strides = [int(s) for s in attrs.get("strides") or [1] * len(kernel)]
    pads = [int(v) for v in attrs.get("pads") or [0] * (2 * len(kernel))]
    half = len(kernel)
    padded = F.pad(x.abs().pow(p), [v for d in reversed(range(half)) for v in (pads[d], pads[d + half])])
    pool = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[half]
    return (pool(padded, kernel, strides, ceil_mode=bool(attrs.get("ceil_mode", 0))) * float(math.prod(kernel))).pow(1.0 / p)


def _col2im(ins, attrs):
    x, image, block = ins[0], [int(v) for v in ins[1].reshape(-1).tolist()], [int(v) for v in ins[2].reshape(-1).tolist()]
    if len(image) != 2:
        raise GraphExecutionError("Col2Im is covered for two spatial dimensions")
    pads = [int(v) for v in attrs.get("pads") or [0, 0, 0, 0]]
    if pads[0] != pads[2] or pads[1] != pads[3]:
        raise GraphExecutionError("Col2Im is covered for symmetric padding")
    return F.fold(x, image, block, dilation=[int(v) for v in attrs.get("dilations") or [1, 1]], padding=pads[:2],
                  stride=[int(v) for v in attrs.get("strides") or [1, 1]])


def _nms(ins, attrs):
    """NonMaxSuppression -> [selected, 3] rows of (batch, class, box), classes in order, boxes by falling score."""
    boxes, scores = ins[0].float(), ins[1].float()
    limit = int(_scalar(_opt(ins, 2), 0))
    iou_thr = float(_scalar(_opt(ins, 3), 0.0))
    score_thr = _scalar(_opt(ins, 4))
    if limit == 0:
        return torch.zeros(0, 3, dtype=torch.int64, device=boxes.device)
    if int(attrs.get("center_point_box", 0)):
        cx, cy, w, h = boxes.unbind(-1)
        x1, y1, x2, y2 = cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2
    else:
        ya, xa, yb, xb = boxes.unbind(-1)
        x1, x2, y1, y2 = torch.minimum(xa, xb), torch.maximum(xa, xb), torch.minimum(ya, yb), torch.maximum(ya, yb)
    area = (x2 - x1) * (y2 - y1)
    rows = []
    for b in range(scores.shape[0]):
        for c in range(scores.shape[1]):
            s = scores[b, c]
            order = torch.argsort(-s, stable=True).tolist()
            kept: list = []
            for i in order:
                if score_thr is not None and float(s[i]) <= score_thr:
                    break
                ok = True
                for j in kept:
                    iw = float(torch.minimum(x2[b, i], x2[b, j]) - torch.maximum(x1[b, i], x1[b, j]))
                    ih = float(torch.minimum(y2[b, i], y2[b, j]) - torch.maximum(y1[b, i], y1[b, j]))
                    inter = max(iw, 0.0) * max(ih, 0.0)
                    union = float(area[b, i] + area[b, j]) - inter
                    if union > 0 and inter / union > iou_thr:
                        ok = False
                        break
                if ok:
                    kept.append(i)
                    if len(kept) == limit:
                        break
            rows += [[b, c, i] for i in kept]
    return torch.tensor(rows, dtype=torch.int64, device=boxes.device).reshape(-1, 3)


# ---- sets and indexing ----------------------------------------------------------------------------------------------------
def _unique(ins, attrs):
    """Unique -> (values, first-occurrence indices, inverse, counts), sorted or in order of first appearance."""
    x = ins[0]
    axis = attrs.get("axis")
    if axis is None:
        flat, dim = x.reshape(-1), 0
    else:
        flat, dim = x, int(axis) % x.dim()
    vals, inverse, counts = torch.unique(flat, sorted=True, return_inverse=True, return_counts=True, dim=dim)
    n = vals.shape[dim]
    positions = torch.arange(inverse.numel(), device=x.device)
    first = torch.full((n,), inverse.numel(), dtype=torch.int64, device=x.device).scatter_reduce(0, inverse.reshape(-1), positions, "amin")
    if not int(attrs.get("sorted", 1)):
        order = torch.argsort(first)
        rank = torch.empty_like(order)
        rank[order] = torch.arange(n, device=x.device)
        vals, first, counts, inverse = vals.index_select(dim, order), first[order], counts[order], rank[inverse]
    return [vals, first, inverse.reshape(-1), counts]


def _compress(ins, attrs):
    x, cond = ins[0], ins[1].bool().reshape(-1)
    axis = attrs.get("axis")
    if axis is None:
        flat = x.reshape(-1)
        return flat[: cond.numel()][cond[: flat.numel()]]
    axis = int(axis) % x.dim()
    idx = torch.nonzero(cond[: x.shape[axis]]).reshape(-1)
    return x.index_select(axis, idx)


def _eye_like(ins, attrs):
    x = ins[0]
    dt = _TORCH_DTYPE.get(int(attrs["dtype"]), x.dtype) if "dtype" in attrs else x.dtype
    return torch.diag(torch.ones(max(x.shape), dtype=dt, device=x.device), int(attrs.get("k", 0)))[: x.shape[0], : x.shape[1]].contiguous()


def _cumprod(ins, attrs):
    x, axis = ins[0], int(_scalar(ins[1]))
    if attrs.get("reverse", 0):
        x = x.flip(axis)
    y = torch.cumprod(x, axis)
    if attrs.get("exclusive", 0):
        y = torch.cat([torch.ones_like(y.narrow(axis, 0, 1)), y.narrow(axis, 0, y.shape[axis] - 1)], dim=axis)
    return y.flip(axis) if attrs.get("reverse", 0) else y


def _hardmax(ins, attrs):
    x, axis = ins[0], int(attrs.get("axis", -1))
    return torch.zeros_like(x).scatter_(axis, x.argmax(dim=axis, keepdim=True), 1.0)     # argmax picks the first of equal maxima


def _fused_gemm(ins, attrs):
    """com.microsoft::FusedGemm: Gemm followed by the activation named in ``activation``."""
    y = OPS["Gemm"](ins, attrs)
    act = attrs.get("activation", "")
    if not act:
        return y
    if act not in OPS:
        raise GraphExecutionError(f"FusedGemm activation {act!r} is not covered")
    inner = {k[len("activation_"):]: v for k, v in attrs.items() if k.startswith("activation_")}
    return OPS[act]([y], inner)


OPS.update({
    "Acos": lambda i, a: i[0].acos(), "Acosh": lambda i, a: i[0].acosh(), "Asin": lambda i, a: i[0].asin(), "Asinh": lambda i, a: i[0].asinh(),
    "Atan": lambda i, a: i[0].atan(), "Atanh": lambda i, a: i[0].atanh(), "Cosh": lambda i, a: i[0].cosh(), "Sinh": lambda i, a: i[0].sinh(),
    "Tan": lambda i, a: i[0].tan(), "Softsign": lambda i, a: i[0] / (1 + i[0].abs()), "Silu": lambda i, a: F.silu(i[0]),
    "Celu": lambda i, a: F.celu(i[0], float(a.get("alpha", 1.0))),
    "Selu": lambda i, a: float(a.get("gamma", 1.0507009873554805)) * torch.where(
        i[0] > 0, i[0], float(a.get("alpha", 1.6732632423543772)) * (i[0].exp() - 1)),
    "ThresholdedRelu": lambda i, a: torch.where(i[0] > float(a.get("alpha", 1.0)), i[0], torch.zeros_like(i[0])),
    "Hardmax": _hardmax,
    "LpNormalization": lambda i, a: i[0] / i[0].abs().pow(int(a.get("p", 2))).sum(int(a.get("axis", -1)), keepdim=True).pow(1.0 / int(a.get("p", 2))),
    "ReduceL1": _reduce(lambda x, ax, k: x.abs().sum(ax, keepdim=k)),
    "ReduceLogSum": _reduce(lambda x, ax, k: x.sum(ax, keepdim=k).log()),
    "ReduceLogSumExp": _reduce(lambda x, ax, k: torch.logsumexp(x, ax, keepdim=k)),
    "GlobalLpPool": lambda i, a: i[0].abs().pow(float(a.get("p", 2))).sum(tuple(range(2, i[0].dim())), keepdim=True).pow(1.0 / float(a.get("p", 2))),
    "LpPool": _lp_pool, "EyeLike": _eye_like, "CumProd": _cumprod, "Compress": _compress, "Unique": _unique,
    "DequantizeLinear": _dequantize_linear, "QuantizeLinear": _quantize_linear, "DynamicQuantizeLinear": _dynamic_quantize_linear,
    "QLinearMatMul": _qlinear_matmul,
    "HannWindow": _window((0.5, -0.5)), "HammingWindow": _window((25.0 / 46.0, -21.0 / 46.0)), "BlackmanWindow": _window((0.42, -0.5, 0.08)),
    "DFT": _dft, "GridSample": _grid_sample, "AffineGrid": _affine_grid, "CenterCropPad": _center_crop_pad, "Col2Im": _col2im,
    "NonMaxSuppression": _nms, "FusedGemm": _fused_gemm,
    "FusedMatMulBias": lambda i, a: i[0] @ i[1] + (i[2] if len(i) > 2 and i[2] is not None else 0),
})
