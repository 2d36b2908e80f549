"""Generic ONNX graph execution for the models around the decoder: encoders, projectors, VAEs, policies.

The decoder itself runs on this package's own kernels and step executor.  A multi-model package also carries graphs
that are not decoders -- a vision tower, an audio encoder, a text encoder, a denoiser, a VAE, small policy graphs
(schedules, solvers, predicates) -- and the workflow runtime needs to call them.  :class:`GraphExecutor` interprets
such a graph node by node in topological order over torch tensors on any device: the role of the reference's
sequential executor over its CPU / CUDA operator registries for graphs outside the decode fast path
(crates/onnx-runtime-session/src/executor/mod.rs; operator coverage crates/onnx-runtime-ep-cpu/src/lib.rs).  These
graphs are off the token loop (they run once per request or per denoising step), so library tensor operations are the
right tool; nothing here is used by the decoder.

Coverage: the dense, convolutional, normalisation, activation, shape and indexing operators of the default domain
that such graphs use (see ``OPS``), plus the ``com.microsoft`` contrib forms ``Gelu``, ``FastGelu``, ``BiasGelu``,
``SkipLayerNormalization``, ``SimplifiedLayerNormalization``, ``SkipSimplifiedLayerNormalization``, ``GroupQueryAttention``
(separate past / present buffers), the attention family, ``MatMulNBits`` and the mixture-of-experts operators; the long
tail lives in ``graph_ops_extra`` and the operators of hybrid and padding-free decoders in ``graph_ops_sequence``.
``If``, ``Loop`` and ``Scan`` run their subgraphs in a scope chained over the enclosing one (bodies may read outer values
by name).  An operator outside the table is an error that names the node and lists what is covered.

``as_component(path)`` wraps a graph as a workflow component: a callable from a dict of input ports to a dict of
output ports (ports are the graph's input and output names).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from . import onnx_pb

_TORCH_DTYPE = {onnx_pb.FLOAT: torch.float32, onnx_pb.UINT8: torch.uint8, onnx_pb.INT8: torch.int8, onnx_pb.INT16: torch.int16,
                onnx_pb.INT32: torch.int32, onnx_pb.INT64: torch.int64, onnx_pb.BOOL: torch.bool, onnx_pb.FLOAT16: torch.float16,
                onnx_pb.DOUBLE: torch.float64, onnx_pb.BFLOAT16: torch.bfloat16}


class GraphExecutionError(RuntimeError):
    pass


def _signed_home(arr):
    """Unsigned 16/32/64-bit arrays move to the signed type that holds them (torch computes on signed integers only)."""
    if arr.dtype == np.uint16:
        return arr.astype(np.int32)
    if arr.dtype in (np.uint32, np.uint64):
        return arr.astype(np.int64)
    return arr


def tensor_to_torch(t: onnx_pb.Tensor, device="cpu") -> torch.Tensor:
    arr = np.ascontiguousarray(t.numpy())
    if t.data_type == onnx_pb.BFLOAT16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16).reshape(tuple(t.dims)).to(device)
    if t.data_type == onnx_pb.FLOAT8E4M3FN:
        return torch.from_numpy(arr.copy()).view(torch.float8_e4m3fn).reshape(tuple(t.dims)).to(device)
    return torch.from_numpy(_signed_home(arr).copy()).reshape(tuple(t.dims)).to(device)


def _ints(x):
    if isinstance(x, torch.Tensor):
        return [int(v) for v in x.reshape(-1).tolist()]
    return [int(v) for v in x]


def _axis_list(attrs, ins, idx=1, name="axes"):
    if len(ins) > idx and ins[idx] is not None:
        return _ints(ins[idx])
    v = attrs.get(name)
    return None if v in (None, 0, []) and name not in attrs else _ints(v if isinstance(v, (list, tuple)) else [v])


def _pads(attrs, nd, x_shape=None, kernel=None, strides=None, dilations=None):
    auto = attrs.get("auto_pad", "NOTSET")
    if auto in ("SAME_UPPER", "SAME_LOWER"):
        pads_b, pads_e = [], []
        for i in range(nd):
            out = math.ceil(x_shape[i] / strides[i])
            total = max(0, (out - 1) * strides[i] + (kernel[i] - 1) * dilations[i] + 1 - x_shape[i])
            lo = total // 2 if auto == "SAME_UPPER" else total - total // 2
            pads_b.append(lo)
            pads_e.append(total - lo)
        return pads_b, pads_e
    p = _ints(attrs.get("pads") or [0] * (2 * nd))
    return p[:nd], p[nd:]


def _conv(ins, attrs, transpose=False):
    x, w = ins[0], ins[1]
    b = ins[2] if len(ins) > 2 else None
    nd = x.dim() - 2
    strides = _ints(attrs.get("strides") or [1] * nd)
    dil = _ints(attrs.get("dilations") or [1] * nd)
    group = int(attrs.get("group", 1) or 1)
    kernel = list(w.shape[2:])
    pb, pe = _pads(attrs, nd, list(x.shape[2:]), kernel, strides, dil)
    fn = {1: (F.conv1d, F.conv_transpose1d), 2: (F.conv2d, F.conv_transpose2d), 3: (F.conv3d, F.conv_transpose3d)}[nd][int(transpose)]
    if transpose:
        if pb != pe:
            raise GraphExecutionError("ConvTranspose with asymmetric pads is not covered")
        out_pad = _ints(attrs.get("output_padding") or [0] * nd)
        return fn(x, w, b, stride=strides, padding=pb, output_padding=out_pad, groups=group, dilation=dil)
    if pb != pe:
        flat = []
        for i in reversed(range(nd)):
            flat += [pb[i], pe[i]]
        x, pb = F.pad(x, flat), [0] * nd
    return fn(x, w, b, stride=strides, padding=pb, dilation=dil, groups=group)


def _pool(ins, attrs, kind):
    x = ins[0]
    nd = x.dim() - 2
    k = _ints(attrs["kernel_shape"])
    strides = _ints(attrs.get("strides") or [1] * nd)
    dil = _ints(attrs.get("dilations") or [1] * nd)
    pb, pe = _pads(attrs, nd, list(x.shape[2:]), k, strides, dil)
    ceil = bool(attrs.get("ceil_mode", 0))
    if pb != pe:
        flat = []
        for i in reversed(range(nd)):
            flat += [pb[i], pe[i]]
        x, pb = F.pad(x, flat, value=float("-inf") if kind == "max" else 0.0), [0] * nd
    if kind == "max":
        return {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd](x, k, strides, pb, dil, ceil)
    include = bool(attrs.get("count_include_pad", 0))
    return {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd](x, k, strides, pb, ceil, include)


def _layer_norm(x, scale, bias, axis, eps):
    dims = tuple(range(axis % x.dim(), x.dim()))
    xf = x.float()
    mean = xf.mean(dims, keepdim=True)
    var = (xf - mean).pow(2).mean(dims, keepdim=True)
    inv = torch.rsqrt(var + eps)
    y = ((xf - mean) * inv).to(x.dtype) * scale
    return [y + bias if bias is not None else y, mean, inv]          # Y, then the optional Mean and InvStdDev outputs


def _rms_norm(x, scale, axis, eps):
    dims = tuple(range(axis % x.dim(), x.dim()))
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dims, keepdim=True) + eps)).to(x.dtype) * scale


def _rms_norm_with_stat(x, scale, axis, eps):
    """The contrib form's optional second output is the inverse root mean square it divided by."""
    dims = tuple(range(axis % x.dim(), x.dim()))
    return [_rms_norm(x, scale, axis, eps), torch.rsqrt(x.float().pow(2).mean(dims, keepdim=True) + eps)]


def _slice(ins, attrs):
    x = ins[0]
    if len(ins) > 1:
        starts, ends = _ints(ins[1]), _ints(ins[2])
        axes = _ints(ins[3]) if len(ins) > 3 and ins[3] is not None else list(range(len(starts)))
        steps = _ints(ins[4]) if len(ins) > 4 and ins[4] is not None else [1] * len(starts)
    else:
        starts, ends = _ints(attrs["starts"]), _ints(attrs["ends"])
        axes = _ints(attrs.get("axes") or list(range(len(starts))))
        steps = [1] * len(starts)
    for s, e, a, st in zip(starts, ends, axes, steps):
        a %= x.dim()
        sel = range(*slice(s, e, st).indices(x.shape[a]))          # the operator clamps exactly as Python slicing does
        if st > 0:
            x = x.narrow(a, sel.start, len(sel)) if st == 1 else x.index_select(a, torch.tensor(list(sel), dtype=torch.long, device=x.device))
        else:
            x = x.index_select(a, torch.tensor(list(sel), dtype=torch.long, device=x.device))
    return x


def _squeeze(ins, attrs):
    x, axes = ins[0], _axis_list(attrs, ins)
    if axes is None:
        return x.squeeze()
    drop = {a % x.dim() for a in axes}
    return x.reshape([s for d, s in enumerate(x.shape) if d not in drop])


def _unsqueeze(ins, attrs):
    x, axes = ins[0], _axis_list(attrs, ins)
    nd = x.dim() + len(axes)
    for d in sorted(a % nd for a in axes):
        x = x.unsqueeze(d)
    return x


def _resize(ins, attrs):
    x = ins[0]
    scales = ins[2] if len(ins) > 2 and ins[2] is not None and ins[2].numel() else None
    sizes = ins[3] if len(ins) > 3 and ins[3] is not None and ins[3].numel() else None
    mode = attrs.get("mode", "nearest")
    nd = x.dim() - 2
    tmode = {"nearest": "nearest", "linear": {1: "linear", 2: "bilinear", 3: "trilinear"}[nd], "cubic": "bicubic"}[mode]
    ctm = attrs.get("coordinate_transformation_mode", "half_pixel")
    kw = {}
    if tmode != "nearest":
        kw["align_corners"] = ctm == "align_corners"
    if sizes is not None:
        return F.interpolate(x, size=_ints(sizes)[2:], mode=tmode, **kw)
    return F.interpolate(x, scale_factor=[float(s) for s in scales.reshape(-1).tolist()][2:], mode=tmode, **kw)


def _matmul_nbits(ins, attrs):
    """com.microsoft::MatMulNBits (4-bit, block-wise): y = x @ dequant(B)^T."""
    x, packed, scales = ins[0], ins[1], ins[2]
    zp = ins[3] if len(ins) > 3 and ins[3] is not None else None
    k, n, block = int(attrs["K"]), int(attrs["N"]), int(attrs["block_size"])
    if int(attrs.get("bits", 4)) != 4:
        raise GraphExecutionError("MatMulNBits is covered for bits=4 only")
    p = packed.reshape(n, -1).to(torch.int32)
    lo, hi = p & 0xF, (p >> 4) & 0xF
    blocks = (k + block - 1) // block
    q = torch.stack([lo, hi], dim=-1).reshape(n, blocks, block).float()       # K is padded to whole blocks in storage
    s = scales.reshape(n, blocks).float()
    if zp is not None:
        z = zp.reshape(n, -1).to(torch.int32)
        z = torch.stack([z & 0xF, (z >> 4) & 0xF], dim=-1).reshape(n, -1)[:, :blocks].float()
    else:
        z = torch.full((n, blocks), 8.0, device=x.device)
    w = (q - z[..., None]) * s[..., None]
    y = x.float() @ w.reshape(n, -1)[:, :k].T
    if len(ins) > 5 and ins[5] is not None:
        y = y + ins[5].float()
    return y.to(x.dtype)


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_IQ4_NL = (-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113)
_BLOCK_FORMATS = {"mxfp4": (32, 17), "iq4_nl": (32, 18), "iq4_xs": (256, 136)}        # values per block, bytes per block


def decode_weight_blocks(packed, fmt: str):
    """[n, blocks, bytes] uint8 -> [n, blocks * values per block] float32 for the block formats of ``BlockQuantizedMatMul``.

    ``mxfp4``: one E8M0 scale byte (2^(e-127); 255 is NaN) then 16 bytes of E2M1 codes, where byte ``j`` holds element
    ``j`` in its low nibble and element ``j + 16`` in its high nibble.  ``iq4_nl``: a little-endian fp16 scale then 16
    bytes laid out the same way, the codes indexing the 16-entry non-linear table.  ``iq4_xs``: super-blocks of 256
    values in 136 bytes -- fp16 scale d, 16 bits holding the two high bits of eight 6-bit sub-block scales, 4 bytes holding
    their low nibbles, then 128 bytes of codes for eight sub-blocks of 32 (16 bytes each, low nibble = element j, high
    nibble = element j + 16); a sub-block's values are d * (scale - 32) * table[code].
    """
    if fmt not in _BLOCK_FORMATS:
        raise GraphExecutionError(f"BlockQuantizedMatMul format {fmt!r} is not covered here (covered: {sorted(_BLOCK_FORMATS)})")
    qk, nbytes = _BLOCK_FORMATS[fmt]
    if packed.dim() != 3 or packed.shape[-1] != nbytes:
        raise GraphExecutionError(f"{fmt} weights must be [N, blocks, {nbytes}] bytes, got {list(packed.shape)}")
    b = packed.to(torch.int32)
    if fmt == "iq4_xs":
        d = (b[..., 0] | (b[..., 1] << 8)).to(torch.int16).view(torch.float16).float()                       # [n, blocks]
        high = b[..., 2] | (b[..., 3] << 8)
        sub = torch.arange(8, device=packed.device)
        low = (b[..., 4:8][..., sub // 2] >> (4 * (sub % 2))) & 0xF                                           # [n, blocks, 8]
        ls = low | (((high[..., None] >> (2 * sub)) & 3) << 4)
        dl = d[..., None] * (ls - 32).float()
        q = b[..., 8:].reshape(*b.shape[:2], 8, 16)
        idx = torch.cat([q & 0xF, (q >> 4) & 0xF], dim=-1).long()                                             # [n, blocks, 8, 32]
        vals = torch.tensor(_IQ4_NL, device=packed.device, dtype=torch.float32)[idx] * dl[..., None]
        return vals.reshape(packed.shape[0], -1)
    head = 1 if fmt == "mxfp4" else 2
    codes = b[..., head:]
    idx = torch.cat([codes & 0xF, (codes >> 4) & 0xF], dim=-1).long()
    if fmt == "mxfp4":
        e = b[..., 0]
        scale = torch.where(e == 255, torch.full_like(e, float("nan"), dtype=torch.float64), torch.pow(2.0, (e - 127).double())).float()
        table = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), device=packed.device)
        vals = table[idx]
        vals = torch.where(vals == 0, torch.zeros_like(vals), vals * scale[..., None])      # a zero code stays zero under a NaN scale
    else:
        raw = (b[..., 0] | (b[..., 1] << 8)).to(torch.int16).view(torch.float16).float()
        vals = torch.tensor(_IQ4_NL, device=packed.device, dtype=torch.float32)[idx] * raw[..., None]
    return vals.reshape(packed.shape[0], -1)


def encode_mxfp4(weight):
    """[n, k] float -> [n, ceil(k/32), 17] uint8 in the ``mxfp4`` block layout (nearest code, power-of-two block scale)."""
    w = weight.detach().float().cpu()
    n, k = w.shape
    blocks = (k + 31) // 32
    w = F.pad(w, (0, blocks * 32 - k)).reshape(n, blocks, 32)
    amax = w.abs().amax(-1).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scaled = w / torch.pow(2.0, e)[..., None]
    table = torch.tensor(_E2M1)
    mag = (scaled.abs()[..., None] - table).abs().argmin(-1)
    code = (mag | ((scaled < 0) & (mag > 0)).long() << 3).to(torch.uint8)
    out = torch.empty(n, blocks, 17, dtype=torch.uint8)
    out[..., 0] = (e + 127).to(torch.uint8)
    out[..., 1:] = code[..., :16] | (code[..., 16:] << 4)
    return out


def _block_quantized_matmul(ins, attrs):
    """pkg.nxrt::BlockQuantizedMatMul: y = A @ dequant(packed_B)^T (+ bias), A [..., K], packed_B [N, blocks, block bytes].

    The reference runs it on its CPU provider (crates/onnx-runtime-ep-cpu/src/kernels/block_quantized_matmul.rs:170-300);
    a partial last block is stored whole and its tail ignored.
    """
    x, packed = ins[0], ins[1]
    k, n = int(attrs["K"]), int(attrs["N"])
    if int(attrs.get("block_layout_version", 1)) != 1:
        raise GraphExecutionError(f"BlockQuantizedMatMul block_layout_version {attrs.get('block_layout_version')} is unknown (known: 1)")
    fmt = attrs.get("format")
    fmt = fmt.decode() if isinstance(fmt, bytes) else fmt
    if x.shape[-1] != k or packed.shape[0] != n:
        raise GraphExecutionError(f"BlockQuantizedMatMul: A {list(x.shape)} / packed_B {list(packed.shape)} do not match K={k}, N={n}")
    w = decode_weight_blocks(packed, str(fmt))[:, :k]
    y = x.float() @ w.T
    if len(ins) > 2 and ins[2] is not None:
        y = y + ins[2].float()
    return y.to(x.dtype)


def _topk(x, k, axis, largest):
    """TopK with the operator's tie rule: among equal values the lower index comes first (``torch.topk`` promises no
    order among ties, and gated scores -- a ReLU's exact zeros -- tie often)."""
    order = torch.argsort(x, dim=axis, descending=largest, stable=True).narrow(axis, 0, k)
    return [torch.gather(x, axis, order), order]


def _gather_nd(data, idx):
    idx = idx.long()
    k = idx.shape[-1]
    flat = idx.reshape(-1, k)
    out = data[tuple(flat[:, i] for i in range(k))]
    return out.reshape(tuple(idx.shape[:-1]) + tuple(data.shape[k:]))


def _reduce(fn):
    def run(ins, attrs):
        x = ins[0]
        axes = _axis_list(attrs, ins)
        keep = bool(attrs.get("keepdims", 1))
        if axes is None or len(axes) == 0:
            if attrs.get("noop_with_empty_axes", 0):
                return x
            axes = list(range(x.dim()))
        return fn(x, tuple(a % x.dim() for a in axes), keep)
    return run


def _constant(ins, attrs, device):
    if "value" in attrs:
        return tensor_to_torch(attrs["value"], device)
    for key, dt in (("value_float", torch.float32), ("value_int", torch.int64)):
        if key in attrs:
            return torch.tensor(attrs[key], dtype=dt, device=device)
    for key, dt in (("value_floats", torch.float32), ("value_ints", torch.int64)):
        if key in attrs:
            return torch.tensor(list(attrs[key]), dtype=dt, device=device)
    raise GraphExecutionError("Constant without a value attribute")


def _pad(ins, attrs):
    x = ins[0]
    pads = _ints(ins[1]) if len(ins) > 1 else _ints(attrs["pads"])
    value = float(ins[2].reshape(-1)[0]) if len(ins) > 2 and ins[2] is not None and ins[2].numel() else float(attrs.get("value", 0.0))
    axes = _ints(ins[3]) if len(ins) > 3 and ins[3] is not None else list(range(x.dim()))
    lo, hi = [0] * x.dim(), [0] * x.dim()
    for i, a in enumerate(axes):
        lo[a % x.dim()], hi[a % x.dim()] = pads[i], pads[i + len(axes)]
    flat = []
    for d in reversed(range(x.dim())):
        flat += [lo[d], hi[d]]
    mode = attrs.get("mode", "constant")
    while len(flat) > 2 and flat[-1] == 0 and flat[-2] == 0:       # leading dimensions without padding need not be listed
        flat = flat[:-2]
    if mode == "constant":
        return F.pad(x, flat, value=value)
    return F.pad(x, flat, mode={"reflect": "reflect", "edge": "replicate", "wrap": "circular"}[mode])


def _split(ins, attrs, n_out):
    x = ins[0]
    axis = int(attrs.get("axis", 0))
    if len(ins) > 1 and ins[1] is not None:
        sizes = _ints(ins[1])
    elif "split" in attrs:
        sizes = _ints(attrs["split"])
    else:
        per = -(-x.shape[axis] // n_out)
        sizes = [min(per, x.shape[axis] - i * per) for i in range(n_out)]
    return list(torch.split(x, sizes, dim=axis))


def _expand(x, shape):
    shape = _ints(shape)
    nd = max(len(shape), x.dim())
    xs = [1] * (nd - x.dim()) + list(x.shape)
    ss = [1] * (nd - len(shape)) + shape
    return x.reshape(xs).expand([max(a, b) for a, b in zip(xs, ss)])


def _reshape(x, shape, allowzero=0):
    shape = _ints(shape)
    if not allowzero:
        shape = [x.shape[i] if s == 0 else s for i, s in enumerate(shape)]
    return x.reshape(shape)


def _rotary(ins, attrs):
    """RotaryEmbedding (opset 23): X is [B, S, H*D] (with ``num_heads``) or [B, H, S, D]; caches are [positions, rot/2]
    when position ids are given, else already gathered [B, S, rot/2]."""
    x, cos, sin = ins[0], ins[1], ins[2]
    pos = ins[3] if len(ins) > 3 and ins[3] is not None else None
    three = x.dim() == 3
    if three:
        heads = int(attrs.get("num_heads", 0))
        if heads <= 0:
            raise GraphExecutionError("RotaryEmbedding on a 3-D input needs the num_heads attribute")
        v = x.reshape(x.shape[0], x.shape[1], heads, -1)
    else:
        v = x.transpose(1, 2)
    d = v.shape[-1]
    rot = int(attrs.get("rotary_embedding_dim", 0)) or d
    if pos is not None:
        cos, sin = cos[pos.long()], sin[pos.long()]
    cos, sin = cos.unsqueeze(2).to(v.dtype), sin.unsqueeze(2).to(v.dtype)
    xr, rest = v[..., :rot], v[..., rot:]
    if attrs.get("interleaved", 0):
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
    else:
        x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
        out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
    out = torch.cat([out, rest], dim=-1)
    return out.reshape(x.shape) if three else out.transpose(1, 2)


def _contrib_rotary(ins, attrs):
    """com.microsoft::RotaryEmbedding: the same rotation with inputs ordered (input, position_ids, cos_cache, sin_cache);
    position ids are [batch, tokens], or one starting offset that the tokens count up from."""
    x, pos, cos, sin = ins[0], ins[1], ins[2], ins[3]
    tokens = x.shape[1] if x.dim() == 3 else x.shape[2]
    if pos.numel() == 1 and (pos.dim() < 2 or tokens > 1):
        pos = (pos.reshape(1, 1).long() + torch.arange(tokens, device=x.device)[None, :]).expand(x.shape[0], tokens)
    return _rotary([x, cos, sin, pos], attrs)


def _opt(ins, i):
    return ins[i] if len(ins) > i and ins[i] is not None else None


def _multi_head_attention(ins, attrs):
    """com.microsoft::MultiHeadAttention with separate 3-D query / key / value ([batch, tokens, heads * dim]).

    Optional inputs: a concatenated Q|K|V projection bias, a key padding mask ([batch, kv] of 0/1, or [batch] valid
    lengths), an additive attention bias broadcast over [batch, heads, q, kv], and past key / value
    ([batch, heads, past, dim]); outputs are the attention result and the present key / value.
    """
    q, k, v = ins[0], _opt(ins, 1), _opt(ins, 2)
    if k is None or v is None or q.dim() != 3 or k.dim() != 3:
        raise GraphExecutionError("MultiHeadAttention is covered for separate 3-D query, key and value inputs")
    h = int(attrs["num_heads"])
    bias, pad, extra, past_k, past_v = (_opt(ins, i) for i in (3, 4, 5, 6, 7))
    if bias is not None:
        bq, bk, bv = torch.split(bias, [q.shape[-1], k.shape[-1], v.shape[-1]])
        q, k, v = q + bq, k + bk, v + bv
    b, s = q.shape[0], q.shape[1]
    q = q.reshape(b, s, h, -1).transpose(1, 2).float()
    k = k.reshape(b, k.shape[1], h, -1).transpose(1, 2).float()
    v = v.reshape(b, v.shape[1], h, -1).transpose(1, 2).float()
    if past_k is not None:
        k, v = torch.cat([past_k.float(), k], dim=2), torch.cat([past_v.float(), v], dim=2)
    total = k.shape[2]
    scale = float(attrs.get("scale", 0.0)) or q.shape[-1] ** -0.5
    scores = q @ k.transpose(-1, -2) * scale
    if extra is not None:
        scores = scores + extra.float()
    if pad is not None:
        keep = (torch.arange(total, device=q.device)[None, :] < pad.reshape(b, 1)) if pad.dim() == 1 else pad.reshape(b, -1)[:, -total:].bool()
        scores = scores.masked_fill(~keep[:, None, None, :], float(attrs.get("mask_filter_value", -10000.0)))
    if int(attrs.get("unidirectional", 0)):
        scores = scores.masked_fill(~torch.ones(s, total, dtype=torch.bool, device=q.device).tril(total - s), float("-inf"))
    out = (torch.softmax(scores, dim=-1) @ v).transpose(1, 2).reshape(b, s, -1)
    return [out.to(ins[0].dtype), k.to(ins[0].dtype), v.to(ins[0].dtype)]


def _index_share(ins, attrs):
    """pkg.nxrt::IndexShare (version 1): attention over the cache positions an exporter selected.

    query [B, N, Sq, H]; key / value [B, Nkv, Skv, H] appended to the optional past pair; ``selected_indices``
    [B, N or 1, Sq, K] holds strictly increasing positions of the dense cache with ``-1`` as trailing padding; an
    optional additive bias broadcasts over [B, N, Sq, total].  Each query attends to its selected positions only; a row
    whose every selected position is masked to -inf gives zeros.  Returns the result and the dense present pair.
    (Contract: the reference's frozen v1 operator note for IndexShare under docs/architecture.)
    """
    q, k, v = ins[0], ins[1], ins[2]
    past_k, past_v, sel, extra = _opt(ins, 3), _opt(ins, 4), _opt(ins, 5), _opt(ins, 6)
    if sel is None or q.dim() != 4 or k.dim() != 4:
        raise GraphExecutionError("IndexShare needs 4-D query / key / value and selected_indices")
    if (past_k is None) != (past_v is None):
        raise GraphExecutionError("IndexShare: past_key and past_value come as a pair")
    n = int(attrs["num_heads"])
    nkv = int(attrs.get("kv_num_heads", n))
    if n % nkv or q.shape[1] != n or k.shape[1] != nkv:
        raise GraphExecutionError(f"IndexShare: {q.shape[1]} query heads / {k.shape[1]} KV heads do not match num_heads={n}, kv_num_heads={nkv}")
    if past_k is not None:
        k, v = torch.cat([past_k, k], dim=2), torch.cat([past_v, v], dim=2)
    total, b, sq = k.shape[2], q.shape[0], q.shape[2]
    sel = sel.long()
    if sel.dim() != 4 or sel.shape[0] != b or sel.shape[1] not in (1, n) or sel.shape[2] != sq:
        raise GraphExecutionError(f"IndexShare: selected_indices {list(sel.shape)} must be [{b}, {n} or 1, {sq}, K]")
    valid = sel >= 0
    if bool(((sel < -1) | (sel >= total)).any()):
        raise GraphExecutionError(f"IndexShare: a selected index lies outside [0, {total})")
    if bool((~valid[..., :1]).any()):
        raise GraphExecutionError("IndexShare: a row of selected_indices is empty")
    if sel.shape[-1] > 1:
        if bool((valid[..., 1:] & ~valid[..., :-1]).any()):
            raise GraphExecutionError("IndexShare: -1 may only pad the end of a row of selected_indices")
        if bool((valid[..., 1:] & (sel[..., 1:] <= sel[..., :-1])).any()):
            raise GraphExecutionError("IndexShare: selected indices must be strictly increasing")
    scale = float(attrs.get("scale", 0.0)) or q.shape[-1] ** -0.5
    if q.is_cuda:                                       # one warp per query row walks its selected positions (online softmax)
        from ..ops import sequence as _seq

        got = _seq.index_share_attention(q, k.to(q.dtype), v.to(q.dtype), sel, extra.to(q.dtype) if extra is not None else None, scale)
        if got is not None:
            return [got, k, v]
    chosen = torch.zeros(b, sel.shape[1], sq, total + 1, dtype=torch.bool, device=q.device)
    chosen.scatter_(3, torch.where(valid, sel, torch.full_like(sel, total)), True)
    chosen = chosen[..., :total]
    scale = float(attrs.get("scale", 0.0)) or q.shape[-1] ** -0.5
    group = n // nkv
    kf, vf = k.float().repeat_interleave(group, dim=1), v.float().repeat_interleave(group, dim=1)
    scores = (q.float() * scale ** 0.5) @ (kf * scale ** 0.5).transpose(-1, -2)
    if extra is not None:
        scores = scores + extra.float()
    scores = scores.masked_fill(~chosen, float("-inf"))
    dead = torch.isneginf(scores).all(dim=-1, keepdim=True)
    probs = torch.softmax(scores.masked_fill(dead, 0.0), dim=-1).masked_fill(dead, 0.0)
    return [(probs @ vf).to(q.dtype), k, v]


def _contrib_attention(ins, attrs):
    """com.microsoft::Attention: the input projection fused in -- ``input [batch, tokens, hidden] @ weights [hidden, 3 * hidden]
    + bias`` split into Q | K | V, then multi-head attention with the same optional mask, past (stacked [2, batch, heads,
    past, dim]) and additive bias as the unfused operator; returns the result and the stacked present."""
    x, w = ins[0], ins[1]
    bias, mask, past, extra = (_opt(ins, i) for i in (2, 3, 4, 5))
    sizes = attrs.get("qkv_hidden_sizes") or [w.shape[1] // 3] * 3
    qkv = x.float() @ w.float() + (bias.float() if bias is not None else 0.0)
    q, k, v = torch.split(qkv, [int(z) for z in sizes], dim=-1)
    pk, pv = (past[0], past[1]) if past is not None else (None, None)
    out, nk, nv = _multi_head_attention([q, k, v, None, mask, extra, pk, pv], attrs)
    return [out.to(x.dtype), torch.stack([nk, nv]).to(x.dtype)]


def _packed_multi_head_attention(ins, attrs):
    """com.microsoft::PackedMultiHeadAttention: padding-free attention over [tokens, heads * dim] rows, where
    ``cumulative_sequence_length`` ([batch + 1]) cuts the rows into sequences that attend only within themselves."""
    q, k, v = ins[0], _opt(ins, 1), _opt(ins, 2)
    if k is None or v is None or q.dim() != 2:
        raise GraphExecutionError("PackedMultiHeadAttention is covered for separate 2-D query, key and value inputs")
    h = int(attrs["num_heads"])
    bias, cu, extra = _opt(ins, 3), _opt(ins, 5), _opt(ins, 6)
    if cu is None:
        raise GraphExecutionError("PackedMultiHeadAttention needs cumulative_sequence_length")
    if bias is not None:
        bq, bk, bv = torch.split(bias, [q.shape[-1], k.shape[-1], v.shape[-1]])
        q, k, v = q + bq, k + bk, v + bv
    t = q.shape[0]
    qh, kh, vh = (x.reshape(t, h, -1).transpose(0, 1).float() for x in (q, k, v))
    scale = float(attrs.get("scale", 0.0)) or qh.shape[-1] ** -0.5
    bounds = [int(c) for c in cu.reshape(-1).tolist()]
    out = torch.zeros(h, t, vh.shape[-1], device=q.device)
    for i, (lo, hi) in enumerate(zip(bounds[:-1], bounds[1:])):
        scores = qh[:, lo:hi] @ kh[:, lo:hi].transpose(-1, -2) * scale
        if extra is not None:
            e = extra.float()
            scores = scores + e[i if e.shape[0] > 1 else 0][..., : hi - lo, : hi - lo]
        out[:, lo:hi] = torch.softmax(scores, dim=-1) @ vh[:, lo:hi]
    return out.transpose(0, 1).reshape(t, -1).to(ins[0].dtype)


def _attention(ins, attrs):
    """Attention (opset 23): scaled dot-product attention with optional mask, past K/V, grouped query heads, softcap."""
    q, k, v = ins[0], ins[1], ins[2]
    mask = ins[3] if len(ins) > 3 else None
    past_k = ins[4] if len(ins) > 4 else None
    past_v = ins[5] if len(ins) > 5 else None
    three = q.dim() == 3
    if three:
        hq, hkv = int(attrs["q_num_heads"]), int(attrs["kv_num_heads"])
        b, s = q.shape[0], q.shape[1]
        q = q.reshape(b, s, hq, -1).transpose(1, 2)
        k = k.reshape(b, k.shape[1], hkv, -1).transpose(1, 2)
        v = v.reshape(b, v.shape[1], hkv, -1).transpose(1, 2)
    if past_k is not None:
        k = torch.cat([past_k, k], dim=2)
    if past_v is not None:
        v = torch.cat([past_v, v], dim=2)
    present_k, present_v = k, v
    if q.shape[1] != k.shape[1]:
        rep = q.shape[1] // k.shape[1]
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scale = float(attrs.get("scale", 0.0)) or 1.0 / math.sqrt(q.shape[-1])
    scores = (q.float() @ k.float().transpose(-1, -2)) * scale
    cap = float(attrs.get("softcap", 0.0))
    if cap > 0:
        scores = cap * torch.tanh(scores / cap)
    nonpad = ins[6].long().reshape(-1) if len(ins) > 6 and ins[6] is not None else None
    if nonpad is not None:
        # fixed-size caches (opset 24): only the first nonpad[b] keys of row b hold tokens, and the queries are its last ones
        t_all, s_q = scores.shape[-1], scores.shape[-2]
        key_pos = torch.arange(t_all, device=scores.device)[None, None, :]
        allowed = key_pos < nonpad[:, None, None]
        if attrs.get("is_causal", 0):
            q_pos = (nonpad[:, None] - s_q + torch.arange(s_q, device=scores.device)[None])[:, :, None]
            allowed = allowed & (key_pos <= q_pos)
        scores = scores.masked_fill(~allowed[:, None], float("-inf"))
    elif attrs.get("is_causal", 0):
        # with past keys the triangle is aligned to the last key (query i sees keys up to past + i), which is what makes a
        # cached step equal the same position of a full pass; without past this is the plain lower triangle
        tri = torch.ones(scores.shape[-2], scores.shape[-1], dtype=torch.bool, device=scores.device).tril(scores.shape[-1] - scores.shape[-2])
        scores = scores.masked_fill(~tri, float("-inf"))
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else scores + mask.float()
    y = (torch.softmax(scores, dim=-1) @ v.float()).to(ins[0].dtype)
    if three:
        y = y.transpose(1, 2).reshape(y.shape[0], y.shape[2], -1)
    return [y, present_k, present_v, scores.to(ins[0].dtype)]


def _group_query_attention(ins, attrs):
    """com.microsoft::GroupQueryAttention with separate past / present buffers: packed [B, S, H*D] projections, optional
    in-op rotary embedding at positions ``seqlens_k + 1 - S + i``, causal attention over past + new keys (bottom-right
    aligned), optional local window."""
    q, k, v = ins[0], ins[1], ins[2]
    past_k = ins[3] if len(ins) > 3 else None
    past_v = ins[4] if len(ins) > 4 else None
    seqlens = ins[5].long().reshape(-1)
    cos = ins[7] if len(ins) > 7 else None
    sin = ins[8] if len(ins) > 8 else None
    if attrs.get("do_rotary", 0) and (cos is None or sin is None):
        raise GraphExecutionError("GroupQueryAttention with do_rotary needs the cos and sin caches")
    hq, hkv = int(attrs["num_heads"]), int(attrs["kv_num_heads"])
    b, s = q.shape[0], q.shape[1]
    if k is None:                                   # packed projections: [q | k | v] along the feature axis
        d = q.shape[2] // (hq + 2 * hkv)
        q, k, v = q[..., : hq * d], q[..., hq * d:(hq + hkv) * d], q[..., (hq + hkv) * d:]
    d = q.shape[2] // hq
    q = q.reshape(b, s, hq, d)
    k = k.reshape(b, s, hkv, d)
    v = v.reshape(b, s, hkv, d).transpose(1, 2)
    pos = (seqlens + 1 - s)[:, None] + torch.arange(s, device=q.device)[None]          # [B, S]
    if attrs.get("do_rotary", 0):
        ra = {"interleaved": int(attrs.get("rotary_interleaved", 0)), "rotary_embedding_dim": 2 * cos.shape[-1]}
        q = _rotary([q.transpose(1, 2), cos, sin, pos], ra).transpose(1, 2)
        k = _rotary([k.transpose(1, 2), cos, sin, pos], ra).transpose(1, 2)
    q, k = q.transpose(1, 2), k.transpose(1, 2)                                          # [B, H, S, D]
    if past_k is not None and past_k.shape[2] > 0:
        k, v = torch.cat([past_k.to(k.dtype), k], dim=2), torch.cat([past_v.to(v.dtype), v], dim=2)
    present_k, present_v = k, v
    t = k.shape[2]
    rep = hq // hkv
    kf, vf = k.repeat_interleave(rep, dim=1).float(), v.repeat_interleave(rep, dim=1).float()
    scale = float(attrs.get("scale", 0.0)) or 1.0 / math.sqrt(d)
    scores = (q.float() @ kf.transpose(-1, -2)) * scale
    cap = float(attrs.get("softcap", 0.0))
    if cap > 0:
        scores = cap * torch.tanh(scores / cap)
    key_pos = torch.arange(t, device=q.device)[None, None, :]
    q_pos = (t - s + torch.arange(s, device=q.device))[None, :, None]
    allowed = key_pos <= q_pos
    window = int(attrs.get("local_window_size", -1))
    if window > 0:
        allowed = allowed & (key_pos > q_pos - window)
    scores = scores.masked_fill(~allowed[:, None], float("-inf"))
    y = (torch.softmax(scores, dim=-1) @ vf).to(ins[0].dtype)
    return [y.transpose(1, 2).reshape(b, s, hq * d), present_k, present_v]


def _tensor_scatter(ins, attrs):
    """TensorScatter (opset 24): write ``update`` into ``past_cache`` along ``axis`` starting at each batch row's write index
    (0 when no indices are given); ``mode="circular"`` wraps around the cache length."""
    cache, update = ins[0], ins[1]
    idx = ins[2].long().reshape(-1) if len(ins) > 2 and ins[2] is not None else torch.zeros(cache.shape[0], dtype=torch.long, device=cache.device)
    axis = int(attrs.get("axis", -2)) % cache.dim()
    if axis == 0:
        raise GraphExecutionError("TensorScatter writes along a sequence axis; axis 0 is the batch")
    out = cache.clone()
    length, n = cache.shape[axis], update.shape[axis]
    circular = attrs.get("mode", "linear") == "circular"
    for b in range(cache.shape[0]):
        pos = int(idx[b]) + torch.arange(n, device=cache.device)
        if circular:
            pos = pos % length
        elif int(pos[-1]) >= length:
            raise GraphExecutionError(f"TensorScatter: row {b} writes positions up to {int(pos[-1])} into a cache of length {length}")
        out[b].index_copy_(axis - 1, pos, update[b].to(out.dtype))
    return out


def _dequant_rows(packed, scales, zero_points, bits, block):
    """[..., out, in / pack] packed integers (least significant bits first along the input axis) with [..., out, in / block]
    scales (and optional packed zero points) -> float weights [..., out, in]."""
    pack = 8 // bits
    mask = (1 << bits) - 1
    p = packed.to(torch.int32)
    if scales.dim() == packed.dim() - 1:            # one scale per output row
        scales = scales[..., None]
        zero_points = zero_points[..., None] if zero_points is not None else None
    parts = [(p >> (bits * i)) & mask for i in range(pack)]
    q = torch.stack(parts, dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * pack).float()
    blocks = scales.shape[-1]
    k = q.shape[-1]
    if zero_points is not None:
        z = zero_points.to(torch.int32)
        z = torch.stack([(z >> (bits * i)) & mask for i in range(pack)], dim=-1).reshape(*zero_points.shape[:-1], -1)[..., :blocks].float()
    else:
        z = torch.full(scales.shape, float(1 << (bits - 1)), device=packed.device)
    per = (k + blocks - 1) // blocks if block <= 0 else block
    qb = q.reshape(*q.shape[:-1], blocks, per)
    return ((qb - z[..., None]) * scales.float()[..., None]).reshape(*q.shape[:-1], k)


def _moe_route(logits, k, normalize):
    """Top-k experts by router logit (ties to the lower index); weights are softmax probabilities over all experts, or
    over the selected ones when ``normalize`` is set."""
    order = torch.argsort(-logits.float(), dim=-1, stable=True)[:, :k]
    e = torch.exp(logits.float() - logits.float().amax(dim=-1, keepdim=True))
    chosen = torch.gather(e, 1, order)
    denom = chosen.sum(dim=-1, keepdim=True) if normalize else e.sum(dim=-1, keepdim=True)
    return order, chosen / denom


def _moe_core(x, router, w1, b1, w2, b2, w3, b3, attrs, agg=None):
    """Mixture of experts on dense expert weights [E, out, in] (``com.microsoft::MoE`` / ``QMoE`` after dequantisation).
    ``agg`` ([rows, experts], optional) supplies the mixing weights of the experts the router logits select."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).float()
    order, weights = _moe_route(router.reshape(x2.shape[0], -1), int(attrs.get("k", 1)), bool(attrs.get("normalize_routing_weights", 0)))
    if agg is not None:
        weights = torch.gather(agg.reshape(x2.shape[0], -1).float(), 1, order)
        if attrs.get("normalize_routing_weights", 0):
            weights = weights / weights.sum(dim=-1, keepdim=True)
    act = attrs.get("activation_type", "relu")
    fusion = int(attrs.get("swiglu_fusion", 0))
    alpha, beta = float(attrs.get("activation_alpha", 1.0)), float(attrs.get("activation_beta", 0.0))
    limit = float(attrs.get("swiglu_limit", float("inf")))

    def glu(g, l):
        g, l = torch.clamp(g, max=limit), torch.clamp(l, -limit, limit)
        return g * torch.sigmoid(alpha * g) * (l + beta)

    out = torch.zeros(x2.shape[0], w2.shape[1])
    out = out.to(x2.device)
    for e in torch.unique(order).tolist():
        rows, slots = (order == e).nonzero(as_tuple=True)
        h = x2[rows] @ w1[e].float().T
        if b1 is not None:
            h = h + b1[e].float()
        if act == "swiglu" and fusion == 1:
            h = glu(h[:, 0::2], h[:, 1::2])
        elif act == "swiglu" and fusion == 2:
            half = h.shape[1] // 2
            h = glu(h[:, :half], h[:, half:])
        elif act == "swiglu":
            l = x2[rows] @ w3[e].float().T + (b3[e].float() if b3 is not None else 0)
            h = glu(h, l)
        elif act == "silu":
            h = F.silu(h) * (x2[rows] @ w3[e].float().T + (b3[e].float() if b3 is not None else 0)) if w3 is not None else F.silu(h)
        elif act == "gelu":
            h = F.gelu(h, approximate="tanh")
        elif act == "relu":
            h = F.relu(h)
        elif act != "identity":
            raise GraphExecutionError(f"MoE activation_type {act!r} is not covered (relu, gelu, silu, swiglu, identity)")
        y = h @ w2[e].float().T
        if b2 is not None:
            y = y + b2[e].float()
        out.index_add_(0, rows, y * weights[rows, slots][:, None])
    return out.to(x.dtype).reshape(*shape[:-1], -1)


def _moe(ins, attrs):
    get = lambda i: ins[i] if len(ins) > i and ins[i] is not None else None
    return _moe_core(ins[0], ins[1], ins[2], get(3), ins[4], get(5), get(6), get(7), attrs)


def _qmoe(ins, attrs):
    """com.microsoft::QMoE with integer expert weights: inputs (x, router, fc1 w, fc1 scales, fc1 bias, fc2 w, fc2 scales,
    fc2 bias, fc3 w, fc3 scales, fc3 bias, fc1 zero points, fc2 zero points, fc3 zero points)."""
    get = lambda i: ins[i] if len(ins) > i and ins[i] is not None else None
    bits, block = int(attrs.get("expert_weight_bits", 4)), int(attrs.get("block_size", 0))
    if bits not in (2, 4, 8) or attrs.get("quant_type", "int") != "int":
        raise GraphExecutionError("QMoE is covered for integer weights of 2, 4 or 8 bits")
    w1 = _dequant_rows(ins[2], ins[3], get(11), bits, block)
    w2 = _dequant_rows(ins[5], ins[6], get(12), bits, block)
    w3 = _dequant_rows(ins[8], ins[9], get(13), bits, block) if get(8) is not None else None
    return _moe_core(ins[0], ins[1], w1, get(4), w2, get(7), w3, get(10), attrs, agg=get(14))


def _bitshift(ins, attrs):
    x, n = ins[0], ins[1]
    if attrs.get("direction", "LEFT") == "LEFT":
        return torch.bitwise_left_shift(x, n)
    if x.dtype == torch.uint8:
        return torch.bitwise_right_shift(x, n)
    # the operator is defined on unsigned integers, which live in int64 here: shift logically, not arithmetically
    n64 = n.to(torch.int64)
    keep = torch.where(n64 > 0, (torch.ones_like(n64) << (64 - n64).clamp(max=63)) - 1, torch.full_like(n64, -1))
    return torch.bitwise_right_shift(x.to(torch.int64), n64) & keep


def _mod(ins, attrs):
    a, b = ins[0], ins[1]
    if attrs.get("fmod", 0) or a.is_floating_point():
        return torch.fmod(a, b)
    return torch.remainder(a, b)                 # integer Mod takes the sign of the divisor


def _erf_gelu(x):
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def _cast(x, to):
    to = int(to)
    if to in (onnx_pb.UINT32, onnx_pb.UINT64, onnx_pb.UINT16):
        # torch has no arithmetic on wide unsigned types: they live in int64 (two's complement wraps like uint64; narrower
        # ones are masked at the cast, so a value that overflows between casts keeps its high bits until the next cast)
        y = x.to(torch.int64)
        return y & 0xFFFFFFFF if to == onnx_pb.UINT32 else (y & 0xFFFF if to == onnx_pb.UINT16 else y)
    dt = _TORCH_DTYPE.get(to)
    if dt is None:
        raise GraphExecutionError(f"Cast to ONNX data type {to} is not covered")
    return x.to(dt)


# op name -> callable(inputs, attrs) -> tensor | list of tensors
OPS = {
    "Add": lambda i, a: i[0] + i[1], "Sub": lambda i, a: i[0] - i[1], "Mul": lambda i, a: i[0] * i[1],
    "Div": lambda i, a: torch.div(i[0], i[1], rounding_mode="trunc") if not i[0].is_floating_point() else i[0] / i[1],
    "Pow": lambda i, a: torch.pow(i[0], i[1].to(i[0].dtype) if i[0].is_floating_point() else i[1]),
    "Neg": lambda i, a: -i[0], "Abs": lambda i, a: i[0].abs(), "Sqrt": lambda i, a: i[0].sqrt(), "Exp": lambda i, a: i[0].exp(),
    "Log": lambda i, a: i[0].log(), "Reciprocal": lambda i, a: 1.0 / i[0], "Floor": lambda i, a: i[0].floor(), "Ceil": lambda i, a: i[0].ceil(),
    "Round": lambda i, a: i[0].round(), "Sin": lambda i, a: i[0].sin(), "Cos": lambda i, a: i[0].cos(), "Tanh": lambda i, a: i[0].tanh(),
    "Erf": lambda i, a: torch.erf(i[0]), "Sign": lambda i, a: i[0].sign(), "Sigmoid": lambda i, a: torch.sigmoid(i[0]),
    "Relu": lambda i, a: F.relu(i[0]), "LeakyRelu": lambda i, a: F.leaky_relu(i[0], float(a.get("alpha", 0.01))),
    "Elu": lambda i, a: F.elu(i[0], float(a.get("alpha", 1.0))), "Softplus": lambda i, a: F.softplus(i[0]),
    "HardSigmoid": lambda i, a: torch.clamp(float(a.get("alpha", 0.2)) * i[0] + float(a.get("beta", 0.5)), 0, 1),
    "HardSwish": lambda i, a: F.hardswish(i[0]), "Mish": lambda i, a: F.mish(i[0]),
    "Gelu": lambda i, a: F.gelu(i[0], approximate="tanh") if a.get("approximate", "none") == "tanh" else _erf_gelu(i[0]),
    "FastGelu": lambda i, a: F.gelu(i[0] + (i[1] if len(i) > 1 and i[1] is not None else 0), approximate="tanh"),
    "BiasGelu": lambda i, a: _erf_gelu(i[0] + i[1]),
    "QuickGelu": lambda i, a: i[0] * torch.sigmoid(float(a.get("alpha", 1.702)) * i[0]),
    "Min": lambda i, a: torch.stack(torch.broadcast_tensors(*i)).amin(0) if len(i) > 1 else i[0],
    "Max": lambda i, a: torch.stack(torch.broadcast_tensors(*i)).amax(0) if len(i) > 1 else i[0],
    "Sum": lambda i, a: sum(i[1:], i[0]), "Mean": lambda i, a: sum(i[1:], i[0]) / len(i),
    "Clip": lambda i, a: (lambda lo, hi: i[0] if lo is None and hi is None else torch.clamp(i[0], min=lo, max=hi))(
        i[1].item() if len(i) > 1 and i[1] is not None else a.get("min"), i[2].item() if len(i) > 2 and i[2] is not None else a.get("max")),
    "Equal": lambda i, a: i[0] == i[1], "Less": lambda i, a: i[0] < i[1], "LessOrEqual": lambda i, a: i[0] <= i[1],
    "Greater": lambda i, a: i[0] > i[1], "GreaterOrEqual": lambda i, a: i[0] >= i[1],
    "Not": lambda i, a: ~i[0], "And": lambda i, a: i[0] & i[1], "Or": lambda i, a: i[0] | i[1], "Xor": lambda i, a: i[0] ^ i[1],
    "Where": lambda i, a: torch.where(i[0], i[1], i[2]), "IsNaN": lambda i, a: torch.isnan(i[0]),
    "BitShift": _bitshift, "BitwiseAnd": lambda i, a: i[0] & i[1], "BitwiseOr": lambda i, a: i[0] | i[1],
    "BitwiseXor": lambda i, a: i[0] ^ i[1], "BitwiseNot": lambda i, a: ~i[0], "Mod": _mod,
    "IsInf": lambda i, a: torch.isinf(i[0]) & ((i[0] > 0) if not a.get("detect_negative", 1) else True) & ((i[0] < 0) if not a.get("detect_positive", 1) else True),
    "Swish": lambda i, a: i[0] * torch.sigmoid(float(a.get("alpha", 1.0)) * i[0]),
    "MoE": _moe, "QMoE": _qmoe, "TensorScatter": _tensor_scatter, "RotaryEmbedding": _rotary, "Attention": _attention, "GroupQueryAttention": _group_query_attention,
    "MatMul": lambda i, a: i[0] @ i[1],
    "Gemm": lambda i, a: float(a.get("alpha", 1.0)) * ((i[0].T if a.get("transA", 0) else i[0]) @ (i[1].T if a.get("transB", 0) else i[1]))
                         + (float(a.get("beta", 1.0)) * i[2] if len(i) > 2 and i[2] is not None else 0),
    "IndexShare": _index_share, "com.microsoft::Attention": _contrib_attention, "com.microsoft::RotaryEmbedding": _contrib_rotary, "MultiHeadAttention": _multi_head_attention, "PackedMultiHeadAttention": _packed_multi_head_attention,
    "NonZero": lambda i, a: torch.nonzero(i[0]).T.contiguous(), "PRelu": lambda i, a: torch.where(i[0] >= 0, i[0], i[0] * i[1]),
    "MatMulNBits": _matmul_nbits, "BlockQuantizedMatMul": _block_quantized_matmul,
    "Conv": lambda i, a: _conv(i, a), "ConvTranspose": lambda i, a: _conv(i, a, transpose=True),
    "MaxPool": lambda i, a: _pool(i, a, "max"), "AveragePool": lambda i, a: _pool(i, a, "avg"),
    "GlobalAveragePool": lambda i, a: i[0].mean(tuple(range(2, i[0].dim())), keepdim=True),
    "GlobalMaxPool": lambda i, a: i[0].amax(tuple(range(2, i[0].dim())), keepdim=True),
    "Resize": _resize, "Upsample": lambda i, a: _resize([i[0], None, i[1]], a),
    "BatchNormalization": lambda i, a: F.batch_norm(i[0], i[3], i[4], i[1], i[2], False, 0.0, float(a.get("epsilon", 1e-5))),
    "InstanceNormalization": lambda i, a: F.instance_norm(i[0], weight=i[1], bias=i[2], eps=float(a.get("epsilon", 1e-5))),
    "GroupNormalization": lambda i, a: F.group_norm(i[0], int(a["num_groups"]), i[1], i[2], float(a.get("epsilon", 1e-5))),
    "LayerNormalization": lambda i, a: _layer_norm(i[0], i[1], i[2] if len(i) > 2 else None, int(a.get("axis", -1)), float(a.get("epsilon", 1e-5))),
    "SimplifiedLayerNormalization": lambda i, a: _rms_norm_with_stat(i[0], i[1], int(a.get("axis", -1)), float(a.get("epsilon", 1e-5))),
    "RMSNormalization": lambda i, a: _rms_norm(i[0], i[1], int(a.get("axis", -1)), float(a.get("epsilon", 1e-5))),
    "Softmax": lambda i, a: torch.softmax(i[0].float(), int(a.get("axis", -1))).to(i[0].dtype),
    "LogSoftmax": lambda i, a: torch.log_softmax(i[0].float(), int(a.get("axis", -1))).to(i[0].dtype),
    "ReduceMean": _reduce(lambda x, ax, k: x.mean(ax, keepdim=k)), "ReduceSum": _reduce(lambda x, ax, k: x.sum(ax, keepdim=k)),
    "ReduceMax": _reduce(lambda x, ax, k: x.amax(ax, keepdim=k)), "ReduceMin": _reduce(lambda x, ax, k: x.amin(ax, keepdim=k)),
    "ReduceProd": _reduce(lambda x, ax, k: torch.prod(x, ax[0], keepdim=k) if len(ax) == 1 else x.flatten().prod()),
    "ReduceL2": _reduce(lambda x, ax, k: x.pow(2).sum(ax, keepdim=k).sqrt()),
    "ReduceSumSquare": _reduce(lambda x, ax, k: x.pow(2).sum(ax, keepdim=k)),
    "ArgMax": lambda i, a: i[0].argmax(int(a.get("axis", 0)), keepdim=bool(a.get("keepdims", 1))),
    "ArgMin": lambda i, a: i[0].argmin(int(a.get("axis", 0)), keepdim=bool(a.get("keepdims", 1))),
    "TopK": lambda i, a: _topk(i[0], int(i[1].reshape(-1)[0]), int(a.get("axis", -1)), bool(a.get("largest", 1))),
    "CumSum": lambda i, a: torch.cumsum(i[0], int(i[1].reshape(-1)[0])),
    "Reshape": lambda i, a: _reshape(i[0], i[1], a.get("allowzero", 0)),
    "Flatten": lambda i, a: i[0].reshape(int(np.prod(i[0].shape[: int(a.get("axis", 1))])) if int(a.get("axis", 1)) else 1, -1),
    "Transpose": lambda i, a: i[0].permute(_ints(a["perm"])) if a.get("perm") else i[0].permute(*reversed(range(i[0].dim()))),
    "Squeeze": _squeeze, "Unsqueeze": _unsqueeze,
    "Concat": lambda i, a: torch.cat([t for t in i if t is not None], dim=int(a.get("axis", 0))),
    "Slice": _slice, "Pad": _pad, "Tile": lambda i, a: i[0].repeat(_ints(i[1])), "Expand": lambda i, a: _expand(i[0], i[1]),
    "Gather": lambda i, a: (lambda x, idx, ax: x.index_select(ax, torch.where(idx < 0, idx + x.shape[ax], idx).reshape(-1).long())
                            .reshape(tuple(x.shape[:ax]) + tuple(idx.shape) + tuple(x.shape[ax + 1:])))(i[0], i[1], int(a.get("axis", 0)) % i[0].dim()),
    "GatherElements": lambda i, a: torch.gather(i[0], int(a.get("axis", 0)), i[1].long()),
    "GatherND": lambda i, a: _gather_nd(i[0], i[1]),
    "ScatterElements": lambda i, a: i[0].scatter(int(a.get("axis", 0)), i[1].long(), i[2]),
    "ScatterND": lambda i, a: (lambda out, idx, upd: out.index_put_(tuple(idx.reshape(-1, idx.shape[-1]).long().T),
                                                                    upd.reshape((-1,) + tuple(out.shape[idx.shape[-1]:]))))(i[0].clone(), i[1], i[2]),
    "Shape": lambda i, a: torch.tensor(list(i[0].shape)[int(a.get("start", 0)): a.get("end")], dtype=torch.int64, device=i[0].device),
    "Size": lambda i, a: torch.tensor(i[0].numel(), dtype=torch.int64, device=i[0].device),
    "ConstantOfShape": lambda i, a: torch.zeros(_ints(i[0]), device=i[0].device) if "value" not in a else
        tensor_to_torch(a["value"], i[0].device).reshape(-1)[0].expand(_ints(i[0])).clone(),
    "Range": lambda i, a: torch.arange(i[0].item(), i[1].item(), i[2].item(), dtype=i[0].dtype, device=i[0].device),
    "Cast": lambda i, a: _cast(i[0], a["to"]), "CastLike": lambda i, a: i[0].to(i[1].dtype),
    "Identity": lambda i, a: i[0], "Dropout": lambda i, a: i[0],
    "Einsum": lambda i, a: torch.einsum(a["equation"], *i),
    "Trilu": lambda i, a: (torch.triu if a.get("upper", 1) else torch.tril)(i[0], int(i[1].item()) if len(i) > 1 and i[1] is not None else 0),
    "OneHot": lambda i, a: (lambda oh, vals: oh * (vals[1] - vals[0]) + vals[0])(F.one_hot(i[0].long() % int(i[1].item()), int(i[1].item())).to(i[2].dtype), i[2]),
    "DepthToSpace": lambda i, a: F.pixel_shuffle(i[0], int(a["blocksize"])) if a.get("mode", "DCR") == "CRD" else
        (lambda x, b: x.reshape(x.shape[0], b, b, x.shape[1] // (b * b), x.shape[2], x.shape[3]).permute(0, 3, 4, 1, 5, 2)
         .reshape(x.shape[0], x.shape[1] // (b * b), x.shape[2] * b, x.shape[3] * b))(i[0], int(a["blocksize"])),
    "SpaceToDepth": lambda i, a: F.pixel_unshuffle(i[0], int(a["blocksize"])),
    "SkipLayerNormalization": lambda i, a: (lambda s: [_layer_norm(s, i[2], i[3] if len(i) > 3 and i[3] is not None else None, -1,
                                                                   float(a.get("epsilon", 1e-5)))[0], None, None, s])(i[0] + i[1] + (i[4] if len(i) > 4 and i[4] is not None else 0)),
    "SkipSimplifiedLayerNormalization": lambda i, a: (lambda s: [_rms_norm(s, i[2], -1, float(a.get("epsilon", 1e-5))), None, None, s])(
        i[0] + i[1] + (i[3] if len(i) > 3 and i[3] is not None else 0)),
}


CONTROL_FLOW = ("If", "Loop", "Scan")
_STRUCTURAL = ("Constant", "Split") + CONTROL_FLOW


def _subgraphs(node):
    return [v for v in node.attrs.values() if isinstance(v, onnx_pb.Graph)]


def _all_nodes(graph):
    for n in graph.nodes:
        yield n
        for sub in _subgraphs(n):
            yield from _all_nodes(sub)


def _free_values(graph) -> set:
    """Names a (sub)graph reads from an enclosing scope: used, but neither its inputs, its initializers nor produced in it."""
    defined = {vi.name for vi in graph.inputs} | set(graph.initializers)
    free = set()
    for n in graph.nodes:
        for x in n.inputs:
            if x and x not in defined:
                free.add(x)
        for sub in _subgraphs(n):
            free |= {x for x in _free_values(sub) if x not in defined}
        defined.update(o for o in n.outputs if o)
    return free


class GraphExecutor:
    def __init__(self, model, device="cpu", dtype=None, optimize=False, release=False):
        """``model``: a path to an ``.onnx`` file or a parsed :class:`onnx_pb.Model`.  Initializers move to ``device``
        (floating-point ones are cast to ``dtype`` when given).  ``optimize``: run the rewrite passes of
        :mod:`graph_optimizer` on the graph first (constant folding, no-op removal, GELU / LayerNorm / Gemm fusion, dead
        nodes); the model object is rewritten in place and ``self.optimization`` holds the report.  ``release``: drop every
        intermediate from the interpreter's scope right after its last reader (lifetimes of :mod:`memory_plan`), so a
        run holds its live set rather than every value it ever produced; ``self.peak_live_bytes`` then reports the
        largest live set of the last run."""
        self.model = onnx_pb.load_model(model) if isinstance(model, str) else model
        self.device = torch.device(device)
        self.optimization = None
        if optimize:
            from .graph_optimizer import optimize as _optimize

            self.optimization = _optimize(self.model)
        g = self.model.graph
        self.constants = {}
        for name, t in g.initializers.items():
            v = tensor_to_torch(t, self.device)
            if dtype is not None and v.is_floating_point():
                v = v.to(dtype)
            self.constants[name] = v
        self.input_names = [vi.name for vi in g.inputs if vi.name not in self.constants]
        self.output_names = [vi.name for vi in g.outputs]
        self.input_types = {vi.name: vi.elem_type for vi in g.inputs}
        unknown = sorted({(n.domain + "::" if n.domain else "") + n.op_type for n in _all_nodes(g) if n.op_type not in OPS
                          and f"{n.domain}::{n.op_type}" not in OPS and n.op_type not in _STRUCTURAL})
        if unknown:
            raise GraphExecutionError(f"graph '{g.name}' uses operators outside the covered set: {', '.join(unknown)} "
                                      f"({len(OPS) + len(_STRUCTURAL)} operators are covered, If, Loop and Scan among them)")
        self._sub_constants: dict = {}        # id(subgraph) -> its initializers on the device
        self.order = self._toposort(g)
        self.runs = 0
        self.release = bool(release)
        self.peak_live_bytes = 0
        self._drop_after: list = []
        if self.release:
            from .memory_plan import lifetimes

            _, born, last = lifetimes(self.model, self.order)
            keep = set(self.output_names)
            self._drop_after = [[] for _ in self.order]
            for name, i in last.items():
                if name in born and name not in keep and i < len(self.order):
                    self._drop_after[i].append(name)

    def _toposort(self, g):
        produced = set(self.constants) | set(self.input_names)
        pending, order = list(g.nodes), []
        while pending:
            rest = []
            for n in pending:
                needs = [x for x in n.inputs if x] + [x for sub in _subgraphs(n) for x in _free_values(sub)]   # bodies capture outer values
                if all(x in produced for x in needs):
                    order.append(n)
                    produced.update(o for o in n.outputs if o)
                else:
                    rest.append(n)
            if len(rest) == len(pending):
                missing = sorted({x for n in rest for x in n.inputs if x and x not in produced})
                raise GraphExecutionError(f"graph '{g.name}' cannot be ordered: values {missing[:6]} are never produced")
            pending = rest
        return order

    @torch.no_grad()
    def run(self, feeds: dict, outputs=None) -> dict:
        """``feeds``: input name -> tensor / array / scalar.  Returns output name -> tensor for ``outputs`` (default: all)."""
        missing = [n for n in self.input_names if n not in feeds]
        if missing:
            raise GraphExecutionError(f"missing graph input(s) {missing}; the graph takes {self.input_names}")
        env = dict(self.constants)
        for name, v in feeds.items():
            t = v if isinstance(v, torch.Tensor) else torch.as_tensor(_signed_home(np.asarray(v)))
            want = _TORCH_DTYPE.get(self.input_types.get(name))
            if want is not None and t.dtype != want and (t.is_floating_point() == want.is_floating_point):
                t = t.to(want)
            env[name] = t.to(self.device)
        if self.release and not outputs:
            # live bytes are counted per storage: an operator may hand back a view of its input (a transpose, a slice), and
            # the bytes stay live until the last name over that storage is dropped.  Inputs and initializers are the caller's.
            def key(t):
                return t.untyped_storage().data_ptr() if isinstance(t, torch.Tensor) and t.numel() else None

            external = {key(t) for t in env.values()}
            holders: dict = {}                       # storage -> [bytes, names bound over it]
            live = peak = 0
            for i, n in enumerate(self.order):
                self._exec_node(n, env)
                for o in n.outputs:
                    k = key(env.get(o)) if o else None
                    if k is None or k in external:
                        continue
                    slot = holders.get(k)
                    if slot is None:
                        slot = holders[k] = [env[o].untyped_storage().nbytes(), set()]
                        live += slot[0]
                    slot[1].add(o)
                peak = max(peak, live)
                for name in self._drop_after[i]:
                    t = env.pop(name, None)
                    slot = holders.get(key(t))
                    if slot is not None:
                        slot[1].discard(name)
                        if not slot[1]:
                            live -= slot[0]
                            del holders[key(t)]
            self.peak_live_bytes = peak
        else:
            for n in self.order:
                self._exec_node(n, env)
        self.runs += 1
        return {name: env[name] for name in (outputs or self.output_names)}


def _exec_node(self, n, env) -> None:
    """Run one node against ``env`` (a dict, or a chained scope for control-flow bodies) and bind its outputs there."""
    ins = [env[x] if x else None for x in n.inputs]
    try:
        if n.op_type == "Constant":
            res = _constant(ins, n.attrs, self.device)
        elif n.op_type == "Split":
            res = _split(ins, n.attrs, len(n.outputs))
        elif n.op_type == "If":
            branch = n.attrs["then_branch"] if bool(ins[0].reshape(-1)[0]) else n.attrs["else_branch"]
            res = self._run_body(branch, env, {})
        elif n.op_type == "Loop":
            res = self._loop(n, ins, env)
        elif n.op_type == "Scan":
            from .graph_ops_sequence import _scan

            res = _scan(self, n, ins, env)
        else:
            res = (OPS.get(f"{n.domain}::{n.op_type}") or OPS[n.op_type])(ins, n.attrs)       # a domain-qualified entry wins
    except GraphExecutionError:
        raise
    except Exception as e:
        shapes = [tuple(t.shape) if isinstance(t, torch.Tensor) else None for t in ins]
        raise GraphExecutionError(f"node '{n.name or n.outputs[0]}' ({n.op_type}) failed on inputs {shapes}: {e}") from e
    if isinstance(res, (list, tuple)):
        for name, r in zip(n.outputs, res):
            if name and r is not None:
                env[name] = r
    else:
        env[n.outputs[0]] = res


def _run_body(self, graph, outer, feeds: dict) -> list:
    """A control-flow body: its own scope over the enclosing one (bodies read outer values by name); returns its outputs."""
    import collections

    consts = self._sub_constants.get(id(graph))
    if consts is None:
        consts = self._sub_constants[id(graph)] = {k: tensor_to_torch(t, self.device) for k, t in graph.initializers.items()}
    scope = collections.ChainMap(dict(feeds), consts, outer)
    for node in graph.nodes:                       # bodies are stored in execution order
        self._exec_node(node, scope)
    return [scope[vi.name] for vi in graph.outputs]


def _loop(self, n, ins, env) -> list:
    """Loop: inputs (trip count | "", condition | "", carried...); body (iteration, condition, carried...) ->
    (condition, carried..., scan outputs...).  Outputs: the final carried values, then each scan output stacked."""
    body = n.attrs["body"]
    limit = int(ins[0].reshape(-1)[0]) if ins[0] is not None else None
    cond = bool(ins[1].reshape(-1)[0]) if len(ins) > 1 and ins[1] is not None else True
    carried = list(ins[2:])
    names = [vi.name for vi in body.inputs]
    n_scan = len(body.outputs) - 1 - len(carried)
    if len(names) != 2 + len(carried) or n_scan < 0:
        raise GraphExecutionError(f"Loop body takes {len(names)} inputs and gives {len(body.outputs)} outputs for {len(carried)} carried values")
    scans = [[] for _ in range(n_scan)]
    it = 0
    while cond and (limit is None or it < limit):
        if it >= 1_000_000:
            raise GraphExecutionError("Loop ran a million iterations without its condition turning false")
        feeds = {names[0]: torch.tensor(it, dtype=torch.int64, device=self.device), names[1]: torch.tensor(cond, device=self.device)}
        feeds.update(zip(names[2:], carried))
        out = self._run_body(body, env, feeds)
        cond = bool(out[0].reshape(-1)[0])
        carried = list(out[1:1 + len(carried)])
        for acc, v in zip(scans, out[1 + len(carried):]):
            acc.append(v)
        it += 1
    stacked = []
    for acc, vi in zip(scans, body.outputs[1 + len(carried):]):
        stacked.append(torch.stack(acc) if acc else torch.zeros((0,), dtype=_TORCH_DTYPE.get(vi.elem_type, torch.float32), device=self.device))
    return carried + stacked


GraphExecutor._exec_node = _exec_node
GraphExecutor._run_body = _run_body
GraphExecutor._loop = _loop


def as_component(model, device="cpu", dtype=None):
    """A workflow component (dict of input ports -> dict of output ports) backed by an ONNX graph."""
    ex = GraphExecutor(model, device, dtype)

    def component(ports: dict) -> dict:
        return ex.run({k: v for k, v in ports.items() if k in ex.input_names})

    component.executor = ex
    return component


from . import graph_ops_extra, graph_ops_sequence  # noqa: E402,F401  (they add operators to OPS; they need the names above)
