"""Graph operators of hybrid and padding-free decoders: recurrent linear attention, the causal short convolution with a
rolling state, attention over token-major packed sequences, block-quantised gathers, the fused attention core, ``Scan``.

Each follows the contract of the reference's CPU kernel of the same name (crates/onnx-runtime-ep-cpu/src/kernels/
linear_attention.rs:1-58, causal_conv.rs:1-40, varlen_attention.rs, packed_varlen_attention.rs,
gather_block_quantized.rs:1-30, fused_attention.rs:1-23) and computes in float32.  Importing this module adds them to
``graph_executor.OPS``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .graph_executor import OPS, GraphExecutionError, _moe_core, _opt, decode_weight_blocks


def _linear_attention(ins, attrs):
    """com.microsoft::LinearAttention: a [d_k, d_v] state per KV head, updated token by token.

    query [B, T, Hq * d_k], key [B, T, Nk * d_k], value [B, T, Hkv * d_v], optional past state [B, Hkv, d_k, d_v], log
    decay [B, T, Hkv] or [B, T, Hkv * d_k], beta [B, T, Hkv] or [B, T, 1].  ``update_rule``: ``linear`` adds k v^T;
    ``gated`` first scales the state by exp(decay); ``delta`` adds k (beta (v - S^T k))^T; ``gated_delta`` does both.
    The readout is ``scale * q^T S`` on the updated state.  More query heads than KV heads share states in contiguous
    groups; fewer query heads than KV heads gives one output head per KV head; key heads may be shared likewise.
    """
    q, k, v = ins[0].float(), ins[1].float(), ins[2].float()
    past, decay, beta = _opt(ins, 3), _opt(ins, 4), _opt(ins, 5)
    hq, hkv = int(attrs["q_num_heads"]), int(attrs["kv_num_heads"])
    rule = attrs.get("update_rule", "gated_delta") or "gated_delta"
    if rule not in ("linear", "gated", "delta", "gated_delta"):
        raise GraphExecutionError(f"LinearAttention: update_rule {rule!r} is not one of linear, gated, delta, gated_delta")
    use_decay, use_delta = rule in ("gated", "gated_delta"), rule in ("delta", "gated_delta")
    b, t = q.shape[0], q.shape[1]
    if q.shape[2] % hq or v.shape[2] % hkv:
        raise GraphExecutionError(f"LinearAttention: widths {q.shape[2]} / {v.shape[2]} do not divide into {hq} / {hkv} heads")
    dk, dv = q.shape[2] // hq, v.shape[2] // hkv
    if k.shape[2] % dk:
        raise GraphExecutionError(f"LinearAttention: key width {k.shape[2]} is not a multiple of d_k = {dk}")
    nk = k.shape[2] // dk
    if hkv % nk or (hq >= hkv and hq % hkv) or (hq < hkv and hkv % hq):
        raise GraphExecutionError(f"LinearAttention: head counts q={hq}, k={nk}, kv={hkv} do not group evenly")
    if (use_decay and decay is None) or (use_delta and beta is None):
        raise GraphExecutionError(f"LinearAttention: update_rule {rule!r} needs its gate input")
    scale = float(attrs.get("scale", 0.0)) or dk ** -0.5
    if ins[0].is_cuda:                                  # the recurrent kernel: one state column per thread, fp32 state in registers
        from ..ops import sequence as _seq

        same = lambda x: x.to(ins[0].dtype) if x is not None else None
        got = _seq.linear_attention(ins[0], same(ins[1]), same(ins[2]), same(past), same(decay), same(beta), hq, hkv, rule, scale)
        if got is not None:
            return [got[0], got[1]]
    qh = q.reshape(b, t, hq, dk)
    kh = k.reshape(b, t, nk, dk).repeat_interleave(hkv // nk, dim=2)                      # [B, T, Hkv, dk]
    vh = v.reshape(b, t, hkv, dv)
    if hq >= hkv:
        group = hq // hkv
        q_of_out, state_of_out = torch.arange(hq), torch.arange(hq) // group
    else:
        q_of_out, state_of_out = torch.arange(hkv) * hq // hkv, torch.arange(hkv)
    state = past.float().clone() if past is not None else torch.zeros(b, hkv, dk, dv, device=q.device)
    if use_decay:
        g = decay.float().reshape(b, t, hkv, -1)                                          # [.., 1] per head or [.., dk] per key dim
    if use_delta:
        bt = beta.float().reshape(b, t, -1).expand(b, t, hkv)
    outs = []
    for step in range(t):
        kt, vt = kh[:, step], vh[:, step]                                                 # [B, Hkv, dk], [B, Hkv, dv]
        if use_decay:
            state = state * torch.exp(g[:, step])[..., None]
        if use_delta:
            retrieved = torch.einsum("bhij,bhi->bhj", state, kt)
            vt = bt[:, step][..., None] * (vt - retrieved)
        state = state + kt[..., :, None] * vt[..., None, :]
        outs.append(scale * torch.einsum("bhi,bhij->bhj", qh[:, step][:, q_of_out], state[:, state_of_out]))
    out = torch.stack(outs, dim=1).reshape(b, t, -1) if outs else torch.zeros(b, 0, max(hq, hkv) * dv, device=q.device)
    return [out.to(ins[0].dtype), state.to(ins[0].dtype)]


def _causal_conv_with_state(ins, attrs):
    """com.microsoft::CausalConvWithState: depthwise 1-D convolution over ``concat(past_state, x)`` -- x [B, C, L], weight
    [C, 1, K], optional bias [C] and past state [B, C, K-1] (zeros when absent) -> y [B, C, L] and the last K-1 frames."""
    x, w = ins[0], ins[1]
    bias, past = _opt(ins, 2), _opt(ins, 3)
    if int(attrs.get("ndim", 1)) != 1 or x.dim() != 3 or w.dim() != 3 or w.shape[1] != 1:
        raise GraphExecutionError("CausalConvWithState is covered for ndim=1: x [B, C, L] with a depthwise weight [C, 1, K]")
    k = w.shape[2]
    act = attrs.get("activation", "none") or "none"
    if x.is_cuda and act in ("none", "silu", "swish"):
        from ..ops import sequence as _seq

        same = lambda t: t.to(x.dtype) if t is not None else None
        got = _seq.causal_conv_state(x, same(w), same(bias), same(past), act != "none")
        if got is not None:
            return [got[0], got[1]]
    if past is None:
        past = torch.zeros(x.shape[0], x.shape[1], k - 1, dtype=x.dtype, device=x.device)
    seq = torch.cat([past.float(), x.float()], dim=2)
    y = F.conv1d(seq, w.float(), bias.float() if bias is not None else None, groups=x.shape[1])
    act = attrs.get("activation", "none") or "none"
    if act in ("silu", "swish"):
        y = F.silu(y)
    elif act != "none":
        raise GraphExecutionError(f"CausalConvWithState: activation {act!r} is not one of none, silu, swish")
    return [y.to(x.dtype), seq[:, :, seq.shape[2] - (k - 1):].to(x.dtype)]


def _offsets(t, name, total):
    vals = [int(v) for v in t.reshape(-1).tolist()]
    if len(vals) < 2 or vals[0] != 0 or vals[-1] != total or any(b < a for a, b in zip(vals, vals[1:])):
        raise GraphExecutionError(f"{name} must rise from 0 to the token count {total}, got {vals}")
    return vals


def _packed_attention(q, k, v, cu_q, cu_kv, nonpad, scale, causal, softcap):
    """q [Tq, Hq, D], k [Tkv, Hkv, D], v [Tkv, Hkv, Dv] in token-major order; sequence ``i`` owns rows cu[i]:cu[i+1]."""
    hq, hkv = q.shape[1], k.shape[1]
    if hq % hkv:
        raise GraphExecutionError(f"{hq} query heads do not group over {hkv} KV heads")
    cq, ckv = _offsets(cu_q, "cu_seqlens_q", q.shape[0]), _offsets(cu_kv, "cu_seqlens_kv", k.shape[0])
    if len(cq) != len(ckv):
        raise GraphExecutionError(f"cu_seqlens_q and cu_seqlens_kv differ in length: {len(cq)} vs {len(ckv)}")
    keep = [int(n) for n in nonpad.reshape(-1).tolist()] if nonpad is not None else None
    if keep is not None and len(keep) != len(cq) - 1:
        raise GraphExecutionError(f"nonpad_kv_seqlen has {len(keep)} entries for {len(cq) - 1} sequences")
    out = torch.zeros(q.shape[0], hq, v.shape[2], device=q.device)
    for i in range(len(cq) - 1):
        ql, kl = cq[i + 1] - cq[i], ckv[i + 1] - ckv[i]
        if keep is not None:
            kl = min(max(keep[i], 0), kl)
        if ql == 0 or kl == 0:
            continue
        qs = q[cq[i]:cq[i + 1]].float().transpose(0, 1)                                    # [Hq, ql, D]
        ks = k[ckv[i]:ckv[i] + kl].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)
        vs = v[ckv[i]:ckv[i] + kl].float().transpose(0, 1).repeat_interleave(hq // hkv, dim=0)
        scores = (qs * scale ** 0.5) @ (ks * scale ** 0.5).transpose(-1, -2)
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        if causal:                                                                          # the last query row sees every key
            scores = scores.masked_fill(~torch.ones(ql, kl, dtype=torch.bool, device=q.device).tril(kl - ql), float("-inf"))
        dead = torch.isneginf(scores).all(dim=-1, keepdim=True)
        probs = torch.softmax(scores.masked_fill(dead, 0.0), dim=-1).masked_fill(dead, 0.0)
        out[cq[i]:cq[i + 1]] = (probs @ vs).transpose(0, 1)
    return out


def _varlen_attention(ins, attrs):
    """pkg.nxrt::VarlenAttention: padding-free attention over [tokens, heads, dim] tensors cut by cumulative lengths;
    optional ``nonpad_kv_seqlen`` [batch] shortens each sequence's keys; ``is_causal`` aligns the last query with the last key."""
    q, k, v = ins[0], ins[1], ins[2]
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise GraphExecutionError("VarlenAttention takes [tokens, heads, dim] query, key and value")
    scale = float(attrs.get("scale", 0.0)) or q.shape[-1] ** -0.5
    out = _packed_attention(q, k, v, ins[3], ins[4], _opt(ins, 5), scale, bool(attrs.get("is_causal", 0)), float(attrs.get("softcap", 0.0)))
    return out.to(q.dtype)


def _packed_varlen_attention(ins, attrs):
    """pkg.nxrt::PackedVarlenAttention: the same over [tokens, heads * dim] rows, head counts from the attributes."""
    q, k, v = ins[0], ins[1], ins[2]
    h = int(attrs["num_heads"])
    hkv = int(attrs.get("kv_num_heads", h) or h)

    def heads(x, n, name):
        if x.dim() == 3:
            return x
        if x.dim() != 2 or x.shape[1] % n:
            raise GraphExecutionError(f"PackedVarlenAttention: {name} {list(x.shape)} is not [tokens, {n} heads * dim]")
        return x.reshape(x.shape[0], n, -1)

    q3, k3, v3 = heads(q, h, "query"), heads(k, hkv, "key"), heads(v, hkv, "value")
    scale = float(attrs.get("scale", 0.0)) or q3.shape[-1] ** -0.5
    out = _packed_attention(q3, k3, v3, ins[3], ins[4], None, scale, bool(attrs.get("is_causal", 0)), float(attrs.get("softcap", 0.0)))
    return (out if q.dim() == 3 else out.reshape(q.shape[0], -1)).to(q.dtype)


def _fused_attention(ins, attrs):
    """com.microsoft::FusedAttention: softmax(Q K^T * scale + mask) V, with K optionally given already transposed."""
    q, k, v, mask = ins[0].float(), ins[1].float(), ins[2].float(), _opt(ins, 3)
    scores = q @ (k if int(attrs.get("k_transposed", 0)) else k.transpose(-1, -2)) * float(attrs.get("scale", 1.0))
    if mask is not None:
        scores = scores + mask.float()
    return (torch.softmax(scores, dim=-1) @ v).to(ins[0].dtype)


def _gather_block_quantized(ins, attrs):
    """com.microsoft::GatherBlockQuantized over uint8 storage: rows picked along axis 0 of a table quantised in blocks of
    the last axis (8 bits, or 4 / 2 bits packed low bits first); value = (q - zero_point) * scale."""
    data, idx, scales, zp = ins[0], ins[1].long(), ins[2], _opt(ins, 3)
    bits, block = int(attrs.get("bits", 4)), int(attrs.get("block_size", 128))
    if data.dtype != torch.uint8 or bits not in (2, 4, 8):
        raise GraphExecutionError("GatherBlockQuantized is covered for uint8 storage of 2, 4 or 8 bits")
    last = data.dim() - 1
    if int(attrs.get("gather_axis", 0)) % data.dim() != 0 or int(attrs.get("quantize_axis", 1)) % data.dim() != last:
        raise GraphExecutionError("GatherBlockQuantized over uint8 gathers along axis 0 and quantises along the last axis")
    if bool(((idx < -data.shape[0]) | (idx >= data.shape[0])).any()):
        raise GraphExecutionError(f"GatherBlockQuantized: an index lies outside the {data.shape[0]} rows")
    pack, mask = 8 // bits, (1 << bits) - 1

    def unpack(t):
        t32 = t.to(torch.int32)
        return torch.stack([(t32 >> (bits * i)) & mask for i in range(pack)], dim=-1).reshape(*t.shape[:-1], t.shape[-1] * pack)

    rows = unpack(data[idx]).float()
    width = rows.shape[-1]
    s = scales[idx].float().repeat_interleave(block, dim=-1)[..., :width]
    if zp is not None:
        z = unpack(zp[idx])[..., : scales.shape[-1]].float().repeat_interleave(block, dim=-1)[..., :width]
    else:
        z = float(1 << (bits - 1))
    return ((rows - z) * s).to(scales.dtype)


def _block_quantized_moe(ins, attrs):
    """pkg.nxrt::BlockQuantizedMoE: the mixture-of-experts layer with self-describing block-format expert weights.

    Inputs (dense order): hidden states, router logits, fc1 weights [E, out, blocks, block bytes], fc1 bias, fc2 weights,
    fc2 bias, optional separate gate weights and bias, optional aggregation weights [rows, E].  Only the experts the
    router selects are decoded.  Activation, SwiGLU fusion and routing attributes are those of ``QMoE``.
    """
    fmt = attrs.get("format")
    fmt = fmt.decode() if isinstance(fmt, bytes) else str(fmt)
    if int(attrs.get("block_layout_version", 1)) != 1:
        raise GraphExecutionError(f"BlockQuantizedMoE block_layout_version {attrs.get('block_layout_version')} is unknown (known: 1)")
    x, router = ins[0], ins[1]
    hidden = x.shape[-1]
    experts = router.shape[-1]
    k = int(attrs.get("k", 1))
    if not 0 < k <= experts:
        raise GraphExecutionError(f"BlockQuantizedMoE: k={k} must lie in 1..{experts}")
    chosen = torch.unique(torch.topk(router.reshape(-1, experts).float(), k, dim=-1).indices).tolist()

    def dense(packed, width):
        if packed is None:
            return None
        if packed.dim() != 4 or packed.shape[0] != experts:
            raise GraphExecutionError(f"BlockQuantizedMoE: packed expert weights must be [{experts}, out, blocks, bytes], got {list(packed.shape)}")
        out = torch.zeros(experts, packed.shape[1], width, device=packed.device)
        for e in chosen:                                               # experts nobody routed to stay packed
            out[e] = decode_weight_blocks(packed[e], fmt)[:, :width]
        return out

    w1 = dense(ins[2], hidden)
    fused = attrs.get("activation_type", "relu") == "swiglu" and int(attrs.get("swiglu_fusion", 0)) in (1, 2)
    inter = w1.shape[1] // 2 if fused else w1.shape[1]
    w2, w3 = dense(ins[4], inter), dense(_opt(ins, 6), hidden)
    return _moe_core(x, router, w1, _opt(ins, 3), w2, _opt(ins, 5), w3, _opt(ins, 7), attrs, agg=_opt(ins, 8))


def _sparse_kv_gather(ins, attrs):
    """pkg.nxrt::SparseKvGather: cache [B, G, C, D] and indices [B, G, Q, K] -> the selected rows [B, G, Q, K, D], index
    order and duplicates kept.  A negative index, one at or past the cache length, or one at or past the row's optional
    ``valid_lengths`` [B] entry is an error (crates/onnx-runtime-ep-cpu/src/kernels/sparse_kv_gather.rs:72-126)."""
    cache, idx = ins[0], ins[1].long()
    lengths = _opt(ins, 2)
    if int(attrs.get("index_layout_version", 1)) != 1 or (attrs.get("out_of_range", "error") or "error") != "error":
        raise GraphExecutionError("SparseKvGather knows index_layout_version 1 with out_of_range='error' only")
    if cache.dim() != 4 or idx.dim() != 4 or cache.shape[:2] != idx.shape[:2]:
        raise GraphExecutionError(f"SparseKvGather: cache {list(cache.shape)} must be [B, G, C, D] and indices {list(idx.shape)} [B, G, Q, K] with equal B and G")
    limit = torch.full((cache.shape[0],), cache.shape[2], dtype=torch.int64, device=cache.device)
    if lengths is not None:
        lengths = lengths.long().reshape(-1)
        if lengths.numel() != cache.shape[0] or bool(((lengths < 0) | (lengths > cache.shape[2])).any()):
            raise GraphExecutionError(f"SparseKvGather: valid_lengths must be [{cache.shape[0]}] values in 0..{cache.shape[2]}")
        limit = lengths
    bad = (idx < 0) | (idx >= limit[:, None, None, None])
    if bool(bad.any()):
        where = [int(v) for v in bad.nonzero()[0].tolist()]
        raise GraphExecutionError(f"SparseKvGather: index {int(idx[tuple(where)])} at {where} lies outside the {int(limit[where[0]])} valid cache rows")
    b, g, q, k = idx.shape
    if cache.is_cuda:
        from ..ops import sequence as _seq

        got = _seq.sparse_kv_gather(cache, idx, lengths)       # the indices were checked above; the kernel checks them again
        if got is not None:
            return got
    picked = torch.gather(cache, 2, idx.reshape(b, g, q * k, 1).expand(b, g, q * k, cache.shape[3]))
    return picked.reshape(b, g, q, k, cache.shape[3])


def _scan(self, n, ins, env):
    """Scan (opset 9+): state variables threaded through the body, scan inputs sliced along their axes (optionally
    reversed), scan outputs stacked along theirs."""
    body = n.attrs["body"]
    m = int(n.attrs["num_scan_inputs"])
    n_state = len(ins) - m
    state, scans = list(ins[:n_state]), list(ins[n_state:])
    in_axes = [int(a) for a in n.attrs.get("scan_input_axes") or [0] * m]
    in_dirs = [int(d) for d in n.attrs.get("scan_input_directions") or [0] * m]
    k = len(body.outputs) - n_state
    out_axes = [int(a) for a in n.attrs.get("scan_output_axes") or [0] * k]
    out_dirs = [int(d) for d in n.attrs.get("scan_output_directions") or [0] * k]
    length = scans[0].shape[in_axes[0] % scans[0].dim()] if scans else 0
    names = [vi.name for vi in body.inputs]
    collected = [[] for _ in range(k)]
    for step in range(length):
        slices = [s.select(a % s.dim(), length - 1 - step if d else step) for s, a, d in zip(scans, in_axes, in_dirs)]
        res = self._run_body(body, env, dict(zip(names, state + slices)))
        state = list(res[:n_state])
        for j in range(k):
            collected[j].append(res[n_state + j])
    outs = []
    for j in range(k):
        items = collected[j][::-1] if out_dirs[j] else collected[j]
        if not items:
            raise GraphExecutionError("Scan over zero iterations has no shape for its scan outputs")
        outs.append(torch.stack(items, dim=out_axes[j] % (items[0].dim() + 1)))
    return state + outs


OPS.update({
    "LinearAttention": _linear_attention, "CausalConvWithState": _causal_conv_with_state, "VarlenAttention": _varlen_attention,
    "PackedVarlenAttention": _packed_varlen_attention, "FusedAttention": _fused_attention, "GatherBlockQuantized": _gather_block_quantized,
    "BlockQuantizedMoE": _block_quantized_moe, "SparseKvGather": _sparse_kv_gather,
})
