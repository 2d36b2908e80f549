"""Operators of hybrid and padding-free decoders, each against a direct loop over its definition."""
import numpy as np
import pytest
import torch

from onnx_genai_b200.package import onnx_pb as pb
from onnx_genai_b200.package.graph_executor import OPS, GraphExecutionError, GraphExecutor


def _linear_attention_loop(q, k, v, past, decay, beta, hq, hkv, rule, scale):
    """The recurrence written out per batch row, KV head and token."""
    b, t = q.shape[0], q.shape[1]
    dk, dv = q.shape[2] // hq, v.shape[2] // hkv
    nk = k.shape[2] // dk
    out_heads = max(hq, hkv)
    out = torch.zeros(b, t, out_heads * dv)
    state = past.clone() if past is not None else torch.zeros(b, hkv, dk, dv)
    for bi in range(b):
        for h in range(hkv):
            s = state[bi, h]
            hk = h // (hkv // nk)
            for ti in range(t):
                kt, vt = k[bi, ti, hk * dk:(hk + 1) * dk], v[bi, ti, h * dv:(h + 1) * dv]
                if rule in ("gated", "gated_delta"):
                    g = decay[bi, ti].reshape(hkv, -1)[h]
                    s = s * torch.exp(g)[:, None] if g.numel() == dk else s * torch.exp(g)
                if rule in ("delta", "gated_delta"):
                    bt = beta[bi, ti].reshape(-1)
                    vt = (bt[h] if bt.numel() == hkv else bt[0]) * (vt - s.T @ kt)
                s = s + kt[:, None] * vt[None, :]
                if hq >= hkv:
                    for g_ in range(hq // hkv):
                        qh = h * (hq // hkv) + g_
                        out[bi, ti, qh * dv:(qh + 1) * dv] = scale * (q[bi, ti, qh * dk:(qh + 1) * dk] @ s)
                else:
                    qh = h * hq // hkv
                    out[bi, ti, h * dv:(h + 1) * dv] = scale * (q[bi, ti, qh * dk:(qh + 1) * dk] @ s)
            state[bi, h] = s
    return out, state


@pytest.mark.parametrize("rule", ["linear", "gated", "delta", "gated_delta"])
@pytest.mark.parametrize("hq, nk, hkv, per_dim", [(4, 2, 2, False), (2, 2, 4, True), (2, 1, 2, False)])
def test_linear_attention_rules_and_head_groupings(rule, hq, nk, hkv, per_dim):
    g = torch.Generator().manual_seed(hq * 10 + hkv)
    b, t, dk, dv = 2, 5, 4, 3
    q, k, v = torch.randn(b, t, hq * dk, generator=g), torch.randn(b, t, nk * dk, generator=g), torch.randn(b, t, hkv * dv, generator=g)
    k = k / k.reshape(b, t, nk, dk).norm(dim=-1, keepdim=True).repeat_interleave(dk, -1).reshape(b, t, -1)
    past = torch.randn(b, hkv, dk, dv, generator=g)
    decay = -torch.rand(b, t, hkv * dk if per_dim else hkv, generator=g)
    beta = torch.rand(b, t, 1 if per_dim else hkv, generator=g)
    attrs = {"q_num_heads": hq, "kv_num_heads": hkv, "update_rule": rule}
    out, state = OPS["LinearAttention"]([q, k, v, past, decay, beta], attrs)
    want_out, want_state = _linear_attention_loop(q, k, v, past, decay, beta, hq, hkv, rule, dk ** -0.5)
    assert tuple(out.shape) == (b, t, max(hq, hkv) * dv)
    assert torch.allclose(out, want_out, atol=1e-5) and torch.allclose(state, want_state, atol=1e-5)
    # the state is the whole memory: two tokens then three, threading the state, equals five at once
    o1, s1 = OPS["LinearAttention"]([q[:, :2], k[:, :2], v[:, :2], past, decay[:, :2], beta[:, :2]], attrs)
    o2, s2 = OPS["LinearAttention"]([q[:, 2:], k[:, 2:], v[:, 2:], s1, decay[:, 2:], beta[:, 2:]], attrs)
    assert torch.allclose(torch.cat([o1, o2], 1), out, atol=1e-5) and torch.allclose(s2, state, atol=1e-5)


def test_linear_attention_refuses_what_it_cannot_group():
    x = torch.zeros(1, 1, 12)
    with pytest.raises(GraphExecutionError, match="update_rule"):
        OPS["LinearAttention"]([x, x, x], {"q_num_heads": 3, "kv_num_heads": 3, "update_rule": "softmax"})
    with pytest.raises(GraphExecutionError, match="group evenly"):
        OPS["LinearAttention"]([x, x, x], {"q_num_heads": 3, "kv_num_heads": 2, "update_rule": "linear"})
    with pytest.raises(GraphExecutionError, match="gate input"):
        OPS["LinearAttention"]([x, x, x], {"q_num_heads": 3, "kv_num_heads": 3})


def test_causal_conv_with_state_streams_like_one_long_convolution():
    g = torch.Generator().manual_seed(5)
    b, c, length, k = 2, 6, 9, 4
    x, w, bias = torch.randn(b, c, length, generator=g), torch.randn(c, 1, k, generator=g), torch.randn(c, generator=g)
    y, state = OPS["CausalConvWithState"]([x, w, bias], {"activation": "silu"})
    want = torch.zeros(b, c, length)
    for t in range(length):
        for j in range(k):
            src = t + j - (k - 1)
            if src >= 0:
                want[:, :, t] += w[:, 0, j] * x[:, :, src]
    want = torch.nn.functional.silu(want + bias[None, :, None])
    assert torch.allclose(y, want, atol=1e-5) and torch.equal(state, x[:, :, -(k - 1):])
    # prefill of five frames, then one frame at a time with the rolling state
    y1, st = OPS["CausalConvWithState"]([x[:, :, :5], w, bias], {"activation": "swish"})
    parts = [y1]
    for t in range(5, length):
        yt, st = OPS["CausalConvWithState"]([x[:, :, t:t + 1], w, bias, st], {"activation": "silu"})
        parts.append(yt)
    assert torch.allclose(torch.cat(parts, dim=2), y, atol=1e-5) and torch.allclose(st, state)
    # a prompt shorter than the filter keeps zeros at the front of the state
    _, short = OPS["CausalConvWithState"]([x[:, :, :2], w, None], {})
    assert torch.equal(short[:, :, 0], torch.zeros(b, c)) and torch.equal(short[:, :, 1:], x[:, :, :2])
    with pytest.raises(GraphExecutionError, match="activation"):
        OPS["CausalConvWithState"]([x, w, bias], {"activation": "relu"})


def _dense_attention(q, k, v, causal, softcap=0.0):
    """q [H, ql, D], k / v [H, kl, D]: the plain definition, last query aligned with the last key."""
    scores = q @ k.transpose(-1, -2) / q.shape[-1] ** 0.5
    if softcap:
        scores = softcap * torch.tanh(scores / softcap)
    if causal:
        ql, kl = q.shape[1], k.shape[1]
        scores = scores.masked_fill(~torch.ones(ql, kl, dtype=torch.bool).tril(kl - ql), float("-inf"))
    return torch.softmax(scores, -1) @ v


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention_equals_per_sequence_attention(causal):
    g = torch.Generator().manual_seed(7)
    hq, hkv, d, dv = 4, 2, 8, 6
    q_lens, kv_lens = [3, 1, 4], [5, 6, 4]
    q, k, v = torch.randn(sum(q_lens), hq, d, generator=g), torch.randn(sum(kv_lens), hkv, d, generator=g), torch.randn(sum(kv_lens), hkv, dv, generator=g)
    cu_q, cu_kv = torch.tensor(np.cumsum([0] + q_lens), dtype=torch.int32), torch.tensor(np.cumsum([0] + kv_lens), dtype=torch.int32)
    nonpad = torch.tensor([5, 4, 4])                                                        # the second sequence's last two keys are padding
    out = OPS["VarlenAttention"]([q, k, v, cu_q, cu_kv, nonpad], {"is_causal": int(causal), "softcap": 20.0})
    assert tuple(out.shape) == (sum(q_lens), hq, dv)
    for i in range(3):
        ql, kl = slice(int(cu_q[i]), int(cu_q[i + 1])), slice(int(cu_kv[i]), int(cu_kv[i]) + int(nonpad[i]))
        want = _dense_attention(q[ql].transpose(0, 1), k[kl].transpose(0, 1).repeat_interleave(2, 0), v[kl].transpose(0, 1).repeat_interleave(2, 0), causal, 20.0)
        assert torch.allclose(out[ql], want.transpose(0, 1), atol=1e-5), i
    packed = OPS["PackedVarlenAttention"]([q.reshape(-1, hq * d), k.reshape(-1, hkv * d), v.reshape(-1, hkv * dv), cu_q, cu_kv],
                                          {"num_heads": hq, "kv_num_heads": hkv, "is_causal": int(causal)})
    plain = OPS["VarlenAttention"]([q, k, v, cu_q, cu_kv], {"is_causal": int(causal)})
    assert tuple(packed.shape) == (sum(q_lens), hq * dv) and torch.allclose(packed, plain.reshape(-1, hq * dv), atol=1e-6)
    with pytest.raises(GraphExecutionError, match="cu_seqlens_kv"):
        OPS["VarlenAttention"]([q, k, v, cu_q, torch.tensor([0, 5, 11, 14])], {})


def test_fused_attention_and_block_quantised_gather():
    g = torch.Generator().manual_seed(9)
    q, k, v = torch.randn(2, 3, 4, 8, generator=g), torch.randn(2, 3, 5, 8, generator=g), torch.randn(2, 3, 5, 8, generator=g)
    mask = torch.randn(1, 1, 4, 5, generator=g)
    want = torch.softmax(q @ k.transpose(-1, -2) * 0.3 + mask, -1) @ v
    assert torch.allclose(OPS["FusedAttention"]([q, k, v, mask], {"scale": 0.3}), want, atol=1e-6)
    assert torch.allclose(OPS["FusedAttention"]([q, k.transpose(-1, -2).contiguous(), v, mask], {"scale": 0.3, "k_transposed": 1}), want, atol=1e-6)

    rows, width, block = 6, 64, 32
    data8 = torch.randint(0, 256, (rows, width), generator=g, dtype=torch.uint8)
    scales = torch.rand(rows, width // block, generator=g) + 0.1
    zps = torch.randint(0, 256, (rows, width // block), generator=g, dtype=torch.uint8)
    idx = torch.tensor([[5, 0], [2, -1]])
    got = OPS["GatherBlockQuantized"]([data8, idx, scales, zps], {"bits": 8, "block_size": block})
    want = (data8.float() - zps.float().repeat_interleave(block, 1)) * scales.repeat_interleave(block, 1)
    assert tuple(got.shape) == (2, 2, width) and torch.allclose(got, want[idx], atol=1e-6)
    # four bits: two values per byte, low nibble first; the default zero point is 8
    data4 = torch.randint(0, 256, (rows, width // 2), generator=g, dtype=torch.uint8)
    got = OPS["GatherBlockQuantized"]([data4, torch.tensor([1, 4]), scales], {"bits": 4, "block_size": block})
    nib = torch.stack([data4 & 0xF, data4 >> 4], dim=-1).reshape(rows, width).float()
    assert torch.allclose(got, ((nib - 8.0) * scales.repeat_interleave(block, 1))[[1, 4]], atol=1e-6)
    with pytest.raises(GraphExecutionError, match="outside"):
        OPS["GatherBlockQuantized"]([data8, torch.tensor([6]), scales], {"bits": 8, "block_size": block})


def test_scan_threads_state_and_stacks_outputs():
    """A running sum over rows: state = state + x_t; scan outputs are the running sum and x_t scaled by an outer value."""
    f32 = lambda name, shape: pb.ValueInfo(name, pb.FLOAT, shape)
    body = pb.Graph(name="body", nodes=[pb.Node("Add", ["acc", "row"], ["acc_out"], name="a"), pb.Node("Identity", ["acc_out"], ["running"], name="b"),
                                        pb.Node("Mul", ["row", "outer_scale"], ["scaled"], name="c")],
                    inputs=[f32("acc", (3,)), f32("row", (3,))], outputs=[f32("acc_out", (3,)), f32("running", (3,)), f32("scaled", (3,))])
    x = np.arange(12, dtype=np.float32).reshape(4, 3)

    def run(**attrs):
        node = pb.Node("Scan", ["init", "x"], ["final", "sums", "scaled_rows"], name="scan", attrs={"body": body, "num_scan_inputs": 1, **attrs})
        graph = pb.Graph(name="g", nodes=[node],
                         initializers={"outer_scale": pb.Tensor(name="outer_scale", dims=(), data_type=pb.FLOAT, array=np.asarray(2.0, dtype=np.float32))},
                         inputs=[f32("init", (3,)), f32("x", ("n", 3))], outputs=[f32("final", (3,)), f32("sums", ()), f32("scaled_rows", ())])
        return GraphExecutor(pb.Model(graph=graph), "cpu").run({"init": np.ones(3, dtype=np.float32), "x": x})

    out = run()
    assert out["final"].tolist() == (1 + x.sum(0)).tolist()
    assert np.allclose(out["sums"].numpy(), 1 + np.cumsum(x, axis=0)) and np.allclose(out["scaled_rows"].numpy(), 2 * x)
    rev = run(scan_input_directions=[1], scan_output_directions=[0, 1], scan_output_axes=[1, 0])
    assert np.allclose(rev["sums"].numpy(), (1 + np.cumsum(x[::-1], axis=0)).T)              # consumed back to front, stacked on axis 1
    assert np.allclose(rev["scaled_rows"].numpy(), 2 * x) and rev["final"].tolist() == out["final"].tolist()


@pytest.mark.parametrize("activation, fusion, gate", [("swiglu", 1, False), ("swiglu", 0, True), ("silu", 0, False)])
def test_block_quantised_moe_equals_dense_moe_on_the_decoded_weights(activation, fusion, gate):
    from onnx_genai_b200.package.graph_executor import decode_weight_blocks, encode_mxfp4

    g = torch.Generator().manual_seed(11)
    rows, hidden, inter, experts, k = 5, 64, 32, 6, 2
    fc1_out = 2 * inter if fusion else inter
    pack = lambda w: torch.stack([encode_mxfp4(w[e]) for e in range(w.shape[0])])
    unpack = lambda p, width: torch.stack([decode_weight_blocks(p[e], "mxfp4")[:, :width] for e in range(p.shape[0])])
    p1, p2 = pack(torch.randn(experts, fc1_out, hidden, generator=g)), pack(torch.randn(experts, hidden, inter, generator=g))
    p3 = pack(torch.randn(experts, inter, hidden, generator=g)) if gate else None
    b1, b2 = torch.randn(experts, fc1_out, generator=g), torch.randn(experts, hidden, generator=g)
    x, logits = torch.randn(rows, hidden, generator=g), torch.randn(rows, experts, generator=g)
    attrs = {"format": "mxfp4", "k": k, "activation_type": activation, "swiglu_fusion": fusion, "normalize_routing_weights": 1}
    got = OPS["BlockQuantizedMoE"]([x, logits, p1, b1, p2, b2, p3], attrs)
    assert tuple(p1.shape) == (experts, fc1_out, 2, 17) and tuple(got.shape) == (rows, hidden)
    dense_attrs = {kk: v for kk, v in attrs.items() if kk != "format"}
    want = OPS["MoE"]([x, logits, unpack(p1, hidden), b1, unpack(p2, inter), b2, unpack(p3, hidden) if gate else None], dense_attrs)
    assert torch.allclose(got, want, atol=1e-5)
    # aggregation weights replace the softmax of the logits but not the selection
    agg = torch.rand(rows, experts, generator=g)
    mixed = OPS["BlockQuantizedMoE"]([x, logits, p1, b1, p2, b2, p3, None, agg], {**attrs, "normalize_routing_weights": 0})
    one_hot = torch.zeros(rows, experts).scatter_(1, torch.topk(logits, k).indices, 1.0)
    assert not torch.allclose(mixed, got, atol=1e-3)
    by_hand = torch.zeros(rows, hidden)
    for e in range(experts):
        only = OPS["BlockQuantizedMoE"]([x, torch.where(torch.arange(experts) == e, 10.0, -10.0).expand(rows, experts), p1, b1, p2, b2, p3], {**attrs, "k": 1})
        by_hand += only * (agg[:, e] * one_hot[:, e])[:, None]
    assert torch.allclose(mixed, by_hand, atol=1e-4)
    with pytest.raises(GraphExecutionError, match="k=9"):
        OPS["BlockQuantizedMoE"]([x, logits, p1, b1, p2, b2, p3], {**attrs, "k": 9})


def test_sparse_kv_gather_keeps_order_and_refuses_bad_indices():
    cache = torch.arange(2 * 2 * 6 * 3, dtype=torch.float32).reshape(2, 2, 6, 3)
    idx = torch.tensor([[[[5, 0, 0]], [[1, 2, 3]]], [[[4, 4, 1]], [[0, 3, 2]]]])                 # [B=2, G=2, Q=1, K=3]
    out = OPS["SparseKvGather"]([cache, idx], {})
    assert tuple(out.shape) == (2, 2, 1, 3, 3)
    for b in range(2):
        for g in range(2):
            assert torch.equal(out[b, g, 0], cache[b, g, idx[b, g, 0]])
    assert torch.equal(OPS["SparseKvGather"]([cache, idx, torch.tensor([6, 5])], {}), out)
    with pytest.raises(GraphExecutionError, match=r"index 4 at \[1, 0, 0, 0\] lies outside the 4 valid"):
        OPS["SparseKvGather"]([cache, idx, torch.tensor([6, 4])], {})
    with pytest.raises(GraphExecutionError, match="index -1"):
        OPS["SparseKvGather"]([cache, torch.where(idx == 5, -1, idx)], {})
    with pytest.raises(GraphExecutionError, match="valid_lengths"):
        OPS["SparseKvGather"]([cache, idx, torch.tensor([6, 7])], {})
    with pytest.raises(GraphExecutionError, match="out_of_range"):
        OPS["SparseKvGather"]([cache, idx], {"out_of_range": "clamp"})
