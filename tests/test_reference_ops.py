"""CPU checks of the PyTorch statements that serve as the oracle for the CUDA kernels."""
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.ops import reference as ref


def test_pack_gate_up_roundtrip():
    torch.manual_seed(0)
    g, u = torch.randn(256, 32), torch.randn(256, 32)
    a = torch.randn(7, 32)
    for half in (32, 64, 128):
        got = ref.swiglu_packed(a, ref.pack_gate_up(g, u, half), half)
        want = torch.nn.functional.silu(a @ g.t()) * (a @ u.t())
        assert torch.allclose(got, want, atol=1e-5)


def test_paged_attention_matches_dense():
    torch.manual_seed(1)
    hq, hkv, d = 4, 2, 32
    ctx, qlen = 45, 7
    pages = (ctx + 15) // 16
    pool = torch.randn(pages + 2, hkv, 2, 16, d)
    table = torch.tensor([[2, 0, 4]], dtype=torch.int32)
    q = torch.randn(qlen, hq * d)
    out = ref.paged_attention(q, pool, table, torch.tensor([ctx]), torch.tensor([0, qlen]), hq, hkv, d)
    k = pool[table[0].long(), :, 0].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
    v = pool[table[0].long(), :, 1].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
    k = k.repeat_interleave(hq // hkv, 0)
    v = v.repeat_interleave(hq // hkv, 0)
    qh = q.view(qlen, hq, d).transpose(0, 1)
    mask = torch.ones(qlen, ctx, dtype=torch.bool).tril(ctx - qlen)
    want = torch.nn.functional.scaled_dot_product_attention(qh, k, v, attn_mask=mask)
    assert torch.allclose(out.view(qlen, hq, d).transpose(0, 1), want, atol=1e-5)


def test_w4_quant_roundtrip():
    torch.manual_seed(2)
    w = torch.randn(24, 96) * 0.02
    for sym in (True, False):
        q, s, zp = ref.quantize_w4(w, 32, symmetric=sym)
        assert q.shape == (24, 3, 16) and q.dtype == torch.uint8
        back = ref.dequant_w4(q, s, zp)
        assert float((back - w).abs().max()) <= float(s.max()) * 0.51 + 1e-6


def test_sampler_oracle_filters():
    w = torch.tensor([100, 50, 25, 10, 0, 5], dtype=torch.int64) * 1000
    assert ref.sample_from_weights(w, 1, 1.0, 0.0, 0.99) == 0
    assert ref.sample_from_weights(w, 0, 0.5, 0.0, 0.99) == 0
    assert ref.sample_from_weights(w, 0, 1.0, 0.0, 0.0) == 0
    assert ref.sample_from_weights(w, 0, 1.0, 0.0, 0.999) == 5
    assert ref.sample_from_weights(w, 2, 1.0, 0.0, 0.999) == 1


def test_cpu_dispatch_uses_reference():
    x = torch.randn(3, 32)
    wt = torch.randn(32)
    y = ops.rmsnorm(x, wt, 1e-6)
    assert torch.allclose(y, ref.rmsnorm(x, wt, 1e-6)[0])
    assert torch.equal(ops.argmax(torch.tensor([[1.0, 3.0, 3.0]])), torch.tensor([1], dtype=torch.int32))
