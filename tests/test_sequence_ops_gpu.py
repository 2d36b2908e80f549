"""CUDA kernels of the hybrid / sparse decoder operators against the graph executor's fp32 torch statement of the same
operator run on the CPU: linear attention (all four update rules, grouped heads both ways, per-dimension decay),
the causal convolution with a rolling state, attention over selected positions, the sparse row gather."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a GPU", allow_module_level=True)

from onnx_genai_b200 import ops  # noqa: E402
from onnx_genai_b200.package import graph_executor as ge  # noqa: E402
from onnx_genai_b200.package import graph_ops_sequence as gs  # noqa: E402

DEV = torch.device("cuda", 0)


def _cuda(ts):
    return [t.to(DEV) if t is not None else None for t in ts]


def _close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    if a.shape != b.shape:
        return False
    if a.numel() == 0:
        return True
    return float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max()))


@pytest.mark.parametrize("rule,hq,nk,hkv,dk,dv,per_dim,beta_one,dtype", [
    ("linear", 4, 4, 4, 64, 64, False, False, torch.float32),
    ("gated", 8, 2, 4, 32, 96, True, False, torch.float32),
    ("delta", 2, 2, 4, 64, 160, False, True, torch.float32),
    ("gated_delta", 4, 2, 2, 128, 128, False, False, torch.float32),
    ("gated_delta", 4, 4, 4, 64, 64, True, False, torch.bfloat16),
])
def test_linear_attention_matches_the_torch_statement(rule, hq, nk, hkv, dk, dv, per_dim, beta_one, dtype):
    torch.manual_seed(3)
    b, t = 2, 9
    q = torch.randn(b, t, hq * dk) * 0.5
    k = torch.nn.functional.normalize(torch.randn(b, t, nk, dk), dim=-1).reshape(b, t, nk * dk)
    v = torch.randn(b, t, hkv * dv) * 0.5
    past = torch.randn(b, hkv, dk, dv) * 0.1
    decay = -torch.rand(b, t, hkv * dk if per_dim else hkv) * 0.3
    beta = torch.rand(b, t, 1 if beta_one else hkv)
    ins = [x.to(dtype) for x in (q, k, v, past, decay, beta)]
    attrs = {"q_num_heads": hq, "kv_num_heads": hkv, "update_rule": rule}
    want_out, want_state = gs._linear_attention(ins, attrs)
    before = ops.launch_counts["linear_attention"]
    got_out, got_state = gs._linear_attention(_cuda(ins), attrs)
    torch.cuda.synchronize()
    assert ops.launch_counts["linear_attention"] == before + 1
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert _close(got_out, want_out, tol) and _close(got_state, want_state, tol)
    # no past state, a single decode token
    ins1 = [ins[0][:, :1], ins[1][:, :1], ins[2][:, :1], None, ins[4][:, :1], ins[5][:, :1]]
    w1, s1 = gs._linear_attention(ins1, attrs)
    g1, gs1 = gs._linear_attention(_cuda(ins1), attrs)
    assert _close(g1, w1, tol) and _close(gs1, s1, tol)


@pytest.mark.parametrize("k,l,act,with_past,dtype", [(4, 7, "silu", True, torch.float32), (4, 1, "silu", True, torch.bfloat16),
                                                     (3, 5, "none", False, torch.float32), (1, 4, "swish", False, torch.float16)])
def test_causal_conv_with_state_matches_the_torch_statement(k, l, act, with_past, dtype):
    torch.manual_seed(4)
    b, c = 3, 70
    x = torch.randn(b, c, l).to(dtype)
    w = (torch.randn(c, 1, k) * 0.5).to(dtype)
    bias = torch.randn(c).to(dtype)
    past = torch.randn(b, c, k - 1).to(dtype) if with_past else None
    attrs = {"activation": act}
    want = gs._causal_conv_with_state([x, w, bias, past], attrs)
    before = ops.launch_counts["causal_conv_state"]
    got = gs._causal_conv_with_state(_cuda([x, w, bias, past]), attrs)
    torch.cuda.synchronize()
    assert ops.launch_counts["causal_conv_state"] == before + 1
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert _close(got[0], want[0], tol) and _close(got[1], want[1], tol) and got[1].shape == want[1].shape


@pytest.mark.parametrize("n,nkv,d,sel_heads,with_bias,dtype", [(4, 2, 64, 4, False, torch.float32), (6, 3, 128, 1, True, torch.float32),
                                                               (4, 4, 32, 4, True, torch.bfloat16)])
def test_index_share_attention_matches_the_torch_statement(n, nkv, d, sel_heads, with_bias, dtype):
    torch.manual_seed(5)
    b, sq, past_len, new, ksel = 2, 3, 20, 3, 6
    total = past_len + new
    q = torch.randn(b, n, sq, d).to(dtype)
    k, v = torch.randn(b, nkv, new, d).to(dtype), torch.randn(b, nkv, new, d).to(dtype)
    pk, pv = torch.randn(b, nkv, past_len, d).to(dtype), torch.randn(b, nkv, past_len, d).to(dtype)
    sel = torch.full((b, sel_heads, sq, ksel), -1, dtype=torch.int64)
    g = torch.Generator().manual_seed(6)
    for bi in range(b):
        for h in range(sel_heads):
            for s in range(sq):
                cnt = int(torch.randint(1, ksel + 1, (1,), generator=g))
                sel[bi, h, s, :cnt] = torch.sort(torch.randperm(total, generator=g)[:cnt]).values
    bias = None
    if with_bias:
        bias = torch.randn(b, 1, sq, total).to(dtype)
        bias[0, 0, 0, int(sel[0, 0, 0, 0])] = float("-inf")            # one selected position masked out
    attrs = {"num_heads": n, "kv_num_heads": nkv}
    want = ge._index_share([q, k, v, pk, pv, sel, bias], attrs)
    before = ops.launch_counts["index_share_attention"]
    got = ge._index_share(_cuda([q, k, v, pk, pv, sel, bias]), attrs)
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_counts["index_share_attention"] == before + 1
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert _close(got[0], want[0], tol) and torch.equal(got[1].cpu(), want[1]) and torch.equal(got[2].cpu(), want[2])


def test_sparse_kv_gather_copies_rows_and_flags_bad_indices():
    torch.manual_seed(7)
    b, g, c, d, qn, kn = 2, 3, 11, 24, 2, 5
    cache = torch.randn(b, g, c, d)
    idx = torch.randint(0, 7, (b, g, qn, kn), dtype=torch.int64)
    lengths = torch.tensor([9, 7], dtype=torch.int64)
    want = gs._sparse_kv_gather([cache, idx, lengths], {})
    before = ops.launch_counts["sparse_kv_gather"]
    got = gs._sparse_kv_gather(_cuda([cache, idx, lengths]), {})
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_counts["sparse_kv_gather"] == before + 1 and torch.equal(got.cpu(), want)
    # the kernel's own check: an index past the row's valid length raises the status word and yields zeros
    from onnx_genai_b200.ops import sequence as seq

    bad = idx.clone()
    bad[1, 0, 0, 0] = 8                                   # row 1 is valid up to 7
    out = seq.sparse_kv_gather(cache.to(DEV).bfloat16(), bad.to(DEV), lengths.to(DEV))
    torch.cuda.synchronize()
    assert float(out[1, 0, 0, 0].abs().max()) == 0
    with pytest.raises(Exception):
        ops.check_status()
    ops.check_status()                                    # the word was reset: the context stays usable
