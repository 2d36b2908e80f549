"""C++ CPU kernels (csrc/cpu_ref) against the fp32 PyTorch statements of the same ops."""
import math

import pytest
import torch

from onnx_genai_b200.ops import cpu, reference

pytestmark = pytest.mark.skipif(not cpu.available(), reason="runtime library not built")


@pytest.mark.parametrize("m,n,k,sym", [(1, 96, 64, True), (4, 130, 688, True), (7, 64, 100, False), (33, 48, 256, False)])
def test_matmul_nbits_matches_dequant_matmul(m, n, k, sym):
    torch.manual_seed(0)
    w = torch.randn(n, k) * 0.1
    q, s, zp = reference.quantize_w4(w, 32, symmetric=sym)
    x = torch.randn(m, k)
    bias = torch.randn(n)
    want = x @ reference.dequant_w4(q, s, zp, 32, k).t() + bias
    got = cpu.matmul_nbits(x, q, s, zp, bias, k)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
    assert torch.allclose(cpu.dequant_nbits(q, s, zp, k), reference.dequant_w4(q, s, zp, 32, k), atol=1e-7)


def test_gemm_rmsnorm_silu():
    torch.manual_seed(1)
    x, w, b, r = torch.randn(5, 77), torch.randn(19, 77), torch.randn(19), torch.randn(5, 19)
    assert torch.allclose(cpu.gemm(x, w, b, r), x @ w.t() + b + r, rtol=1e-4, atol=1e-4)
    xx, d, g = torch.randn(6, 96), torch.randn(6, 96), torch.rand(96) + 0.5
    y, nx = cpu.rmsnorm(xx, g, 1e-6, d)
    yr, nxr = reference.rmsnorm(xx, g, 1e-6, d)
    assert torch.allclose(y, yr, rtol=1e-5, atol=1e-5) and torch.allclose(nx, nxr)
    gu = torch.randn(3, 64)
    assert torch.allclose(cpu.silu_mul(gu), reference.silu_mul(gu), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("interleaved,rotary", [(False, 16), (True, 16), (False, 8)])
def test_rope_append_and_paged_attention(interleaved, rotary):
    torch.manual_seed(2)
    hq, hkv, d = 4, 2, 16
    cs = reference.rope_table(64, rotary, 10000.0)
    lens, q_lens = [19, 5, 33], [19, 2, 1]                    # fresh prefill, chunk continuing a sequence, decode row
    pages_per = 3
    pool_a = torch.randn(16, hkv, 2, 16, d)
    pool_b = pool_a.clone()
    table = torch.randperm(16)[: len(lens) * pages_per].to(torch.int32).view(len(lens), pages_per)
    t = sum(q_lens)
    qkv_a = torch.randn(t, (hq + 2 * hkv) * d)
    qkv_b = qkv_a.clone()
    pos, slots = [], []
    for s, (ctx, qn) in enumerate(zip(lens, q_lens)):
        for p_ in range(ctx - qn, ctx):
            pos.append(p_)
            slots.append(int(table[s, p_ // 16]) * 16 + p_ % 16)
    pos, slots = torch.tensor(pos, dtype=torch.int32), torch.tensor(slots, dtype=torch.int32)
    reference.rope_kv_append(qkv_a, pos, slots, cs, pool_a, hq, hkv, d, rotary, interleaved)
    cpu.rope_kv_append(qkv_b, pos, slots, cs, pool_b, hq, hkv, d, rotary, interleaved)
    assert torch.allclose(qkv_a, qkv_b, atol=1e-6) and torch.allclose(pool_a, pool_b, atol=1e-6)
    ctx_len = torch.tensor(lens, dtype=torch.int32)
    cu = torch.tensor([0, 19, 21, 22], dtype=torch.int32)
    for window in (0, 7):
        want = reference.paged_attention(qkv_a, pool_a, table, ctx_len, cu, hq, hkv, d, 1 / math.sqrt(d), window)
        got = cpu.paged_attention(qkv_b, pool_b, table, ctx_len, cu, hq, hkv, d, 1 / math.sqrt(d), window)
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), window
    with pytest.raises(IndexError):
        cpu.rope_kv_append(qkv_b, pos + 1000, slots, cs, pool_b, hq, hkv, d, rotary, interleaved)


def test_argmax_and_sampler_follow_the_integer_statement():
    torch.manual_seed(3)
    logits = torch.randn(64, 500) * 3
    logits[0, 7] = logits[0, 3] = logits[0].max() + 1          # tie: lowest index wins
    logits[1, 0] = float("nan")
    assert torch.equal(cpu.argmax(logits), reference.argmax(logits))
    temp = torch.full((64,), 0.8)
    temp[5] = 0.0
    top_k = torch.tensor([0, 40, 5, 0] * 16, dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 0.5, 1.0] * 16)
    min_p = torch.tensor([0.0, 0.0, 0.05, 0.2] * 16)
    u = torch.rand(64)
    clean = torch.nan_to_num(logits, nan=-1e30)
    got = cpu.sample(clean, temp, top_k, top_p, min_p, u)
    want = reference.sample(clean, temp, top_k, top_p, min_p, u)
    assert (got == want).float().mean() >= 0.97             # exp() rounding may move a weight by one unit at a threshold
    assert int(got[5]) == int(reference.argmax(clean[5:6])[0])


def test_ops_route_fp32_cpu_tensors_to_the_cpp_kernels():
    from onnx_genai_b200 import ops

    before = dict(cpu.calls)
    x = torch.randn(4, 32)
    ops.rmsnorm(x, torch.ones(32), 1e-6)
    ops.silu_mul(torch.randn(4, 64))
    ops.argmax(torch.randn(2, 50))
    for name in ("rmsnorm", "silu_mul", "argmax"):
        assert cpu.calls.get(name, 0) == before.get(name, 0) + 1, name


def test_int4_package_runs_on_the_cpp_kernels_and_matches_dense_weights(tmp_path):
    """The CPU-only configuration end to end: exported int4 package -> Engine -> greedy tokens, with the packed
    weights read by the C++ MatMulNBits kernel and, as the oracle, dequantised to dense fp32 at load."""
    import numpy as np

    from onnx_genai_b200.bench.config_bench import _export
    from onnx_genai_b200.engine.api import Engine, GenerateOptions

    cfg = _export("tiny-llama", str(tmp_path), "fp32", layers=2)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (32, 17)]
    opt = GenerateOptions(max_new_tokens=8, greedy=True, ignore_eos=True)
    before = cpu.calls.get("matmul_nbits", 0)
    packed = Engine.from_dir(str(tmp_path), device="cpu", max_seqs=4, max_seq_len=64, keep_int4=True).generate_batch(prompts, opt)
    assert cpu.calls.get("matmul_nbits", 0) > before
    dense = Engine.from_dir(str(tmp_path), device="cpu", max_seqs=4, max_seq_len=64, keep_int4=False).generate_batch(prompts, opt)
    assert [r.token_ids for r in packed] == [r.token_ids for r in dense]
