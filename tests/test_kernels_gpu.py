"""Numerics of every sm_100a kernel against the fp32 PyTorch statement of the same op."""
import math

import pytest
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("m,n,k,bn", [
    (128, 256, 64, 256), (200, 384, 512, 128), (1, 3584, 3584, 0), (300, 4608, 3584, 256),
    (257, 1000, 448, 64), (77, 96, 128, 32), (1300, 3584, 2368, 0),
])
def test_gemm_tcgen05(m, n, k, bn):
    torch.manual_seed(0)
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    bias = torch.randn(n, device=DEV).bfloat16()
    out = ops.gemm(a, w, bias=bias, bn=bn)
    torch.cuda.synchronize()
    ops.check_status()
    want = ref.gemm(a, w, bias, out_dtype=torch.float32)
    assert _rel_err(out, want) < 1e-2
    out32 = ops.gemm(a, w, out_f32=True, bn=bn)
    assert _rel_err(out32, ref.gemm(a, w, out_dtype=torch.float32)) < 1e-5 + 1e-3


@pytest.mark.parametrize("m,n,k,epi", [(1280, 3584, 18944, "residual"), (1280, 4608, 3584, "bias"), (256, 4608, 3584, "none"),
                                       (1500, 3584, 2368, "none"), (1280, 9472, 3584, "swiglu"), (200, 768, 3584, "bias"),
                                       (128, 256, 8192, "none")])
def test_gemm_stream_k_matches_data_parallel_and_fp32(m, n, k, epi):
    """Tile counts that are not a multiple of the SM count run stream-K: k-block ranges cross tile boundaries, partial
    accumulators meet in the fp32 workspace.  Results must match the fp32 statement like the data-parallel kernel's."""
    torch.manual_seed(m + n + k)
    a = (torch.randn(m, k, device=DEV) * 0.1).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    bias = (torch.randn(n, device=DEV) * 0.1).bfloat16() if epi == "bias" else None
    res = torch.randn(m, n, device=DEV).bfloat16() if epi == "residual" else None
    if epi == "swiglu":
        gate, up = w[: n // 2].contiguous(), w[n // 2:].contiguous()
        wp = ops.pack_gate_up(gate, up, 128)
        run = lambda: ops.gemm(a, wp, epilogue="swiglu", swiglu_half=128)
        want = torch.nn.functional.silu(a.float() @ gate.float().t()) * (a.float() @ up.float().t())
    else:
        run = lambda: ops.gemm(a, w, bias=bias, residual=res, epilogue="residual" if res is not None else "none")
        want = a.float() @ w.float().t()
        if bias is not None:
            want = want + bias.float()
        if res is not None:
            want = want + res.float()
    old = ops.set_stream_k(True)
    try:
        got_sk = run().float()
        got_sk2 = run().float()                    # the workspace and its flags are reused by the next launch
        ops.set_stream_k(False)
        got_dp = run().float()
    finally:
        ops.set_stream_k(old)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel_err(got_sk, want) < 1e-2 and _rel_err(got_dp, want) < 1e-2
    assert torch.equal(got_sk, got_sk2)
    assert _rel_err(got_sk, got_dp) < 4e-3         # the same products, summed in a different order


def test_gemm_residual_in_place():
    torch.manual_seed(1)
    m, n, k = 390, 3584, 512
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    res = torch.randn(m, n, device=DEV).bfloat16()
    want = ref.gemm(a, w, None, res, "residual", torch.float32)
    got = ops.gemm(a, w, residual=res, epilogue="residual", out=res)
    torch.cuda.synchronize()
    ops.check_status()
    assert got.data_ptr() == res.data_ptr()
    assert _rel_err(got, want) < 1e-2


@pytest.mark.parametrize("half", [32, 64, 128])
def test_gemm_swiglu(half):
    torch.manual_seed(2)
    m, inter, k = 333, 1024, 896
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    g = (torch.randn(inter, k, device=DEV) * 0.05).bfloat16()
    u = (torch.randn(inter, k, device=DEV) * 0.05).bfloat16()
    packed = ops.pack_gate_up(g, u, half)
    got = ops.gemm(a, packed, epilogue="swiglu", swiglu_half=half)
    torch.cuda.synchronize()
    ops.check_status()
    want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
    assert got.shape == (m, inter)
    assert _rel_err(got, want) < 1.5e-2


@pytest.mark.parametrize("rows,hidden", [(5, 896), (300, 3584), (3, 16384)])
def test_rmsnorm(rows, hidden):
    torch.manual_seed(3)
    x = torch.randn(rows, hidden, device=DEV).bfloat16()
    w = torch.randn(hidden, device=DEV).bfloat16()
    want, _ = ref.rmsnorm(x, w, 1e-6)
    got = ops.rmsnorm(x, w, 1e-6)
    assert _rel_err(got, want) < 5e-3
    delta = torch.randn(rows, hidden, device=DEV).bfloat16()
    x2 = x.clone()
    want2, newx = ref.rmsnorm(x, w, 1e-6, delta)
    got2 = ops.rmsnorm(x2, w, 1e-6, delta=delta)
    assert torch.equal(x2, newx)
    assert _rel_err(got2, want2) < 5e-3


def test_embedding_bounds():
    table = torch.randn(100, 64, device=DEV).bfloat16()
    ids = torch.tensor([0, 5, 99], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    bad = torch.tensor([3, 100], dtype=torch.int32, device=DEV)
    ops.embedding(bad, table)
    with pytest.raises(Exception, match="index out of range"):
        ops.check_status()
    ops.check_status()  # word was reset


def _make_paged(num_seqs, ctx_lens, hkv, d, extra_pages=3, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_per = [(c + ref.PAGE - 1) // ref.PAGE for c in ctx_lens]
    total = sum(pages_per) + extra_pages
    perm = torch.randperm(total, generator=g)
    max_pages = max(pages_per)
    table = torch.zeros(num_seqs, max_pages, dtype=torch.int32)
    o = 0
    for s, n in enumerate(pages_per):
        table[s, :n] = perm[o:o + n].to(torch.int32)
        o += n
    pool = (torch.randn(total, hkv, 2, ref.PAGE, d, generator=g) * 0.5).bfloat16()
    return pool.to(DEV), table.to(DEV)


@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (14, 2, 64), (4, 1, 128), (3, 1, 128)])
def test_paged_decode(hq, hkv, d):
    torch.manual_seed(4)
    ctx = [1, 15, 16, 17, 63, 64, 65, 300, 1000]
    n = len(ctx)
    pool, table = _make_paged(n, ctx, hkv, d)
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    q = torch.randn(n, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    out = torch.zeros(n, hq * d, device=DEV, dtype=torch.bfloat16)
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d)
    for splits in (1, 4):
        out.zero_()
        ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, num_splits=splits)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(out, want) < 2e-2, splits


@pytest.mark.parametrize("tc", [True, False])                                                   # tcgen05 kernel / mma.sync kernel
@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (14, 2, 64), (4, 2, 128), (4, 1, 64)])   # 64-, 32- and 16-row CTAs
def test_paged_prefill(hq, hkv, d, tc, monkeypatch):
    monkeypatch.setattr(ops, "PREFILL_TC", tc)
    torch.manual_seed(5)
    q_lens = [1, 5, 64, 65, 200, 130, 257, 128]
    past = [0, 11, 0, 64, 37, 512, 2200, 128]          # up to 20 key blocks per tile: every ring slot is reused many times
    ctx = [a + b for a, b in zip(q_lens, past)]
    n = len(ctx)
    pool, table = _make_paged(n, ctx, hkv, d, seed=1)
    t = sum(q_lens)
    q = torch.randn(t, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    ts, tq = ops.prefill_tiles(q_lens)
    tile_seq = torch.tensor(ts, dtype=torch.int32, device=DEV)
    tile_q0 = torch.tensor(tq, dtype=torch.int32, device=DEV)
    out = torch.zeros(t, hq * d, device=DEV, dtype=torch.bfloat16)
    before = ops.launch_counts["paged_prefill_tc"]
    ops.paged_prefill(q, out, pool, table, ctx_t, cu, tile_seq, tile_q0, len(ts), hq, hkv, d)
    torch.cuda.synchronize()
    ops.check_status()
    assert (ops.launch_counts["paged_prefill_tc"] > before) == tc
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d)
    assert _rel_err(out, want) < 2e-2
    for s0, s1 in zip(cu[:-1].tolist(), cu[1:].tolist()):      # every sequence on its own: a short one must not hide in the norm
        assert _rel_err(out[s0:s1], want[s0:s1]) < 3e-2, (s0, s1)
    # sliding window
    out.zero_()
    ops.paged_prefill(q, out, pool, table, ctx_t, cu, tile_seq, tile_q0, len(ts), hq, hkv, d, window=48)
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, window=48)
    assert _rel_err(out, want) < 2e-2


def test_rope_kv_append():
    torch.manual_seed(6)
    hq, hkv, d, t, pages = 14, 2, 64, 37, 9
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (t,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * ref.PAGE, device=DEV)[:t].to(torch.int32)
    slots[3] = -1
    cs = ref.rope_table(512, d, 1e6, DEV)
    pool = torch.zeros(pages, hkv, 2, ref.PAGE, d, device=DEV, dtype=torch.bfloat16)
    qkv_ref, pool_ref = qkv.clone(), pool.clone()
    ref.rope_kv_append(qkv_ref, pos, slots, cs, pool_ref, hq, hkv, d)
    ops.rope_kv_append(qkv, pos, slots, cs, pool, hq, hkv, d)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel_err(qkv, qkv_ref) < 4e-3
    assert _rel_err(pool, pool_ref) < 4e-3


def test_argmax_and_ties():
    torch.manual_seed(7)
    logits = torch.randn(9, 151936, device=DEV).bfloat16()
    logits[0, 777] = 50.0
    logits[0, 12345] = 50.0
    logits[1, 5] = float("nan")
    got = ops.argmax(logits)
    want = ref.argmax(logits)
    assert torch.equal(got.cpu(), want.cpu())
    assert int(got[0]) == 777


def test_sampler_matches_integer_oracle():
    torch.manual_seed(8)
    rows, vocab = 12, 32000
    logits = (torch.randn(rows, vocab, device=DEV) * 3).bfloat16()
    temperature = torch.tensor([0.7, 1.0, 0.0, 0.7, 1.3, 0.7, 0.7, 1.0, 0.5, 0.7, 0.7, 2.0], device=DEV)
    top_k = torch.tensor([0, 50, 0, 1, 0, 40, 0, 0, 5, 0, 1000, 0], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([0.9, 1.0, 1.0, 1.0, 0.5, 0.95, 1.0, 0.1, 0.9, 0.9, 0.8, 1.0], device=DEV)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.05, 0.2, 0.0, 0.0, 0.0, 0.01, 0.0], device=DEV)
    for trial in range(3):
        u = torch.rand(rows, device=DEV)
        got = ops.sample(logits, temperature, top_k, top_p, min_p, u).cpu()
        # the oracle consumes the device's own fixed-point weights semantics: recompute them in torch
        for r in range(rows):
            t = float(temperature[r])
            if t <= 0:
                assert int(got[r]) == int(ref.argmax(logits[r:r + 1])[0])
                continue
            w = ref.sample_weights(logits[r].cpu(), t)
            want = ref.sample_from_weights(w, int(top_k[r]), float(top_p[r]), float(min_p[r]), float(u[r]))
            if int(got[r]) != want:
                # The device computes its weights with __expf, torch with exp: single weights differ in the last
                # place, so the two cumulative sums differ by ~1e-6 of the total.  A different token is accepted
                # only when (a) it survives the *filtered* distribution (weight at or above the oracle's
                # threshold, give or take that rounding) and (b) the draw falls within 1e-4 of the total mass of
                # the token's own interval of the filtered CDF.  A sampler whose top-k / top-p / min-p filter is
                # wrong fails (a); one that draws from the wrong place fails (b).
                g = int(got[r])
                thr = ref.sample_threshold(w, int(top_k[r]), float(top_p[r]), float(min_p[r]))
                assert int(w[g]) >= thr * (1 - 1e-4), ("filtered-out token sampled", r, g, int(w[g]), thr)
                kept = torch.where(w >= thr, w, torch.zeros_like(w))
                target, total = ref.sample_draw_target(kept, float(u[r]))
                csum = torch.cumsum(kept, 0)
                lo = int(csum[g - 1]) if g > 0 else 0
                hi = int(csum[g]) if int(kept[g]) > 0 else lo + int(w[g])
                tol = max(2, int(1e-4 * total))
                assert lo - tol <= target <= hi + tol, ("draw far from the sampled token's interval", r, g, want, lo, target, hi)


def test_sampler_distribution():
    torch.manual_seed(9)
    vocab = 64
    logits = torch.randn(1, vocab, device=DEV).bfloat16().repeat(4096, 1)
    n = logits.shape[0]
    temperature = torch.full((n,), 1.0, device=DEV)
    top_k = torch.zeros(n, dtype=torch.int32, device=DEV)
    top_p = torch.ones(n, device=DEV)
    min_p = torch.zeros(n, device=DEV)
    u = torch.rand(n, device=DEV)
    got = ops.sample(logits, temperature, top_k, top_p, min_p, u)
    freq = torch.bincount(got.long(), minlength=vocab).float() / n
    p = torch.softmax(logits[0].float(), -1)
    assert float((freq - p).abs().max()) < 0.03


def test_spec_verify_greedy():
    torch.manual_seed(10)
    s, k, vocab = 5, 4, 1000
    logits = torch.randn(s * (k + 1), vocab, device=DEV).bfloat16()
    best = ref.argmax(logits).view(s, k + 1)
    draft = best[:, :k].clone()
    draft[1, 2] = (draft[1, 2] + 1) % vocab
    draft[3, 0] = (draft[3, 0] + 1) % vocab
    acc, out = ops.spec_verify_greedy(logits, draft.contiguous(), k)
    acc_r, out_r = ref.spec_verify_greedy(logits, draft, k)
    assert torch.equal(acc.cpu(), acc_r.cpu()) and torch.equal(out.cpu(), out_r.cpu())
    assert acc.cpu().tolist() == [4, 2, 4, 0, 4]


def test_kv_page_utils():
    pool = torch.randn(10, 2, 2, 16, 64, device=DEV).bfloat16()
    orig = pool.clone()
    src = torch.tensor([1, 2], dtype=torch.int64, device=DEV)
    dst = torch.tensor([7, 8], dtype=torch.int64, device=DEV)
    ops.kv_page_copy(pool, src, dst)
    assert torch.equal(pool[7], orig[1]) and torch.equal(pool[8], orig[2])
    staging = torch.zeros(2, 2, 2, 16, 64, device=DEV, dtype=torch.bfloat16)
    ops.kv_gather_pages(pool, staging, src)
    assert torch.equal(staging[0], orig[1])
    pool[1].zero_()
    ops.kv_scatter_pages(pool, staging, src)
    assert torch.equal(pool[1], orig[1])


@pytest.mark.parametrize("m,n,k,sym,fp32_scales", [(1, 896, 896, True, False), (3, 1152, 896, False, True), (8, 896, 4864, True, False),
                                                   (5, 100, 688, False, False), (40, 1152, 896, True, False),
                                                   (16, 1152, 896, False, True), (128, 896, 4864, True, False),
                                                   (1024, 1000, 1760, False, False), (300, 3584, 3584, True, True)])
def test_w4a16_linear(m, n, k, sym, fp32_scales):
    from onnx_genai_b200.ops.quant import QuantLinear

    torch.manual_seed(11)
    w = torch.randn(n, k) * 0.05
    q, s, zp = ref.quantize_w4(w, 32, symmetric=sym)
    if not fp32_scales:
        s = s.bfloat16()
    bias = torch.randn(n) * 0.1
    lin = QuantLinear(q, s, zp, bias, k=k, device=DEV)
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    got = lin(x)
    torch.cuda.synchronize()
    ops.check_status()
    want = x.float().cpu() @ ref.dequant_w4(q, s.float(), zp, 32, k).t() + bias.bfloat16().float()
    assert _rel_err(got.cpu(), want) < 1.2e-2
    assert ops.launch_counts["w4a16_gemv_fused" if m <= 4 else ("w4a16_gemv" if (m <= 8 and n % 32) else "w4a16_gemm")] > 0
    assert lin._scratch is None                        # no bf16 copy of the weights exists


@pytest.mark.parametrize("m,n,k,sym,fp32_scales", [(300, 3584, 3584, True, True), (64, 896, 4864, False, True), (700, 19072, 3584, True, False)])
def test_w4a16_gemm_repeated_runs_agree_bit_for_bit(m, n, k, sym, fp32_scales):
    """Eight launches over the same inputs (one tile per CTA; many k-blocks on few CTAs; several tiles per CTA): every
    result equals the first bit for bit and the fp32 statement to bf16 accuracy -- a slot of the operand ring that is
    read before it is written, or overwritten while it is read, shows up as a run that differs."""
    from onnx_genai_b200.ops.quant import QuantLinear

    torch.manual_seed(11)
    q, s, zp = ref.quantize_w4(torch.randn(n, k) * 0.05, 32, symmetric=sym)
    if not fp32_scales:
        s = s.bfloat16()
    lin = QuantLinear(q, s, zp, None, k=k, device=DEV)
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    want = x.float() @ ref.dequant_w4(q, s.float(), zp, 32, k).to(DEV).t()
    first = lin(x).clone()
    assert float((first.float() - want).abs().max()) < 0.08 + 0.03 * float(want.abs().max())
    for _ in range(7):
        assert torch.equal(lin(x), first)
    torch.cuda.synchronize()
    ops.check_status()


def test_w4a16_gemm_strided_output_matches_the_dense_arm():
    """The int4 tensor-core GEMM writes a column slice of a wider buffer and nothing else, and agrees with the bf16 GEMM
    over a dequantised copy of the same weights (the A/B arm) to bf16 rounding of the weights."""
    from onnx_genai_b200.ops.quant import QuantLinear

    torch.manual_seed(17)
    m, n, k = 200, 640, 1024
    q, s, zp = ref.quantize_w4(torch.randn(n, k) * 0.05, 32, symmetric=False)
    lin = QuantLinear(q, s.bfloat16(), zp, None, k=k, device=DEV)
    x = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    wide = torch.zeros(m, n + 128, device=DEV, dtype=torch.bfloat16)
    lin(x, out=wide[:, 64:64 + n])
    assert float(wide[:, :64].abs().max()) == 0 and float(wide[:, 64 + n:].abs().max()) == 0
    dense = QuantLinear(q, s.bfloat16(), zp, None, k=k, device=DEV)
    dense.large_m = "dense"
    want = dense(x)
    torch.cuda.synchronize()
    ops.check_status()
    assert dense._scratch is not None and dense.device_weight_bytes() > 4 * lin.device_weight_bytes() * 0.9
    assert _rel_err(wide[:, 64:64 + n].float().cpu(), want.float().cpu()) < 4e-3


@pytest.mark.parametrize("m,n,k,sym", [(1, 896, 896, True), (2, 1152, 896, False), (4, 128, 4864, True), (7, 100, 688, False), (8, 64, 9000, True)])
def test_w4a16_fused_prologues_and_residual(m, n, k, sym):
    """RMSNorm prologue, SiLU*up prologue and residual epilogue of the decode-size int4 projection, each against
    the unfused fp32 statement with the same bf16 rounding points (K = 9000 spans three shared-memory chunks)."""
    from onnx_genai_b200.ops.quant import QuantLinear

    torch.manual_seed(13)
    w = torch.randn(n, k) * 0.05
    q, s, zp = ref.quantize_w4(w, 32, symmetric=sym)
    lin = QuantLinear(q, s.bfloat16(), zp, torch.randn(n) * 0.1, k=k, device=DEV)
    wd = ref.dequant_w4(q, s.bfloat16().float(), zp, 32, k)
    bias = lin.bias.float().cpu()
    # RMSNorm prologue
    x = (torch.randn(m, k, device=DEV) * 0.7).bfloat16()
    g = (torch.rand(k, device=DEV) + 0.5).bfloat16()
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    lin.fused(x, out, norm_weight=g, eps=1e-6)
    h, _ = ref.rmsnorm(x.cpu(), g.cpu(), 1e-6)
    assert _rel_err(out.cpu(), h.float() @ wd.t() + bias) < 1.2e-2
    # SiLU(gate) * up prologue + residual epilogue written in place
    gu = (torch.randn(m, 2 * k, device=DEV) * 0.8).bfloat16()
    res = torch.randn(m, n, device=DEV).bfloat16()
    want = ref.silu_mul(gu.cpu()).float() @ wd.t() + bias + res.float().cpu()
    lin.fused(gu, res, silu_mul=True, residual=res)
    assert _rel_err(res.cpu(), want) < 1.2e-2
    # plain + residual into a strided output
    wide = torch.zeros(m, n + 64, device=DEV, dtype=torch.bfloat16)
    r2 = torch.randn(m, n, device=DEV).bfloat16()
    lin.fused(x, wide[:, 32:32 + n], residual=r2)
    assert _rel_err(wide[:, 32:32 + n].cpu(), x.float().cpu() @ wd.t() + bias + r2.float().cpu()) < 1.2e-2
    assert float(wide[:, :32].abs().max()) == 0 and float(wide[:, 32 + n:].abs().max()) == 0
    torch.cuda.synchronize()
    ops.check_status()


@pytest.mark.parametrize("t,e,k,hidden,inter", [(37, 16, 4, 256, 128), (300, 128, 8, 512, 256), (5, 8, 2, 256, 768)])
def test_moe_experts_grouped_gemm(t, e, k, hidden, inter):
    from onnx_genai_b200.ops import moe as moe_ops

    torch.manual_seed(12)
    half = 128
    h = (torch.randn(t, hidden, device=DEV) * 0.5).bfloat16()
    router = torch.randn(t, e, device=DEV).bfloat16()
    gate = (torch.randn(e, inter, hidden, device=DEV) * 0.05).bfloat16()
    up = (torch.randn(e, inter, hidden, device=DEV) * 0.05).bfloat16()
    down = (torch.randn(e, hidden, inter, device=DEV) * 0.05).bfloat16()
    packed = torch.stack([ops.pack_gate_up(gate[i], up[i], half) for i in range(e)]).contiguous()
    x0 = torch.randn(t, hidden, device=DEV).bfloat16()
    ws = moe_ops.MoEWorkspace(t, k, e, hidden, inter, DEV)
    got = moe_ops.moe_experts(h, router, packed, down, ws, x0.clone(), k, True, half)
    torch.cuda.synchronize()
    ops.check_status()
    ids, w = ref.moe_route(router, k, True)
    want = x0.float().clone()
    for tok in range(t):
        for j in range(k):
            ex = int(ids[tok, j])
            a = torch.nn.functional.silu(h[tok].float() @ gate[ex].float().t()) * (h[tok].float() @ up[ex].float().t())
            want[tok] += float(w[tok, j]) * (a.bfloat16().float() @ down[ex].float().t())
    assert _rel_err(got, want) < 2.5e-2
    assert int(ws.meta[1]) == t * k
    # expert-parallel slice: only experts [e/2, e) -> partial sums of the two halves add up to the full result
    lo = moe_ops.moe_experts(h, router, packed[: e // 2].contiguous(), down[: e // 2].contiguous(),
                             moe_ops.MoEWorkspace(t, k, e // 2, hidden, inter, DEV), torch.zeros_like(x0), k, True, half, 0, False)
    hi = moe_ops.moe_experts(h, router, packed[e // 2:].contiguous(), down[e // 2:].contiguous(),
                             moe_ops.MoEWorkspace(t, k, e // 2, hidden, inter, DEV), torch.zeros_like(x0), k, True, half, e // 2, False)
    assert _rel_err(lo.float() + hi.float() + x0.float(), want) < 3e-2


QMAX = {"fp8": 448.0, "int8": 127.0, "e5m2": 57344.0}
POOL_DTYPE = {"fp8": torch.uint8, "int8": torch.int8, "e5m2": torch.float8_e5m2}


def _dequant(pool, scales):
    raw = pool.view(torch.float8_e4m3fn) if pool.dtype == torch.uint8 else pool
    return raw.float() * scales[..., None, None]


def _make_paged_fp8(ctx_lens, hkv, d, seed=0, fmt="fp8"):
    """Random KV quantised to e4m3 (or int8) per (page, head, K|V) with amax scaling; returns pool bytes, scales, table."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    pages_per = [(c + ref.PAGE - 1) // ref.PAGE for c in ctx_lens]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g)
    table = torch.zeros(len(ctx_lens), max(pages_per), dtype=torch.int32)
    o = 0
    for s, n in enumerate(pages_per):
        table[s, :n] = perm[o:o + n].to(torch.int32)
        o += n
    vals = torch.randn(total, hkv, 2, ref.PAGE, d, generator=g) * torch.rand(total, hkv, 2, 1, 1, generator=g) * 2
    scales = vals.abs().amax(dim=(-1, -2)).clamp_min(1e-6) / QMAX[fmt]
    if fmt == "int8":
        q8 = torch.round(vals / scales[..., None, None]).clamp(-127, 127).to(torch.int8)
    elif fmt == "e5m2":
        q8 = (vals / scales[..., None, None]).to(torch.float8_e5m2)
    else:
        q8 = (vals / scales[..., None, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    return q8.to(DEV), scales.float().to(DEV), table.to(DEV)


@pytest.mark.parametrize("fmt", ["fp8", "int8", "e5m2"])
def test_paged_attention_fp8_pages(fmt):
    torch.manual_seed(13)
    hq, hkv, d = 28, 4, 128
    ctx = [1, 16, 17, 63, 64, 65, 300, 1000]
    n = len(ctx)
    pool, scales, table = _make_paged_fp8(ctx, hkv, d, fmt=fmt)
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    q = torch.randn(n, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, kv_scales=scales)
    out = torch.zeros(n, hq * d, device=DEV, dtype=torch.bfloat16)
    for splits in (1, 4):
        out.zero_()
        ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, num_splits=splits, kv_scales=scales)
        torch.cuda.synchronize()
        ops.check_status()
        assert _rel_err(out, want) < 2e-2, splits
    # chunked prefill over the same pages
    q_lens = [1, 7, 17, 40, 64, 65, 130, 200]
    t = sum(q_lens)
    qp = torch.randn(t, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ts, tq = ops.prefill_tiles(q_lens)
    outp = torch.zeros(t, hq * d, device=DEV, dtype=torch.bfloat16)
    ops.paged_prefill(qp, outp, pool, table, ctx_t, cu, torch.tensor(ts, dtype=torch.int32, device=DEV),
                      torch.tensor(tq, dtype=torch.int32, device=DEV), len(ts), hq, hkv, d, kv_scales=scales)
    torch.cuda.synchronize()
    ops.check_status()
    wantp = ref.paged_attention(qp, pool, table, ctx_t, cu, hq, hkv, d, kv_scales=scales)
    assert _rel_err(outp, wantp) < 2e-2


@pytest.mark.parametrize("hq,hkv", [(28, 4), (32, 4), (8, 2), (4, 4)])
def test_decode_over_e4m3_pages_as_mma_operands_is_as_accurate_as_expanding_them(hq, hkv):
    """The kernel that feeds raw e4m3 bytes to e4m3 MMAs (queries and probabilities carried as a hi + lo pair of rows)
    against fp32, and against the kernel that expands pages to bf16: block edges of its 128-key stages, split counts
    that leave splits empty, large query magnitudes, and pages whose V scale is tiny next to the others'."""
    torch.manual_seed(17)
    d = 128
    ctx = [1, 31, 32, 33, 127, 128, 129, 255, 257, 700, 2000]
    n = len(ctx)
    pool, scales, table = _make_paged_fp8(ctx, hkv, d, seed=3)
    scales[::3, :, 1] *= 1e-4                                     # some V pages count for almost nothing
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    q = (torch.randn(n, (hq + 2 * hkv) * d, device=DEV) * torch.tensor([0.05, 1.0, 30.0] * 4, device=DEV)[:n, None]).bfloat16()
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, kv_scales=scales)
    errs = {}
    old = ops.set_e4m3_mma(2)
    try:
        for mma in (2, 1, 0):
            ops.set_e4m3_mma(mma)
            for splits in (1, 3, 8):
                out = torch.full((n, hq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
                ops.paged_decode(q, out, pool, table, ctx_t, hq, hkv, d, num_splits=splits, kv_scales=scales)
                torch.cuda.synchronize()
                ops.check_status()
                assert torch.isfinite(out.float()).all(), (mma, splits)
                errs[mma, splits] = _rel_err(out, want)
                worst = ((out.float() - want.float()).norm(dim=1) / want.float().norm(dim=1).clamp_min(1e-6)).max().item()
                assert worst < 2e-2, (mma, splits, worst)
    finally:
        ops.set_e4m3_mma(old)
    for splits in (1, 3, 8):
        for mma in (2, 1):
            assert errs[mma, splits] < 1e-2 and errs[mma, splits] < 1.5 * errs[0, splits] + 1e-3, errs


@pytest.mark.parametrize("fmt", ["fp8", "int8", "e5m2"])
def test_rope_kv_append_fp8_roundtrip(fmt):
    torch.manual_seed(14)
    qmax = QMAX[fmt]
    hq, hkv, d, pages = 4, 2, 128, 4
    t = pages * ref.PAGE
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    pos = torch.arange(t, dtype=torch.int32, device=DEV)
    slots = torch.arange(t, dtype=torch.int32, device=DEV)       # tokens land in order: offset 0 of each page first
    cs = ref.rope_table(256, d, 1e4, DEV)
    pool = torch.zeros(pages, hkv, 2, ref.PAGE, d, device=DEV, dtype=POOL_DTYPE[fmt])
    scales = torch.zeros(pages, hkv, 2, device=DEV)
    want_qkv = qkv.clone()
    bf_pool = torch.zeros(pages, hkv, 2, ref.PAGE, d, device=DEV, dtype=torch.bfloat16)
    ref.rope_kv_append(want_qkv, pos, slots, cs, bf_pool, hq, hkv, d)
    for s0 in range(0, t, ref.PAGE):          # one launch per position inside a page keeps the "first token sets the scale" order
        for off in range(ref.PAGE):
            i = s0 + off
            ops.rope_kv_append(qkv[i:i + 1], pos[i:i + 1], slots[i:i + 1], cs, pool, hq, hkv, d, kv_scales=scales)
    torch.cuda.synchronize()
    ops.check_status()
    deq = _dequant(pool, scales)
    clipped = (bf_pool.float().abs() > qmax * scales[..., None, None]).float().mean()
    assert float(clipped) < 0.02                                   # 2x headroom over the first token's amax
    err = (deq - bf_pool.float()).abs() / (bf_pool.float().abs() + 0.05 * bf_pool.float().abs().amax())
    assert float(err[(bf_pool.float().abs() <= qmax * scales[..., None, None])].mean()) < 0.05


@pytest.mark.parametrize("fmt", ["fp8", "int8", "e5m2"])
def test_rope_kv_append_fp8_one_launch_equals_token_by_token(fmt):
    """A prefill chunk appends many tokens of a page in one launch; the stored bytes and scales must be exactly those
    of appending the tokens one launch at a time (every token of a page uses the scale of the page's first token),
    also when the pages held another sequence's scales before, and when a later chunk continues a page."""
    torch.manual_seed(15)
    hq, hkv, d, pages = 4, 2, 128, 5
    t = pages * ref.PAGE - 5                                        # the last page stays partly empty
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, device=DEV) * torch.linspace(0.2, 3.0, t, device=DEV)[:, None]).bfloat16()
    pos = torch.arange(t, dtype=torch.int32, device=DEV)
    slots = torch.arange(t, dtype=torch.int32, device=DEV)
    cs = ref.rope_table(256, d, 1e4, DEV)

    def fresh():
        pool = torch.zeros(pages, hkv, 2, ref.PAGE, d, device=DEV, dtype=POOL_DTYPE[fmt])
        scales = torch.full((pages, hkv, 2), 123.0, device=DEV)      # stale scales of a previous owner
        return pool, scales

    pool_a, scales_a = fresh()
    for i in range(t):
        ops.rope_kv_append(qkv[i:i + 1].clone(), pos[i:i + 1], slots[i:i + 1], cs, pool_a, hq, hkv, d, kv_scales=scales_a)
    pool_b, scales_b = fresh()
    ops.rope_kv_append(qkv.clone(), pos, slots, cs, pool_b, hq, hkv, d, kv_scales=scales_b)
    pool_c, scales_c = fresh()                                      # two chunks; the second starts in the middle of a page
    cut = 2 * ref.PAGE + 7
    ops.rope_kv_append(qkv[:cut].clone(), pos[:cut], slots[:cut], cs, pool_c, hq, hkv, d, kv_scales=scales_c)
    ops.rope_kv_append(qkv[cut:].clone(), pos[cut:], slots[cut:], cs, pool_c, hq, hkv, d, kv_scales=scales_c)
    torch.cuda.synchronize()
    ops.check_status()
    for pool, scales in ((pool_b, scales_b), (pool_c, scales_c)):
        assert torch.equal(scales, scales_a)
        assert torch.equal(pool, pool_a)


@pytest.mark.parametrize("fmt", ["fp8", "int8", "e5m2"])
def test_fp8_append_kernel_matches_the_cpu_codec_byte_for_byte(fmt):
    """The device one-byte append (rotation launch + codec launch) against the CPU statement of the same codec."""
    torch.manual_seed(16)
    hq, hkv, d, pages = 4, 2, 128, 3
    t = pages * ref.PAGE - 3
    qkv = (torch.randn(t, (hq + 2 * hkv) * d) * torch.linspace(0.3, 2.5, t)[:, None]).bfloat16()
    pos = torch.arange(t, dtype=torch.int32)
    slots = torch.arange(t, dtype=torch.int32)
    cs = ref.rope_table(128, d, 1e4)
    pool_c = torch.zeros(pages, hkv, 2, ref.PAGE, d, dtype=POOL_DTYPE[fmt])
    sc_c = torch.zeros(pages, hkv, 2)
    q_c = qkv.clone()
    ref.rope_kv_append(q_c, pos, slots, cs, pool_c, hq, hkv, d, kv_scales=sc_c)
    pool_g = torch.zeros(pages, hkv, 2, ref.PAGE, d, dtype=POOL_DTYPE[fmt], device=DEV)
    sc_g = torch.zeros(pages, hkv, 2, device=DEV)
    q_g = qkv.to(DEV)
    ops.rope_kv_append(q_g, pos.to(DEV), slots.to(DEV), cs.to(DEV), pool_g, hq, hkv, d, kv_scales=sc_g)
    torch.cuda.synchronize()
    ops.check_status()
    # the rotation runs in fp32 on both sides and rounds to bf16: identical inputs for the codec up to rare 1-ulp ties
    same_rot = (q_g.cpu() == q_c).float().mean()
    assert float(same_rot) > 0.999
    assert torch.allclose(sc_g.cpu(), sc_c, rtol=1e-2)
    as_bytes = lambda x: x.view(torch.uint8) if x.dtype == torch.float8_e5m2 else x
    mismatch = (as_bytes(pool_g.cpu()) != as_bytes(pool_c)).float()
    assert float(mismatch.mean()) < 0.01                            # bytes differ only where the rotated input differed by an ulp


def test_vmm_growable_buffer_keeps_its_address_and_contents():
    from onnx_genai_b200.utils import vmm

    assert vmm.available(0)
    buf = vmm.GrowableBuffer(64 << 20, 0)
    assert buf.mapped == 0 and buf.reserved >= 64 << 20 and buf.granularity >= 1 << 16
    base = buf.ptr
    buf.grow(3 << 20)
    first = buf.mapped
    assert first >= 3 << 20 and first % buf.granularity == 0 and buf.chunks == 1
    a = buf.view(torch.int32)
    a.copy_(torch.arange(a.numel(), dtype=torch.int32, device=DEV))
    buf.grow(2 << 20)                                       # already covered: nothing happens
    assert buf.mapped == first and buf.chunks == 1
    buf.grow(first + (5 << 20))
    assert buf.ptr == base and buf.mapped > first and buf.chunks == 2
    whole = buf.view(torch.int32)
    assert whole.data_ptr() == a.data_ptr() == base
    whole[a.numel():].fill_(-7)
    torch.cuda.synchronize()
    assert torch.equal(whole[: a.numel()].cpu(), torch.arange(a.numel(), dtype=torch.int32))
    assert int(whole[-1]) == -7
    tail = buf.view(torch.float32, (4, 8), offset_bytes=first)
    assert tail.data_ptr() == base + first
    with pytest.raises(vmm.VmmError, match="exceeds"):
        buf.view(torch.uint8, (buf.mapped + 1,))
    with pytest.raises(vmm.VmmError, match="address space was reserved"):
        buf.grow(buf.reserved + 1)
    del whole, tail
    assert buf.shrink(first) == first and buf.chunks == 1   # the second chunk goes back to the device
    assert torch.equal(buf.view(torch.int32).cpu(), torch.arange(a.numel(), dtype=torch.int32))
    free_before = torch.cuda.mem_get_info()[0]
    buf.grow(48 << 20)
    assert torch.cuda.mem_get_info()[0] <= free_before - (buf.mapped - first) + (1 << 20)
    del a
    buf.close()
    assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)


def _punch_holes(table, ctx, q_lens, window, sink):
    """What the scheduler does under a sliding window: entries of pages wholly between the sinks and the window of the
    sequence's first query row become -1."""
    table = table.clone()
    for s, (c, ql) in enumerate(zip(ctx, q_lens)):
        lo, hi = (sink + 15) // 16, max(0, c - ql - window + 1) // 16
        if hi > lo:
            table[s, lo:hi] = -1
    return table


@pytest.mark.parametrize("window,sink", [(100, 0), (100, 16), (300, 32), (64, 48)])
@pytest.mark.parametrize("pages", ["bf16", "fp8", "int8"])
def test_sliding_window_with_attention_sinks(pages, window, sink):
    """Decode (with and without KV splits) and chunked prefill under window + sinks, with the invisible pages taken out of
    the page table, against the fp32 reference on the same pages."""
    torch.manual_seed(21)
    hq, hkv, d = 28, 4, 128
    ctx = [1, 17, 90, 129, 257, 700, 1500]
    n = len(ctx)
    if pages == "bf16":
        pool, table = _make_paged(n, ctx, hkv, d)
        scales = None
    else:
        pool, scales, table = _make_paged_fp8(ctx, hkv, d, seed=5, fmt=pages)
    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=DEV)
    q = torch.randn(n, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    cu = torch.arange(n + 1, dtype=torch.int32, device=DEV)
    holes = _punch_holes(table, ctx, [1] * n, window, sink)
    assert bool((holes < 0).any())
    want = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, window=window, kv_scales=scales, sink=sink)
    full = ref.paged_attention(q, pool, table, ctx_t, cu, hq, hkv, d, kv_scales=scales)
    assert _rel_err(want, full) > 0.05                      # the mask matters on this data
    modes = (2, 1, 0) if pages == "fp8" else (None,)
    old = ops.set_e4m3_mma(2)
    try:
        for mode in modes:
            if mode is not None:
                ops.set_e4m3_mma(mode)
            for splits in (1, 4):
                out = torch.full((n, hq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
                ops.paged_decode(q, out, pool, holes, ctx_t, hq, hkv, d, num_splits=splits, window=window, kv_scales=scales, sink=sink)
                torch.cuda.synchronize()
                ops.check_status()
                assert torch.isfinite(out.float()).all() and _rel_err(out, want) < 2e-2, (mode, splits, _rel_err(out, want))
    finally:
        ops.set_e4m3_mma(old)
    q_lens = [1, 7, 40, 64, 65, 130, 200]
    t = sum(q_lens)
    qp = torch.randn(t, (hq + 2 * hkv) * d, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ts, tq = ops.prefill_tiles(q_lens)
    holes = _punch_holes(table, ctx, q_lens, window, sink)
    wantp = ref.paged_attention(qp, pool, table, ctx_t, cu, hq, hkv, d, window=window, kv_scales=scales, sink=sink)
    outp = torch.full((t, hq * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.paged_prefill(qp, outp, pool, holes, ctx_t, cu, torch.tensor(ts, dtype=torch.int32, device=DEV),
                      torch.tensor(tq, dtype=torch.int32, device=DEV), len(ts), hq, hkv, d, window=window, kv_scales=scales, sink=sink)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.isfinite(outp.float()).all() and _rel_err(outp, wantp) < 2e-2, _rel_err(outp, wantp)
