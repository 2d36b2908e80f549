"""Plain PyTorch fp32 statements of every fused op.

These are the numerics oracle for the CUDA kernels (tests compare each kernel against the
function of the same name here) and the execution path for CPU tensors.  Conventions follow the
reference's CPU kernels: RMSNorm with fp32 statistics, half-rotation or interleaved rotary
(crates/onnx-runtime-ep-cuda/src/kernels/rotary_embedding.rs:45), GQA causal softmax
(crates/onnx-runtime-ep-cpu/src/kernels/group_query_attention.rs), MatMulNBits dequantisation
``(code - zp) * scale`` with the low nibble holding the even k
(crates/onnx-runtime-ep-cpu/src/kernels/matmul_nbits.rs:1-17), sampler order temperature ->
top-k -> top-p -> min-p (crates/onnx-genai-engine/src/processors.rs:18-215) and argmax ties to
the lowest token id (crates/onnx-genai-engine/src/sampling.rs:120-132).
"""
from __future__ import annotations

import math

import torch

PAGE = 16


def gemm(a, w, bias=None, residual=None, epilogue="none", out_dtype=None):
    """a [M,K] @ w[N,K]^T with fp32 accumulation.  ``swiglu``: w rows are tile-interleaved gate|up."""
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if epilogue == "residual":
        y = y + residual.float()
    out_dtype = out_dtype or a.dtype
    return y.to(out_dtype)


def swiglu_packed(a, w_packed, half, out_dtype=None):
    """SwiGLU over a weight packed by :func:`pack_gate_up` with tile half-width ``half``."""
    y = a.float() @ w_packed.float().t()
    m, n = y.shape
    y = y.view(m, n // (2 * half), 2, half)
    g, u = y[:, :, 0, :], y[:, :, 1, :]
    return (torch.nn.functional.silu(g) * u).reshape(m, n // 2).to(out_dtype or a.dtype)


def pack_gate_up(gate_w, up_w, half):
    """Interleave gate and up projection rows in blocks of ``half`` so one GEMM tile of width
    ``2*half`` holds matching gate and up columns: [g0..g(half-1), u0..u(half-1), g(half).. ...]."""
    inter, k = gate_w.shape
    assert inter % half == 0, (inter, half)
    g = gate_w.view(inter // half, 1, half, k)
    u = up_w.view(inter // half, 1, half, k)
    return torch.cat([g, u], dim=1).reshape(2 * inter, k).contiguous()


def rmsnorm(x, weight, eps, delta=None):
    """Returns (normed, new_residual).  With ``delta`` the residual is x + delta, rounded to x.dtype first."""
    if delta is not None:
        x = (x.float() + delta.float()).to(x.dtype)
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype), x


def silu_mul(gate_up):
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter].float(), gate_up[..., inter:].float()
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def rope_table(max_pos, rotary_dim, theta, device="cpu"):
    """[max_pos, rotary_dim/2, 2] fp32 (cos, sin), computed in float64 then rounded."""
    half = rotary_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rotary_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).float().to(device)


def apply_rope(x, positions, cos_sin, rotary_dim, interleaved=False):
    """x [T, H, D] -> rotated copy (fp32 math, result in x.dtype)."""
    t, h, d = x.shape
    half = rotary_dim // 2
    cs = cos_sin[positions.long()]  # [T, half, 2]
    c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
    xf = x.float().clone()
    if interleaved:
        x0, x1 = xf[..., 0:rotary_dim:2], xf[..., 1:rotary_dim:2]
        r0, r1 = x0 * c - x1 * s, x1 * c + x0 * s
        xf[..., 0:rotary_dim:2], xf[..., 1:rotary_dim:2] = r0, r1
    else:
        x0, x1 = xf[..., :half], xf[..., half:rotary_dim]
        r0, r1 = x0 * c - x1 * s, x1 * c + x0 * s
        xf[..., :half], xf[..., half:rotary_dim] = r0, r1
    return xf.to(x.dtype)


def e4m3_bytes(x):
    """fp32 -> e4m3 bytes with saturation at +-448 (round to nearest even), as the device conversion does."""
    return x.float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def e5m2_bytes(x):
    """fp32 -> e5m2 with saturation at +-57344 (round to nearest even)."""
    return x.float().clamp(-57344.0, 57344.0).to(torch.float8_e5m2)


def int8_bytes(x):
    """fp32 -> symmetric int8 with saturation at +-127 (round to nearest even)."""
    return torch.round(x.float().clamp(-127.0, 127.0)).to(torch.int8)


def kv_append_fp8(qkv, slots, pool, scales, hq, hkv, d):
    """One-byte page codec (e4m3 in a uint8 pool, symmetric int8 in an int8 pool): one scale per (page, head, K|V),
    fixed by the page's first token at amax * 2 / qmax, qmax = 448 or 127 (headroom
    for the 15 tokens that follow, which saturate to it).  Tokens are taken in row order, so a chunk that starts a
    page and continues it in the same call behaves like one append per token.  pool [P,hkv,2,PAGE,d] uint8,
    scales [P,hkv,2] fp32; qkv already rotated."""
    t = qkv.shape[0]
    v = qkv.view(t, hq + 2 * hkv, d).float()
    qmax, encode = (127.0, int8_bytes) if pool.dtype == torch.int8 else ((57344.0, e5m2_bytes) if pool.dtype == torch.float8_e5m2 else (448.0, e4m3_bytes))
    for i in range(t):
        slot = int(slots[i])
        if slot < 0:
            continue
        page, off = slot // PAGE, slot % PAGE
        for kv in range(2):
            for h in range(hkv):
                vec = v[i, hq + kv * hkv + h]
                if off == 0 or not float(scales[page, h, kv]) > 0.0:
                    scales[page, h, kv] = max(float(vec.abs().max()) * 2.0, 1e-6) / qmax
                inv = torch.tensor(1.0, dtype=torch.float32) / scales[page, h, kv].float()
                pool[page, h, kv, off] = encode(vec * inv)


def rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim=None, interleaved=False, kv_scales=None):
    """In place: rotate q,k inside qkv [T,(hq+2hkv)*d]; write k,v to pool [P,hkv,2,PAGE,d] at slots
    (e4m3 bytes with per-(page, head) scales when ``kv_scales`` is given)."""
    rotary_dim = rotary_dim or d
    t = qkv.shape[0]
    v = qkv.view(t, hq + 2 * hkv, d)
    v[:, : hq + hkv] = apply_rope(v[:, : hq + hkv], positions, cos_sin, rotary_dim, interleaved)
    if kv_scales is not None:
        kv_append_fp8(qkv, slots, pool, kv_scales, hq, hkv, d)
        return qkv
    ok = slots >= 0
    page, off = (slots // PAGE).long(), (slots % PAGE).long()
    k, vv = v[:, hq : hq + hkv], v[:, hq + hkv :]
    pool[page[ok], :, 0, off[ok]] = k[ok].to(pool.dtype)
    pool[page[ok], :, 1, off[ok]] = vv[ok].to(pool.dtype)
    return qkv


def _live_pages(table, n_pages):
    """Page ids of a sequence; entries of released pages (-1: between the attention sinks and the sliding window, never
    visible to a query) are replaced by a live page so that the gather stays in range -- their keys are masked."""
    idx = table[:n_pages].long()
    if bool((idx < 0).any()):
        idx = torch.where(idx < 0, idx[idx >= 0][-1], idx)
    return idx


def _gather_kv(pool, table, ctx):
    n_pages = (ctx + PAGE - 1) // PAGE
    pages = pool[_live_pages(table, n_pages)]  # [n, hkv, 2, PAGE, d]
    k = pages[:, :, 0].permute(1, 0, 2, 3).reshape(pool.shape[1], -1, pool.shape[-1])[:, :ctx]
    v = pages[:, :, 1].permute(1, 0, 2, 3).reshape(pool.shape[1], -1, pool.shape[-1])[:, :ctx]
    return k.float(), v.float()


def paged_attention(q, pool, page_table, ctx_len, cu_q, hq, hkv, d, scale=None, window=0, kv_scales=None, sink=0):
    """Varlen causal GQA over paged KV.  q [T, >=hq*d] (first hq*d columns used); returns [T, hq*d].

    Sequence s owns query rows cu_q[s]:cu_q[s+1]; its last row sits at position ctx_len[s]-1.
    ``kv_scales`` [P,hkv,2] dequantises fp8 pages.  ``window`` > 0 keeps the last ``window`` keys of each query and,
    with ``sink`` > 0, the first ``sink`` keys of the sequence as well (attention sinks).
    """
    scale = scale or 1.0 / math.sqrt(d)
    t = q.shape[0]
    out = torch.zeros(t, hq * d, dtype=q.dtype, device=q.device)
    g = hq // hkv
    for s in range(len(ctx_len)):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        ctx = int(ctx_len[s])
        if e <= b or ctx <= 0:
            continue
        if kv_scales is not None:
            n_pages = (ctx + PAGE - 1) // PAGE
            idx = _live_pages(page_table[s], n_pages)
            raw = pool[idx]
            if raw.dtype == torch.uint8:   # e4m3 bytes
                raw = raw.view(torch.float8_e4m3fn)
            pages = raw.float() * kv_scales[idx][:, :, :, None, None]
            k = pages[:, :, 0].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
            v = pages[:, :, 1].permute(1, 0, 2, 3).reshape(hkv, -1, d)[:, :ctx]
        else:
            k, v = _gather_kv(pool, page_table[s], ctx)
        qs = q[b:e, : hq * d].float().view(e - b, hkv, g, d)
        scores = torch.einsum("thgd,hkd->thgk", qs, k) * scale
        qpos = torch.arange(ctx - (e - b), ctx, device=q.device)[:, None]
        kpos = torch.arange(ctx, device=q.device)[None, :]
        mask = kpos <= qpos
        if window > 0:
            mask &= (kpos > qpos - window) | (kpos < sink)
        scores = scores.masked_fill(~mask[:, None, None, :], float("-inf"))
        p = torch.softmax(scores, dim=-1)
        o = torch.einsum("thgk,hkd->thgd", p, v)
        out[b:e] = o.reshape(e - b, hq * d).to(q.dtype)
    return out


def argmax(logits):
    """Lowest index wins ties; NaN never wins."""
    l = logits.float()
    l = torch.where(torch.isnan(l), torch.full_like(l, float("-inf")), l)
    mx = l.max(dim=-1, keepdim=True).values
    idx = torch.arange(l.shape[-1], device=l.device).expand_as(l)
    cand = torch.where(l == mx, idx, torch.full_like(idx, l.shape[-1]))
    return cand.min(dim=-1).values.to(torch.int32)


def sample_weights(logits_row, temperature):
    """Fixed-point weights w = min(round(exp((l - max)/T) * 2^30), 2^30 - 1) as int64 (the device sampler's mass unit)."""
    l = logits_row.float()
    e = torch.exp((l - l.max()) / temperature)
    e = torch.where(torch.isnan(e), torch.zeros_like(e), e)
    return torch.floor(e.double() * 1073741824.0 + 0.5).clamp_max(1073741823.0).to(torch.int64)


def sample_threshold(w, top_k, top_p, min_p):
    """Weight threshold that top-k, then top-p, then min-p leave: a token survives iff its weight is >= the result."""
    vocab = w.numel()
    thr = 1
    total = int(w.sum())
    if 0 < top_k < vocab:
        kth = int(torch.sort(w, descending=True).values[top_k - 1])
        thr = max(thr, kth)
        total = int(w[w >= thr].sum())
    if 0.0 < top_p < 1.0:
        target = max(1, int(float(total) * float(top_p)))
        vals = torch.sort(w[w >= thr], descending=True).values
        csum = torch.cumsum(vals, 0)
        pos = int(torch.searchsorted(csum, torch.tensor(target, dtype=csum.dtype), right=False))
        pos = min(pos, vals.numel() - 1)
        thr = max(thr, int(vals[pos]))
    if min_p > 0.0:
        thr = max(thr, int(torch.tensor(min(min_p, 1.0), dtype=torch.float32) * 1073741824.0))
    return thr


def sample_draw_target(kept, u):
    """(target mass, total mass) of the draw ``u`` over the surviving weights ``kept``."""
    final_total = int(kept.sum())
    uu = min(max(float(torch.tensor(u, dtype=torch.float32)), 0.0), 0.99999994)
    return min(int(uu * float(final_total)), final_total - 1), final_total


def sample_from_weights(w, top_k, top_p, min_p, u):
    """Exact integer statement of the sampler: thresholds keep ties; draw walks tokens in index order."""
    thr = sample_threshold(w, top_k, top_p, min_p)
    kept = torch.where(w >= thr, w, torch.zeros_like(w))
    if int(kept.sum()) == 0:
        return int(torch.argmax(w))
    target, _ = sample_draw_target(kept, u)
    csum = torch.cumsum(kept, 0)
    return int(torch.searchsorted(csum, torch.tensor(target, dtype=csum.dtype), right=True))


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    rows = logits.shape[0]
    out = torch.zeros(rows, dtype=torch.int32)
    for r in range(rows):
        t = float(temperature[r])
        if not t > 0.0:
            out[r] = int(argmax(logits[r : r + 1])[0])
            continue
        w = sample_weights(logits[r].cpu(), t)
        out[r] = sample_from_weights(w, int(top_k[r]), float(top_p[r]), float(min_p[r]), float(uniform[r]))
    return out.to(logits.device)


def spec_verify_greedy(logits, draft, k):
    """logits [S*(k+1), V]; draft [S, k] -> (accept_len [S], out_tokens [S, k+1] padded with -1)."""
    s = draft.shape[0]
    best = argmax(logits).view(s, k + 1)
    accept = torch.zeros(s, dtype=torch.int32)
    out = torch.full((s, k + 1), -1, dtype=torch.int32)
    for i in range(s):
        a = 0
        while a < k and int(draft[i, a]) == int(best[i, a]):
            a += 1
        accept[i] = a
        out[i, :a] = draft[i, :a].to(torch.int32)
        out[i, a] = best[i, a]
    return accept.to(logits.device), out.to(logits.device)


def dequant_w4(qweight, scales, zero_points=None, block=32, k=None):
    """MatMulNBits int4: qweight [N, ceil(K/block), block/2] uint8, scales [N, ceil(K/block)] -> W [N, K] fp32."""
    n, kb, _ = qweight.shape
    lo = (qweight & 0xF).to(torch.int16)
    hi = (qweight >> 4).to(torch.int16)
    codes = torch.stack([lo, hi], dim=-1).reshape(n, kb, block).float()
    if zero_points is None:
        zp = torch.full((n, kb), 8.0, device=qweight.device)
    else:
        zlo = (zero_points & 0xF).to(torch.int16)
        zhi = (zero_points >> 4).to(torch.int16)
        zp = torch.stack([zlo, zhi], dim=-1).reshape(n, -1)[:, :kb].float()
    w = ((codes - zp[:, :, None]) * scales.float()[:, :, None]).reshape(n, kb * block)
    return w[:, :k].contiguous() if k is not None and k < kb * block else w


def quantize_w4(w, block=32, symmetric=True):
    """Block-wise int4 quantisation producing the MatMulNBits layout (used by exporters and tests)."""
    n, k = w.shape
    if k % block:  # MatMulNBits pads the last K block with zeros
        w = torch.cat([w.float(), torch.zeros(n, block - k % block)], 1)
        k = w.shape[1]
    wb = w.float().view(n, k // block, block)
    if symmetric:
        amax = wb.abs().amax(-1).clamp_min(1e-8)
        scales = amax / 7.0
        codes = torch.clamp(torch.round(wb / scales[:, :, None]) + 8, 0, 15).to(torch.uint8)
        zp = None
    else:
        mn, mx = wb.amin(-1), wb.amax(-1)
        scales = ((mx - mn) / 15.0).clamp_min(1e-8)
        zpv = torch.clamp(torch.round(-mn / scales), 0, 15)
        codes = torch.clamp(torch.round(wb / scales[:, :, None]) + zpv[:, :, None], 0, 15).to(torch.uint8)
        kb = k // block
        zpi = zpv.to(torch.uint8)
        if kb % 2:
            zpi = torch.cat([zpi, torch.zeros(n, 1, dtype=torch.uint8)], dim=1)
        zp = (zpi[:, 0::2] | (zpi[:, 1::2] << 4)).contiguous()
    q = (codes[:, :, 0::2] | (codes[:, :, 1::2] << 4)).contiguous()
    return q, scales, zp


def moe_route(router_logits, k, renormalize=True):
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, ids = torch.topk(probs, k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), w
