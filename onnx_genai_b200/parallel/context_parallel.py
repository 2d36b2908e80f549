"""Context parallelism: one long sequence's attention split over ranks along the sequence axis.

Each rank keeps a slice of the sequence -- its query rows and the K / V rows of the same tokens -- and the K / V slices
travel once around a ring.  At every hop a rank attends its queries over the slice it currently holds and folds the
result into a running (output, log-sum-exp) pair, so after ``world - 1`` hops every query has seen every key it may see
and no rank ever held more than two slices.  Causal masking works on absolute token positions, which lets the slices be
any partition of the sequence; :func:`zigzag_slices` is the partition that balances causal work (rank r takes chunk r and
chunk 2·world − 1 − r, so every rank owns one early and one late chunk).

Blocking ``send`` / ``recv`` of the communicator carry the ring: even ranks send first and then receive, odd ranks the
other way round, which cannot deadlock on a ring of any length.

(The reference has no sequence or context parallelism: docs/execution/NATIVE_CUDA_DECODE.md:103-105 lists it as out of
scope.  This is net-new, for prompts whose prefill one GPU should not do alone.  The merge below is the same log-sum-exp
combination the split-KV decode kernel of this package uses across KV partitions.)
"""
from __future__ import annotations

import math

import torch


def contiguous_slices(total: int, world: int) -> list[torch.Tensor]:
    """Token positions of each rank when the sequence is cut into ``world`` near-equal contiguous runs."""
    base, extra = divmod(total, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append(torch.arange(start, start + n))
        start += n
    return out


def zigzag_slices(total: int, world: int) -> list[torch.Tensor]:
    """Token positions of each rank under the zigzag partition: the sequence is cut into 2·world chunks and rank r owns
    chunks r and 2·world − 1 − r.  Under a causal mask the number of (query, key) pairs a rank computes is then the same
    on every rank to within one chunk's rounding, where contiguous runs give the last rank about twice the mean."""
    chunks = contiguous_slices(total, 2 * world)
    return [torch.cat([chunks[r], chunks[2 * world - 1 - r]]) for r in range(world)]


def causal_pairs(slices: list[torch.Tensor]) -> list[int]:
    """(query, key) pairs each rank computes under a causal mask -- the load a partition gives each rank."""
    everything = torch.cat(slices)
    return [int((everything[None, :] <= s[:, None]).sum()) for s in slices]


def block_attention(q, k, v, q_pos, k_pos, scale: float, causal: bool = True, window: int = 0):
    """Attention of ``q`` [B, Hq, Tq, D] over one K / V block [B, Hkv, Tk, D] (grouped heads: Hq a multiple of Hkv),
    masked on absolute positions.  Returns the block-normalised output [B, Hq, Tq, D] (fp32) and the log-sum-exp of the
    scores [B, Hq, Tq] (fp32; −inf where a query sees no key of the block, with a zero output row)."""
    b, hq, tq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    qf = q.float().view(b, hkv, g, tq, d)
    s = torch.einsum("bhgqd,bhkd->bhgqk", qf, k.float()) * scale
    if causal or window > 0:
        allowed = torch.ones(tq, k.shape[2], dtype=torch.bool, device=q.device)
        if causal:
            allowed &= k_pos[None, :] <= q_pos[:, None]
        if window > 0:
            allowed &= k_pos[None, :] > q_pos[:, None] - window
        s = s.masked_fill(~allowed, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    out = torch.einsum("bhgqk,bhkd->bhgqd", p, v.float())
    return out.reshape(b, hq, tq, d), lse.reshape(b, hq, tq)


def merge_partials(out_a, lse_a, out_b, lse_b):
    """Fold two normalised partial attentions over disjoint key sets into the attention over their union."""
    lse = torch.logaddexp(lse_a, lse_b)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    wa = torch.where(torch.isinf(lse_a), torch.zeros_like(lse_a), torch.exp(lse_a - safe))
    wb = torch.where(torch.isinf(lse_b), torch.zeros_like(lse_b), torch.exp(lse_b - safe))
    return out_a * wa[..., None] + out_b * wb[..., None], lse


def _ring_step(comm, rank: int, world: int, send_buf: torch.Tensor, recv_buf: torch.Tensor) -> None:
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    if rank % 2 == 0:
        comm.send(send_buf, nxt)
        comm.recv(recv_buf, prv)
    else:
        comm.recv(recv_buf, prv)
        comm.send(send_buf, nxt)


def ring_attention(q, k, v, positions, comm, rank: int, world: int, slice_sizes: list[int], all_positions=None,
                   scale: float | None = None, causal: bool = True, window: int = 0):
    """Attention of this rank's queries over the whole sequence.

    ``q`` [B, Hq, T_r, D], ``k`` / ``v`` [B, Hkv, T_r, D] and ``positions`` [T_r] are this rank's slice; ``slice_sizes``
    gives every rank's T (slices may differ in length) and ``all_positions`` every rank's positions (default: contiguous
    runs in rank order).  Returns [B, Hq, T_r, D] in ``q``'s dtype and the fp32 log-sum-exp [B, Hq, T_r].

    Under a causal mask with contiguous slices, a block that lies wholly in this rank's future is skipped without any
    arithmetic (it still travels on, since later ranks need it)."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if all_positions is None:
        all_positions, start = [], 0
        for n in slice_sizes:
            all_positions.append(torch.arange(start, start + n))
            start += n
    pos = positions.to(q.device)
    out, lse = block_attention(q, k, v, pos, pos, scale, causal, window)
    if world == 1:
        return out.to(q.dtype), lse
    b, hkv = k.shape[0], k.shape[1]
    cap = max(slice_sizes)

    def packed(kk, vv):
        buf = torch.zeros(2, b, hkv, cap, d, dtype=k.dtype, device=k.device)
        buf[0, :, :, : kk.shape[2]] = kk
        buf[1, :, :, : vv.shape[2]] = vv
        return buf

    held, held_owner = packed(k, v), rank
    q_lo, q_hi = int(pos.min()), int(pos.max())
    for _ in range(world - 1):
        incoming = torch.empty_like(held)
        _ring_step(comm, rank, world, held, incoming)
        held, held_owner = incoming, (held_owner - 1) % world
        n = slice_sizes[held_owner]
        if n == 0:
            continue
        kpos = all_positions[held_owner].to(q.device)
        if causal and int(kpos.min()) > q_hi:
            continue                                        # wholly in the future of every query here
        if window > 0 and int(kpos.max()) <= q_lo - window:
            continue                                        # wholly behind every query's window
        o2, l2 = block_attention(q, held[0, :, :, :n], held[1, :, :, :n], pos, kpos, scale, causal, window)
        out, lse = merge_partials(out, lse, o2, l2)
    return out.to(q.dtype), lse


def ring_bytes_per_rank(batch: int, kv_heads: int, head_dim: int, slice_len: int, world: int, elem_bytes: int = 2) -> int:
    """Bytes one rank sends around the ring for one attention layer: its K and V slice, ``world − 1`` times."""
    return 2 * batch * kv_heads * slice_len * head_dim * elem_bytes * (world - 1)


def context_parallel_prefill(cfg, weights, token_ids, comm, rank: int, world: int, partition: str = "zigzag"):
    """Prefill of one prompt with its tokens split over ``world`` ranks (weights replicated, dense layers).

    Every token-wise part of the layer (norms, projections, MLP) runs on this rank's tokens only; attention is the ring
    above.  Returns ``(positions, hidden, kv)``: this rank's token positions, their final-norm hidden rows [T_r, H], and
    per layer the roped K and V rows [T_r, Hkv, D] of those tokens -- what a KV cache stores for them, so decode can
    continue on any layout once the rows are written to their pages.  The rank holding the last position computes the
    first token's logits with ``weights.lm_head``.

    The arithmetic is the plain fp32-accumulating statement of each operator (``ops/reference.py``): this is the
    sequence-split schedule, checked on CPU ranks; the fused kernels of the single-GPU path are not driven from here."""
    from ..ops import reference as ref

    total = len(token_ids)
    slices = zigzag_slices(total, world) if partition == "zigzag" else contiguous_slices(total, world)
    mine = slices[rank]
    sizes = [len(s) for s in slices]
    hq, hkv, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    rotary = cfg.rotary_dim or d
    table = ref.rope_table(max(total, 1), rotary, cfg.rope_theta)
    ids = torch.as_tensor(token_ids, dtype=torch.long)[mine]
    x = weights.embed[ids]
    delta, kv = None, []
    for lw in weights.layers:
        h, x = ref.rmsnorm(x, lw.ln1, cfg.rms_eps, delta)
        qkv = ref.gemm(h, lw.qkv_w, lw.qkv_b)
        q = ref.apply_rope(qkv[:, : hq * d].reshape(-1, hq, d), mine, table, rotary, cfg.rotary_interleaved)
        k = ref.apply_rope(qkv[:, hq * d: (hq + hkv) * d].reshape(-1, hkv, d), mine, table, rotary, cfg.rotary_interleaved)
        v = qkv[:, (hq + hkv) * d:].reshape(-1, hkv, d)
        kv.append((k, v))
        att, _ = ring_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], mine, comm, rank, world,
                                sizes, all_positions=slices, causal=True, window=cfg.sliding_window)
        att = att[0].transpose(0, 1).reshape(-1, hq * d)
        o = ref.gemm(att, lw.o_w)
        h, x = ref.rmsnorm(x, lw.ln2, cfg.rms_eps, o)
        act = ref.swiglu_packed(h, lw.gate_up_w, weights.swiglu_half)
        delta = ref.gemm(act, lw.down_w)
    hidden, _ = ref.rmsnorm(x, weights.final_norm, cfg.rms_eps, delta)
    return mine, hidden, kv
