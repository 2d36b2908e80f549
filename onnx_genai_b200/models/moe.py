"""MoE feed-forward block of the decoder executor (Qwen3-MoE style: softmax router, top-k, renormalised).

Expert parallelism here rides on the tensor-parallel group: attention output is reduced to every
rank, so each rank already holds every token's hidden state; it runs the routes whose experts it
owns (experts are split contiguously over ranks) and the per-rank partial outputs are summed by
the communicator -- by the peer-memory exchange kernel when the fused communicator is active, by
ncclAllReduce otherwise.  Dispatch therefore needs no all-to-all; combine is the one reduction.  The
reference only sketches EP (docs/quantization/MOE_EXPERT_PARALLELISM.md:60-100) and runs float
MoE on the CPU (crates/onnx-runtime-ep-cpu/src/kernels/moe.rs:1-8).
"""
from __future__ import annotations

from .. import ops
from ..ops import moe as moe_ops
from ..parallel.sharding import shard_range


def moe_forward(model, h, lw, x):
    cfg = model.cfg
    t = h.shape[0]
    e_local = lw.expert_gate_up.shape[0]
    e0, _ = shard_range(cfg.moe.num_experts, model.tp, model.rank)
    ws = getattr(model, "_moe_ws", None)
    if ws is None and h.is_cuda:
        ws = moe_ops.MoEWorkspace(model.max_tokens, cfg.moe.top_k, e_local, cfg.hidden, cfg.moe.expert_intermediate,
                                  model.device, h.dtype)
        model._moe_ws = ws
    router_logits = ops.gemm(h, lw.router_w)
    if model.tp == 1:
        moe_ops.moe_experts(h, router_logits, lw.expert_gate_up, lw.expert_down, ws, x, cfg.moe.top_k, cfg.moe.renormalize,
                            model.w.swiglu_half, e0, accumulate=True)
        return None
    fc = getattr(model, "fused_comm", None)
    if fc is not None and fc.ready:
        # combine over the peer-memory exchange: this rank's experts write their partial sum into the symmetric
        # staging buffer, the owners reduce all ranks' rows (NVSwitch multicast from TP=4) into the residual stream
        part = fc.staging_view(1, t)
        moe_ops.moe_experts(h, router_logits, lw.expert_gate_up, lw.expert_down, ws, part, cfg.moe.top_k, cfg.moe.renormalize,
                            model.w.swiglu_half, e0, accumulate=False)
        fc.reduce_partial(t, 1)
        return None
    if ep_dispatch_mode(model) == "a2a":
        return moe_forward_token_sharded(model, h, lw, ws)
    part = model.partial[:t]
    moe_ops.moe_experts(h, router_logits, lw.expert_gate_up, lw.expert_down, ws, part, cfg.moe.top_k, cfg.moe.renormalize,
                        model.w.swiglu_half, e0, accumulate=False)
    model.comm.all_reduce(part)
    return part


def ep_dispatch_mode(model) -> str:
    """``replicated`` (default): every rank routes every token and the partial outputs are summed.  ``a2a``
    (``OGB_EP_DISPATCH=a2a`` or ``model.ep_dispatch``): each rank routes its slice of the tokens and the rows travel to
    the experts' owners and back (``parallel/ep_dispatch.py``).  The second form is for the plain communicator; the
    fused communicator keeps the replicated combine, which its exchange kernel does in one pass."""
    import os

    return getattr(model, "ep_dispatch", None) or os.environ.get("OGB_EP_DISPATCH", "replicated")


def moe_forward_token_sharded(model, h, lw, ws):
    """The MoE block with tokens sharded over the group: this rank routes rows ``[lo, hi)`` of ``h``, each (row, expert)
    pair is sent to the expert's owner (``exchange_counts`` + ``all_to_all_v``), the owner runs its experts on what it
    received, the outputs return and are summed with the router weights, and an all-gather of the slices restores the
    replicated layout the next block expects.  Returns the block's output for all rows.

    Every rank computes each of its rows' routes once (the replicated form computes them ``tp`` times) and an expert's
    GEMM sees only the rows routed to it; what it costs is two all-to-alls and an all-gather per layer in place of one
    all-reduce."""
    import torch

    from ..ops import reference
    from ..parallel.ep_dispatch import EpDispatcher

    cfg = model.cfg
    t, hidden = h.shape
    ops.launch_counts["ep_dispatch_a2a"] += 1
    lo, hi = shard_range(t, model.tp, model.rank)
    mine = h[lo:hi]
    e0, _ = shard_range(cfg.moe.num_experts, model.tp, model.rank)
    disp = getattr(model, "_ep_dispatcher", None)
    if disp is None:
        disp = model._ep_dispatcher = EpDispatcher(model.comm, cfg.moe.num_experts)
    logits = ops.gemm(mine, lw.router_w) if hi > lo else mine.new_zeros(0, cfg.moe.num_experts)
    ids, wts = reference.moe_route(logits, cfg.moe.top_k, cfg.moe.renormalize)
    plan = disp.plan(ids)
    rows = disp.dispatch(mine, plan).contiguous()
    out_rows = torch.zeros_like(rows)
    if rows.shape[0]:
        # the grouped expert kernel takes router logits: a one-hot row per received row selects its expert with weight 1
        sel = torch.full((rows.shape[0], cfg.moe.num_experts), -30.0, dtype=logits.dtype, device=rows.device)
        sel.scatter_(1, (plan.recv_experts.to(rows.device) + e0).reshape(-1, 1), 30.0)
        ws_rows = ws if (ws is not None and rows.shape[0] <= ws.max_routes) else (
            moe_ops.MoEWorkspace(rows.shape[0], 1, lw.expert_gate_up.shape[0], hidden, cfg.moe.expert_intermediate, model.device, h.dtype)
            if h.is_cuda else None)
        moe_ops.moe_experts(rows, sel, lw.expert_gate_up, lw.expert_down, ws_rows, out_rows, 1, True, model.w.swiglu_half, e0, accumulate=False)
    part = disp.combine(out_rows, wts, plan)
    per = -(-t // model.tp)
    padded = torch.zeros(per, hidden, dtype=h.dtype, device=h.device)
    padded[: hi - lo] = part
    gathered = torch.empty(model.tp * per, hidden, dtype=h.dtype, device=h.device)
    model.comm.all_gather(gathered, padded)
    out = torch.empty(t, hidden, dtype=h.dtype, device=h.device)
    for r in range(model.tp):
        a, b = shard_range(t, model.tp, r)
        out[a:b] = gathered[r * per: r * per + (b - a)]
    return out


def moe_forward_fused(model, h, lw, ready, next_norm):
    """The MoE block under the fused communicator's row-sharded residual: the router GEMM waits for the rows of ``h``
    (``ready``), this rank's experts write their partial sum into the symmetric staging buffer, and one exchange
    reduces all ranks' partials into the owners' residual rows, applies the next RMSNorm and all-gathers ``h``."""
    cfg, fc = model.cfg, model.fused_comm
    t = h.shape[0]
    e_local = lw.expert_gate_up.shape[0]
    e0, _ = shard_range(cfg.moe.num_experts, model.tp, model.rank)
    ws = getattr(model, "_moe_ws", None)
    if ws is None:
        ws = moe_ops.MoEWorkspace(model.max_tokens, cfg.moe.top_k, e_local, cfg.hidden, cfg.moe.expert_intermediate,
                                  model.device, h.dtype)
        model._moe_ws = ws
    router_logits = ops.gemm(h, lw.router_w, a_ready=ready)      # completes only when every tile of h has arrived
    part = fc.staging_view(1, t)
    moe_ops.moe_experts(h, router_logits, lw.expert_gate_up, lw.expert_down, ws, part, cfg.moe.top_k, cfg.moe.renormalize,
                        model.w.swiglu_half, e0, accumulate=False)
    fc.reduce_partial_norm(t, 1, next_norm, cfg.rms_eps)
