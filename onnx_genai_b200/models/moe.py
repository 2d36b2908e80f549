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
    part = model.partial[:t]
    moe_ops.moe_experts(h, router_logits, lw.expert_gate_up, lw.expert_down, ws, part, cfg.moe.top_k, cfg.moe.renormalize,
                        model.w.swiglu_half, e0, accumulate=False)
    model.comm.all_reduce(part)
    return part


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
