"""Mixture-of-experts ops: router top-k, expert permutation, grouped tcgen05 GEMM, weighted combine."""
from __future__ import annotations

import torch

from . import _native, launch_counts, reference, status_word, timed_region

P, I = _native.P, _native.I
_native.register("ogb_moe_route_topk", [P, P, P, I, I, I, I, I, P])
_native.register("ogb_moe_permute", [P] * 8 + [I] * 5 + [P])
_native.register("ogb_moe_gather_rows", [P, P, P, P, I, I, I, P])
_native.register("ogb_moe_combine", [P, P, P, P, I, I, I, I, P])
_native.register("ogb_grouped_gemm_bf16", [P] * 5 + [I] * 7 + [P, P])


def _stream():
    return torch.cuda.current_stream().cuda_stream


class MoEWorkspace:
    """Device scratch of one MoE layer invocation, sized once for the largest step."""

    def __init__(self, max_tokens, k, experts_local, hidden, inter, device, dtype=torch.bfloat16):
        routes = max_tokens * k
        self.max_routes = routes
        self.max_mtiles = (routes + 127) // 128 + experts_local
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=device)
        self.topk_ids, self.route_pos, self.sorted_route = i32(routes), i32(routes), i32(routes)
        self.topk_w = torch.zeros(routes, dtype=torch.float32, device=device)
        self.counts, self.offsets, self.cursor = i32(experts_local), i32(experts_local + 1), i32(experts_local)
        self.tile_tab, self.meta = i32(4 * self.max_mtiles), i32(2)
        # rows are padded to whole 128-row tiles so a tile's TMA box never leaves the buffer
        rows = self.max_mtiles * 128
        self.xs = torch.zeros(rows, hidden, dtype=dtype, device=device)
        self.act = torch.zeros(rows, inter, dtype=dtype, device=device)
        self.ys = torch.zeros(rows, hidden, dtype=dtype, device=device)


def moe_experts(h, router_logits, expert_gate_up, expert_down, ws: MoEWorkspace, out, k, renormalize, half, e0=0,
                accumulate=True):
    """out (+)= sum over this rank's experts of w * down(swiglu(gate_up(h))).

    router_logits [T, E_total] bf16; expert_gate_up [E_local, 2I, H] packed per expert with half-width
    ``half``; expert_down [E_local, H, I]; e0 = first global expert id held locally.
    """
    t, hidden = h.shape
    e_total = router_logits.shape[1]
    e_local, two_i, _ = expert_gate_up.shape
    inter = two_i // 2
    if not h.is_cuda:
        ids, w = reference.moe_route(router_logits, k, renormalize)
        res = out.float() if accumulate else torch.zeros_like(out, dtype=torch.float32)
        for e in range(e_local):
            mask = ids == (e0 + e)
            rows = mask.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            a = reference.swiglu_packed(h[rows].float(), expert_gate_up[e].float(), half, torch.float32)
            y = a @ expert_down[e].float().t()
            res[rows] += y * (w[rows] * mask[rows]).sum(-1, keepdim=True)
        out.copy_(res.to(out.dtype))
        return out
    lib = _native.load()
    st = status_word(h.device).data_ptr()
    s = _stream()
    with timed_region("moe_route_permute"):
        rc = lib.ogb_moe_route_topk(router_logits.data_ptr(), ws.topk_ids.data_ptr(), ws.topk_w.data_ptr(), t, e_total, k,
                                    int(renormalize), router_logits.stride(0), s)
        _native.check(rc, "ogb_moe_route_topk")
        rc = lib.ogb_moe_permute(ws.topk_ids.data_ptr(), ws.counts.data_ptr(), ws.offsets.data_ptr(), ws.cursor.data_ptr(),
                                 ws.sorted_route.data_ptr(), ws.route_pos.data_ptr(), ws.tile_tab.data_ptr(), ws.meta.data_ptr(),
                                 t, k, e0, e_local, ws.max_mtiles, s)
        _native.check(rc, "ogb_moe_permute")
        rc = lib.ogb_moe_gather_rows(h.data_ptr(), ws.sorted_route.data_ptr(), ws.meta.data_ptr(), ws.xs.data_ptr(), t * k, k,
                                     hidden, s)
        _native.check(rc, "ogb_moe_gather_rows")
    max_mtiles = min(ws.max_mtiles, (t * k + 127) // 128 + e_local)
    rows = max_mtiles * 128
    with timed_region("moe_grouped_gemm_gate_up"):
        rc = lib.ogb_grouped_gemm_bf16(ws.xs.data_ptr(), expert_gate_up.data_ptr(), ws.act.data_ptr(), ws.tile_tab.data_ptr(),
                                       ws.meta.data_ptr(), e_local, rows, max_mtiles, two_i, hidden, 2, 2 * half, st, s)
    _native.check(rc, "ogb_grouped_gemm_bf16[gate_up]")
    bn = 256 if hidden % 256 == 0 else 128
    with timed_region("moe_grouped_gemm_down"):
        rc = lib.ogb_grouped_gemm_bf16(ws.act.data_ptr(), expert_down.data_ptr(), ws.ys.data_ptr(), ws.tile_tab.data_ptr(),
                                       ws.meta.data_ptr(), e_local, rows, max_mtiles, hidden, inter, 0, bn, st, s)
    _native.check(rc, "ogb_grouped_gemm_bf16[down]")
    with timed_region("moe_combine"):
        rc = lib.ogb_moe_combine(ws.ys.data_ptr(), ws.route_pos.data_ptr(), ws.topk_w.data_ptr(), out.data_ptr(), t, k, hidden,
                                 int(accumulate), s)
    _native.check(rc, "ogb_moe_combine")
    launch_counts["moe_route_topk"] += 1
    launch_counts["moe_permute"] += 4
    launch_counts["moe_gather_rows"] += 1
    launch_counts["moe_grouped_gemm"] += 2
    launch_counts["moe_combine"] += 1
    return out
