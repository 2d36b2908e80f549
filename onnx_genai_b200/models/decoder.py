"""Fused decoder executor: one static plan of ~8 kernels per layer over a paged KV pool.

The reference executes the decoder ONNX graph node by node (≈300-2600 kernel nodes per token,
docs/execution/NATIVE_CUDA_DECODE.md:133-150) after graph-level fusions
(crates/onnx-runtime-ep-cuda/src/optimizer.rs:106-158).  Here the recognised pattern
(RMSNorm -> qkv MatMul -> rotary + GQA with KV append -> o_proj + residual -> RMSNorm ->
gate/up MatMul + SwiGLU -> down MatMul + residual) is lowered once to this plan:

    rmsnorm | gemm(qkv,+bias) | rope_kv_append | paged_decode + paged_prefill |
    gemm(o_proj,+residual) | rmsnorm | gemm(gate_up, SwiGLU epilogue) | gemm(down,+residual)

Every buffer is preallocated for the largest step, so a step launches kernels and nothing else.
Under tensor parallelism the two row-parallel GEMMs produce partial sums that the communicator
reduces; the residual add then rides in the next RMSNorm (``delta``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .. import ops
from ..ops import reference as ref
from ..parallel.sharding import shard_heads, shard_range
from .config import DecoderConfig


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    qkv_w: torch.Tensor
    qkv_b: torch.Tensor | None
    o_w: torch.Tensor
    ln2: torch.Tensor
    gate_up_w: torch.Tensor | None = None     # packed by ops.pack_gate_up
    down_w: torch.Tensor | None = None
    # MoE
    router_w: torch.Tensor | None = None
    expert_gate_up: torch.Tensor | None = None  # [E_local, 2*I, H] packed per expert
    expert_down: torch.Tensor | None = None     # [E_local, H, I]
    quant: dict = field(default_factory=dict)   # int4 tensors keyed by projection name


@dataclass
class DecoderWeights:
    embed: torch.Tensor
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    swiglu_half: int = 128


def pick_swiglu_half(inter_local: int) -> int:
    for half in (128, 64, 32):
        if inter_local % half == 0:
            return half
    raise ValueError(f"intermediate size {inter_local} is not a multiple of 32")


def pad_mlp(gate, up, down, multiple: int = 64):
    """Zero-pad the MLP's intermediate dimension to a multiple of the GEMM tile half-width.  Exact:
    padded gate/up rows produce silu(0) * 0 = 0 and meet zero columns of the down projection."""
    inter = gate.shape[0]
    pad = (-inter) % multiple
    if pad == 0:
        return gate, up, down
    z = torch.zeros(pad, gate.shape[1], dtype=gate.dtype, device=gate.device)
    zd = torch.zeros(down.shape[0], pad, dtype=down.dtype, device=down.device)
    return torch.cat([gate, z], 0), torch.cat([up, z], 0), torch.cat([down, zd], 1)


def random_weights(cfg: DecoderConfig, device, tp: int = 1, rank: int = 0, seed: int = 0, std: float = 0.02,
                   dtype=torch.bfloat16) -> DecoderWeights:
    """Seeded N(0, std) weights of the architecture, sharded for (tp, rank).

    Each full matrix is drawn from its own generator seed, then sliced, so every rank of any
    TP degree sees slices of the same global matrices.
    """
    dev = torch.device(device)
    counter = [seed * 1000003]

    def draw(*shape):
        counter[0] += 1
        g = torch.Generator(device=dev).manual_seed(counter[0])
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)

    hs = shard_heads(cfg.num_heads, cfg.num_kv_heads, tp, rank)
    d, hid = cfg.head_dim, cfg.hidden
    q_rows = torch.tensor([h * d + i for h in hs.q_heads for i in range(d)], device=dev)
    kv_rows = torch.tensor([h * d + i for h in hs.kv_heads for i in range(d)], device=dev)
    moe = cfg.moe.num_experts > 0
    if not moe:
        i0, i1 = shard_range(cfg.intermediate, tp, rank, math.gcd(cfg.intermediate, 32) if tp > 1 else 1)
        half = pick_swiglu_half((i1 - i0) + (-(i1 - i0)) % 64 if (i1 - i0) % 32 else (i1 - i0))
    else:
        half = pick_swiglu_half(cfg.moe.expert_intermediate)
    embed = draw(cfg.vocab, hid)
    layers = []
    for _ in range(cfg.num_layers):
        wq, wk, wv = draw(cfg.q_size, hid), draw(cfg.kv_size, hid), draw(cfg.kv_size, hid)
        qkv_w = torch.cat([wq[q_rows], wk[kv_rows], wv[kv_rows]], 0).contiguous()
        qkv_b = None
        if cfg.qkv_bias:
            bq, bk, bv = draw(cfg.q_size), draw(cfg.kv_size), draw(cfg.kv_size)
            qkv_b = torch.cat([bq[q_rows], bk[kv_rows], bv[kv_rows]], 0).contiguous()
        del wq, wk, wv
        o_w = draw(hid, cfg.q_size)[:, q_rows].contiguous()
        lw = LayerWeights(ln1=torch.ones(hid, device=dev, dtype=dtype), qkv_w=qkv_w, qkv_b=qkv_b, o_w=o_w,
                          ln2=torch.ones(hid, device=dev, dtype=dtype))
        if not moe:
            g = draw(cfg.intermediate, hid)[i0:i1]
            u = draw(cfg.intermediate, hid)[i0:i1]
            dn = draw(hid, cfg.intermediate)[:, i0:i1]
            if (i1 - i0) % 32:
                g, u, dn = pad_mlp(g, u, dn)
            lw.gate_up_w = ops.pack_gate_up(g.contiguous(), u.contiguous(), half)
            del g, u
            lw.down_w = dn.contiguous()
        else:
            e0, e1 = shard_range(cfg.moe.num_experts, tp, rank)
            lw.router_w = draw(cfg.moe.num_experts, hid)
            inter = cfg.moe.expert_intermediate
            gus, dws = [], []
            for e in range(cfg.moe.num_experts):
                g, u, dw = draw(inter, hid), draw(inter, hid), draw(hid, inter)
                if e0 <= e < e1:
                    gus.append(ops.pack_gate_up(g, u, half))
                    dws.append(dw)
            lw.expert_gate_up = torch.stack(gus).contiguous()
            lw.expert_down = torch.stack(dws).contiguous()
        layers.append(lw)
    final_norm = torch.ones(hid, device=dev, dtype=dtype)
    lm_head = embed if cfg.tie_embeddings else draw(cfg.vocab, hid)
    return DecoderWeights(embed=embed, layers=layers, final_norm=final_norm, lm_head=lm_head, swiglu_half=half)


@dataclass
class StepInputs:
    """Device views of one packed step plan (see csrc/runtime/core.h PlanLayout)."""
    num_tokens: int
    num_decode: int
    num_prefill_seqs: int
    num_tiles: int
    num_logit_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    slots: torch.Tensor
    ctx_len: torch.Tensor          # [S] decode rows first
    page_table: torch.Tensor       # [S, max_pages]
    cu_q: torch.Tensor             # [Np + 1]
    tile_seq: torch.Tensor
    tile_q0: torch.Tensor
    logit_rows: torch.Tensor       # [R]
    max_ctx: int = 0
    # Speculative verification over long contexts: when every "prefill" sequence of the step is just a handful
    # of draft rows, the engine describes those rows as decode rows (one page-table row and context length per
    # query row) so attention runs on the split-KV decode kernel instead of walking the whole context in one CTA.
    verify_table: torch.Tensor | None = None   # [rows, max_pages]
    verify_ctx: torch.Tensor | None = None     # [rows]
    verify_splits: int = 1
    force_python: bool = False                 # run this step op by op from Python even if the C++ executor is bound


class KVCache:
    """Per-layer paged pools [pages, kv_heads_local, 2, 16, head_dim] (bf16, or e4m3 + scales).

    With ``max_pages`` > ``num_pages`` on a CUDA device each pool (and scale table) is a view over a reserved address
    range of ``max_pages`` pages of which only the first ``num_pages`` are backed; :meth:`grow` backs more in place, so
    page ids, tensor addresses, cached TMA descriptors and captured graphs stay valid.  Nothing may touch pages
    beyond ``num_pages``; the page allocator never hands them out before :meth:`grow` has returned."""

    def __init__(self, cfg: DecoderConfig, num_pages: int, device, kv_heads_local: int | None = None, dtype="bf16",
                 max_pages: int = 0, layers=None, allocator=None):
        """``layers``: the layer indices this process runs (a pipeline stage); the others get no pool.  ``allocator``: an
        engine allocator (engine/allocator.py) the fixed-size pools come from; torch's allocator when absent."""
        hkv = kv_heads_local or cfg.num_kv_heads
        own = set(range(cfg.num_layers)) if layers is None else set(layers)
        self.own_layers = sorted(own)
        self.num_pages = num_pages
        self.dtype = dtype
        if dtype not in ("bf16", "fp8", "int8", "fp8_e5m2"):
            raise ValueError(f"kv dtype {dtype!r} is not supported; use bf16, fp8 (e4m3 pages), fp8_e5m2 or int8")
        # one-byte pools say their format by dtype
        tdtype = {"bf16": torch.bfloat16, "fp8": torch.uint8, "int8": torch.int8, "fp8_e5m2": torch.float8_e5m2}[dtype]
        if torch.device(device).type == "cpu" and dtype == "bf16":
            tdtype = torch.float32
        quant = dtype in ("fp8", "int8", "fp8_e5m2")
        self.max_pages = max(int(max_pages), num_pages)
        self.buffers = None
        if self.max_pages > num_pages and torch.device(device).type == "cuda":
            from ..utils.vmm import GrowableBuffer

            dev = torch.device(device).index or 0
            self.page_nbytes = hkv * 2 * ops.PAGE * cfg.head_dim * torch.empty(0, dtype=tdtype).element_size()
            self.scale_nbytes = hkv * 2 * 4
            self.buffers, self.scale_buffers, self.pools, self.scales = [], [], [], [] if quant else None
            for _ in range(cfg.num_layers):
                buf = GrowableBuffer(self.max_pages * self.page_nbytes, dev, num_pages * self.page_nbytes)
                self.buffers.append(buf)
                buf.view(torch.uint8).zero_()
                self.pools.append(buf.span(tdtype, (self.max_pages, hkv, 2, ops.PAGE, cfg.head_dim)))
                if quant:
                    sb = GrowableBuffer(self.max_pages * self.scale_nbytes, dev, num_pages * self.scale_nbytes)
                    self.scale_buffers.append(sb)
                    sb.view(torch.uint8).zero_()
                    self.scales.append(sb.span(torch.float32, (self.max_pages, hkv, 2)))
            self._mark_backed()
            return
        self.max_pages = num_pages
        if allocator is not None:
            make = lambda shape, dt, tag: allocator.tensor(shape, dt, "kv", tag)
        else:
            make = lambda shape, dt, tag: torch.zeros(*shape, dtype=dt, device=device)
        self.pools = [make((num_pages, hkv, 2, ops.PAGE, cfg.head_dim), tdtype, f"pages of layer {li}") if li in own else None
                      for li in range(cfg.num_layers)]
        self.scales = None
        if quant:
            self.scales = [make((num_pages, hkv, 2), torch.float32, f"page scales of layer {li}") if li in own else None
                           for li in range(cfg.num_layers)]

    def _mark_backed(self) -> None:
        """Record the mapped page count on every pool tensor: kernels bound page ids by it (ops.backed_pages)."""
        for t in self.pools:
            t.backed_pages = self.num_pages

    @property
    def growable(self) -> bool:
        return self.buffers is not None and self.num_pages < self.max_pages

    def grow(self, new_pages: int) -> int:
        """Back pages up to ``new_pages`` (clamped to ``max_pages``) in every layer; returns the new page count.  If the
        device runs out of memory part-way, layers that already grew keep their extra backing (harmless) and the page
        count stays where it was."""
        if self.buffers is None:
            return self.num_pages
        new_pages = min(int(new_pages), self.max_pages)
        if new_pages <= self.num_pages:
            return self.num_pages
        for buf in self.buffers:
            old = buf.mapped
            buf.grow(new_pages * self.page_nbytes)
            if buf.mapped > old:     # scale tables rely on zero meaning "page not started"; pools are zeroed for tidiness
                buf.view(torch.uint8, (buf.mapped - old,), old).zero_()
        for sb in self.scale_buffers:
            old = sb.mapped
            sb.grow(new_pages * self.scale_nbytes)
            if sb.mapped > old:
                sb.view(torch.uint8, (sb.mapped - old,), old).zero_()
        self.num_pages = new_pages
        self._mark_backed()
        return new_pages

    def allocations(self) -> list:
        """The allocator's records behind the pools and scale tables (empty when torch's allocator made them)."""
        ts = [t for t in (self.pools + (self.scales or [])) if t is not None]
        return [t.ogb_allocation for t in ts if hasattr(t, "ogb_allocation")]

    @property
    def own_pools(self) -> list:
        """The pools this process holds (all of them unless it is a pipeline stage), in layer order."""
        return [self.pools[li] for li in self.own_layers]

    @property
    def own_scales(self):
        return [self.scales[li] for li in self.own_layers] if self.scales is not None else None

    def mapped_bytes(self) -> int:
        if self.buffers is None:
            return sum(p.numel() * p.element_size() for p in self.own_pools) + sum(s.numel() * 4 for s in (self.own_scales or []))
        return sum(b.mapped for b in self.buffers) + sum(b.mapped for b in self.scale_buffers)

    def page_bytes(self) -> int:
        p = self.own_pools[0]
        return p.stride(0) * p.element_size() * len(self.own_layers)


class DecoderModel:
    def __init__(self, cfg: DecoderConfig, weights: DecoderWeights, device, max_tokens: int, max_seqs: int,
                 tp: int = 1, rank: int = 0, comm=None):
        self.cfg, self.w, self.device = cfg, weights, torch.device(device)
        self.tp, self.rank, self.comm = tp, rank, comm
        hs = shard_heads(cfg.num_heads, cfg.num_kv_heads, tp, rank)
        self.hq, self.hkv, self.d = len(hs.q_heads), len(hs.kv_heads), cfg.head_dim
        self.rotary_dim = cfg.rotary_dim or cfg.head_dim
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        if self.device.type == "cuda" and cfg.head_dim not in (64, 128):
            raise ValueError(f"head dimension {cfg.head_dim} is not supported on CUDA: the paged attention kernels are built for 64 and 128 "
                             "(the CPU path and the node-by-node graph backend take any head dimension)")
        dt = weights.embed.dtype
        dev = self.device
        hid = cfg.hidden
        cs = getattr(weights, "cos_sin", None)   # a loaded package brings its own cos/sin caches
        self.cos_sin = (cs.to(dev) if cs is not None
                        else ref.rope_table(cfg.max_position, self.rotary_dim, cfg.rope_theta, dev))
        z = lambda *s: torch.zeros(*s, dtype=dt, device=dev)
        self.fused_comm = comm if (comm is not None and hasattr(comm, "row_parallel") and dev.type == "cuda") else None
        self.x = z(max_tokens, hid)                 # residual stream (under fused TP: only the rows this rank owns stay current)
        if self.fused_comm is not None:
            if not self.fused_comm.ready:
                self.fused_comm.setup(hid, max_tokens)
            self.fused_comm.bind_residual(self.x)
            self.h = self.fused_comm.h              # normed activations live in the peer-mapped region: owners deliver their rows
        else:
            self.h = z(max_tokens, hid)             # normed activations
        self.qkv = z(max_tokens, (self.hq + 2 * self.hkv) * self.d)
        self.attn = z(max_tokens, self.hq * self.d)
        inter_local = (weights.layers[0].gate_up_w.shape[0] // 2) if weights.layers[0].gate_up_w is not None else 0
        self.act = z(max_tokens, max(inter_local, 8))
        self.partial = z(max_tokens, hid) if tp > 1 else None
        if any(l.quant for l in weights.layers):     # MatMulNBits layers: build the int4 projections
            from ..ops.quant import QuantLinear

            for l in weights.layers:
                if l.quant and not isinstance(l.quant.get("o"), QuantLinear):
                    mk = lambda lin: QuantLinear(lin.q, lin.scales, lin.zp, lin.bias, lin.k, lin.block, dev)
                    l.quant = {"qkv": [mk(p) for p in l.quant["qkv"]], "o": mk(l.quant["o"]), "gate": mk(l.quant["gate"]),
                               "up": mk(l.quant["up"]), "down": mk(l.quant["down"])}
                    # sibling projections of one input become one launch (the reference does this in its
                    # CudaQkvProjectionFusion / gate_up fusion passes, ep-cuda/src/optimizer.rs:64-83,3175)
                    merged_qkv = QuantLinear.merge(l.quant["qkv"])
                    if merged_qkv is not None:
                        l.quant["qkv"] = [merged_qkv]
                    l.quant["gate_up"] = QuantLinear.merge([l.quant["gate"], l.quant["up"]])
            inter_q = weights.layers[0].quant["gate"].n
            self.partial = z(max_tokens, hid)
            self.gate_up = z(max_tokens, 2 * inter_q)
            self.act_q = z(max_tokens, inter_q)
        self.h_last = z(max_seqs, hid)
        self.x_last = z(max_seqs, hid)
        self.logits = z(max_seqs, cfg.vocab)
        self.scale = 1.0 / math.sqrt(self.d)
        self.decode_splits = 1
        self.part_o = self.part_ml = None
        self._tp_args_cache: dict = {}
        self.pipeline = (0, 1)      # (stage, stages): see set_pipeline
        self.native = None          # C++ step executor (dense bf16 layers, bf16 pages; TP needs the fused communicator)
        self.native_launches = 0

    def bind_native(self, kv: "KVCache", max_pages_per_seq: int) -> bool:
        """Create the C++ step executor over this model's buffers; returns False when the
        configuration needs the Python-driven path (TP > 1, MoE, int4 weights, fp8 pages, CPU)."""
        import ctypes

        from ..ops import _native

        cfg, w = self.cfg, self.w
        if (self.device.type != "cuda" or (self.tp != 1 and self.fused_comm is None) or kv.scales is not None
                or ops._BASELINE
                or any(l.gate_up_w is None or l.quant for l in w.layers)):
            return False
        lib = _native.load()
        lib.ogb_decoder_create.restype = ctypes.c_void_p
        lib.ogb_decoder_create.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.ogb_decoder_step.restype = ctypes.c_int
        lib.ogb_decoder_step.argtypes = ([ctypes.c_void_p] * 10 + [ctypes.c_int] * 6 + [ctypes.c_void_p, ctypes.c_void_p,
                                                                                         ctypes.c_int])
        lib.ogb_decoder_launches.restype = ctypes.c_longlong
        lib.ogb_decoder_launches.argtypes = [ctypes.c_void_p]
        lib.ogb_decoder_counter.restype = ctypes.c_longlong
        lib.ogb_decoder_counter.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.ogb_decoder_set_split_scratch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.ogb_decoder_set_split_scratch.restype = None
        inter_local = w.layers[0].gate_up_w.shape[0] // 2
        ip = (ctypes.c_int * 16)(cfg.num_layers, cfg.hidden, self.hq, self.hkv, self.d, self.rotary_dim,
                                 int(cfg.rotary_interleaved), inter_local, cfg.vocab, 2 * w.swiglu_half,
                                 cfg.sliding_window, max_pages_per_seq, self.cos_sin.shape[0], self.tp,
                                 1 if ops.PREFILL_TC else 0, cfg.sink_len)
        fp = (ctypes.c_float * 2)(cfg.rms_eps, self.scale)
        ptr = lambda t: 0 if t is None else t.data_ptr()
        g = [w.embed, w.final_norm, w.lm_head, self.cos_sin, self.x, self.h, self.qkv, self.attn, self.act, self.x_last,
             self.h_last, self.logits, self.partial, self.part_o, self.part_ml, ops.status_word(self.device)]
        gp = (ctypes.c_uint64 * len(g))(*[ptr(t) for t in g])
        lp = (ctypes.c_uint64 * (8 * cfg.num_layers))()
        for i, lw in enumerate(w.layers):
            for j, t in enumerate((lw.ln1, lw.qkv_w, lw.qkv_b, lw.o_w, lw.ln2, lw.gate_up_w, lw.down_w, kv.pools[i])):
                lp[8 * i + j] = ptr(t)
        self._native_lib = lib
        lib.ogb_decoder_set_num_pages.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        lib.ogb_decoder_set_num_pages.restype = None
        self.native = lib.ogb_decoder_create(ip, kv.num_pages, fp, gp, lp)   # backed pages: ids beyond them are refused
        if self.native and getattr(self, "weight_offload_layers", 0) > 0:
            self._page_weights(lib, int(self.weight_offload_layers))
        return bool(self.native)

    def _page_weights(self, lib, n_layers: int) -> None:
        """Move the matrices of the last ``n_layers`` layers to pinned host memory, one contiguous pack per layer, and let
        the step executor stream them through two device slots (the copy of layer l + 1 runs under the compute of layer
        l).  Device memory then holds the first layers, two slots and the activations; the cost is one PCIe pass over the
        paged weights per step.  The device copies are released here."""
        import ctypes

        w = self.w
        n_layers = min(n_layers, len(w.layers))
        first = len(w.layers) - n_layers
        names = ("qkv_w", "o_w", "gate_up_w", "down_w")
        align = lambda b: (b + 255) // 256 * 256
        sizes = [align(getattr(w.layers[first], n).numel() * 2) for n in names]
        offsets = [sum(sizes[:i]) for i in range(4)]
        total = sum(sizes)
        self.weight_packs, self.weight_slots = [], [torch.empty(total, dtype=torch.uint8, device=self.device) for _ in range(2)]
        for lw in w.layers[first:]:
            pack = torch.empty(total, dtype=torch.uint8, pin_memory=True)
            for n, off in zip(names, offsets):
                t = getattr(lw, n)
                if t.numel() * 2 > sizes[names.index(n)] or t.dtype != torch.bfloat16:
                    raise ValueError("weight paging needs layers of one shape in bf16")
                pack[off:off + t.numel() * 2].copy_(t.contiguous().view(torch.uint8).reshape(-1))
                setattr(lw, n, None)                      # the device copy goes away; the Python-driven path cannot run paged layers
            self.weight_packs.append(pack)
        lib.ogb_decoder_set_weight_paging.restype = ctypes.c_int
        lib.ogb_decoder_set_weight_paging.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        lib.ogb_decoder_weight_copies.restype = ctypes.c_longlong
        lib.ogb_decoder_weight_copies.argtypes = [ctypes.c_void_p]
        hp = (ctypes.c_uint64 * n_layers)(*[p.data_ptr() for p in self.weight_packs])
        sp = (ctypes.c_uint64 * 2)(*[s.data_ptr() for s in self.weight_slots])
        op = (ctypes.c_int64 * 4)(*offsets)
        rc = lib.ogb_decoder_set_weight_paging(self.native, first, hp, sp, total, op)
        if rc != 0:
            raise RuntimeError(f"ogb_decoder_set_weight_paging failed with code {rc}")
        self.paged_weight_bytes = total * n_layers
        torch.cuda.empty_cache()

    def weight_copies(self) -> int:
        """Layer packs copied host -> device by the step executor so far (weight paging)."""
        return int(self._native_lib.ogb_decoder_weight_copies(self.native)) if self.native and getattr(self, "weight_packs", None) else 0

    def native_counter(self, which: int) -> int:
        """Kernels the C++ step executor has launched so far: 0 all, 1 scatter-epilogue GEMMs, 2 exchange kernels."""
        return int(self._native_lib.ogb_decoder_counter(self.native, which)) if self.native else 0

    def set_backed_pages(self, num_pages: int) -> None:
        """The KV pool grew in place: the step executor bounds page ids by the new backed count from now on."""
        if self.native:
            self._native_lib.ogb_decoder_set_num_pages(self.native, int(num_pages))

    def _tp_step_args(self, rows: int):
        """(pointer to the 4 device-struct addresses for this step's row chunk, chunk) or (None, 0)."""
        fc = self.fused_comm
        if fc is None:
            return None, 0
        import ctypes

        chunk = fc.chunk_for(rows)
        hit = self._tp_args_cache.get(chunk)
        if hit is None:
            sc0, rd0 = fc._get_structs(0, chunk, fc.push)
            sc1, rd1 = fc._get_structs(1, chunk, fc.push)
            hit = (ctypes.c_uint64 * 7)(sc0.data_ptr(), rd0.data_ptr(), sc1.data_ptr(), rd1.data_ptr(),
                                        (1 if fc.nvls else 0) | (2 if fc.push else 0),
                                        fc.ready_ptrs(0)[0], fc.ready_ptrs(1)[0])
            self._tp_args_cache[chunk] = hit
        return hit, chunk

    def ensure_split_scratch(self, splits: int) -> bool:
        """Scratch for `splits` partial results per (row, head); grows only.  True when it was reallocated (pointers
        captured in CUDA graphs are then stale)."""
        if splits <= 1 or self.device.type != "cuda" or splits <= getattr(self, "_split_capacity", 1):
            return False
        self._split_capacity = splits
        self.part_o = torch.empty(self.max_seqs * self.hq * splits * self.d, dtype=torch.float32, device=self.device)
        self.part_ml = torch.empty(self.max_seqs * self.hq * splits * 2, dtype=torch.float32, device=self.device)
        if self.native:
            self._native_lib.ogb_decoder_set_split_scratch(self.native, self.part_o.data_ptr(), self.part_ml.data_ptr())
        return True

    def set_decode_splits(self, splits: int) -> bool:
        self.decode_splits = splits
        return self.ensure_split_scratch(splits)

    # --------------------------------------------------------------------------------------
    def set_pipeline(self, stage: int, stages: int, ranges) -> None:
        """Make this model one stage of a pipeline: it keeps the layers ``ranges[stage]`` (the others' weights are
        dropped), the first stage embeds, every other stage receives the residual stream from its predecessor, the last
        stage applies the final norm and the LM head.  Stages run the step op by op from Python."""
        if self.tp != 1:
            raise ValueError("pipeline stages are built for tp = 1 (one GPU per stage)")
        lo, hi = ranges[stage]
        self.pipeline = (stage, stages)
        self.layer_range = (lo, hi)
        if self.native:
            self._native_lib.ogb_decoder_destroy(self.native)
            self.native = None
        for li in range(len(self.w.layers)):
            if not lo <= li < hi:
                self.w.layers[li] = None

    def set_hidden_taps(self, layers) -> None:
        """Keep, for every logit row of a step, the residual stream entering each of ``layers`` (0 = the embeddings,
        ``num_layers`` is not allowed: that state is ``h_last`` before its norm).  Draft heads that read intermediate
        features (EAGLE-3 style) use them.  Taps make the step run layer by layer from Python."""
        layers = sorted(set(int(l) for l in layers))
        if any(l < 0 or l >= self.cfg.num_layers for l in layers):
            raise ValueError(f"tap layers {layers} must lie in [0, {self.cfg.num_layers})")
        if layers and self.tp != 1:
            raise ValueError("hidden taps are supported on one GPU only: with tensor parallelism the residual is completed lazily")
        self.tap_layers = layers
        self.taps = {l: torch.zeros_like(self.h_last) for l in layers}

    def forward(self, si: StepInputs, kv: KVCache) -> torch.Tensor:
        """Runs one step; returns logits [num_logit_rows, vocab] (a view of a static buffer)."""
        cfg, w = self.cfg, self.w
        t, nd = si.num_tokens, si.num_decode
        tapping = bool(getattr(self, "tap_layers", None))
        if self.native and not si.force_python and not tapping:
            before = self._native_lib.ogb_decoder_launches(self.native)
            rc = self._native_lib.ogb_decoder_step(
                self.native, si.token_ids.data_ptr(), si.positions.data_ptr(), si.slots.data_ptr(), si.ctx_len.data_ptr(),
                si.page_table.data_ptr(), si.cu_q.data_ptr(), si.tile_seq.data_ptr(), si.tile_q0.data_ptr(),
                si.logit_rows.data_ptr(), t, nd, si.num_prefill_seqs, si.num_tiles, si.num_logit_rows,
                self.decode_splits, torch.cuda.current_stream().cuda_stream, *self._tp_step_args(t))
            if rc != 0:
                raise RuntimeError(f"ogb_decoder_step failed with code {rc}")
            n = self._native_lib.ogb_decoder_launches(self.native) - before
            ops.launch_counts["native_step_kernels"] += n
            return self.logits[: si.num_logit_rows]
        if self.fused_comm is not None and self.tp > 1:
            return self._forward_tp_fused(si, kv)
        x, h, qkv, attn = self.x[:t], self.h[:t], self.qkv[:t], self.attn[:t]
        stage, stages = self.pipeline
        if stage == 0:
            ops.embedding(si.token_ids[:t], w.embed, out=x) if x.is_cuda else x.copy_(w.embed[si.token_ids[:t].long()])
        else:
            self.comm.recv(x, stage - 1)                 # the residual stream after the previous stage's last layer
        pending = None  # partial sums still to be added to the residual (TP only)
        # int4 layers at decode size: norm, SwiGLU glue and residual adds live inside the GEMV launches
        fused_q = (x.is_cuda and t <= 4 and self.tp == 1 and all(l is not None and l.quant and len(l.quant["qkv"]) == 1 and
                                                                 l.quant.get("gate_up") is not None for l in w.layers))
        for li, lw in enumerate(w.layers):
            if lw is None:                               # a layer of another pipeline stage
                continue
            pool = kv.pools[li]
            if fused_q:
                if tapping and li in self.taps:
                    torch.index_select(x, 0, si.logit_rows[:si.num_logit_rows].long(), out=self.taps[li][:si.num_logit_rows])
                lw.quant["qkv"][0].fused(x, qkv, norm_weight=lw.ln1, eps=cfg.rms_eps)
                ops.rope_kv_append(qkv, si.positions[:t], si.slots[:t], self.cos_sin, pool, self.hq, self.hkv, self.d,
                                   self.rotary_dim, cfg.rotary_interleaved,
                                   kv_scales=kv.scales[li] if kv.scales is not None else None)
                if nd > 0:
                    ops.paged_decode(qkv[:nd], attn[:nd], pool, si.page_table[:nd], si.ctx_len[:nd], self.hq, self.hkv,
                                     self.d, self.scale, self.decode_splits, self.part_o, self.part_ml, cfg.sliding_window,
                                     kv_scales=kv.scales[li] if kv.scales is not None else None, sink=cfg.sink_len)
                if si.num_prefill_seqs > 0:
                    np_ = si.num_prefill_seqs
                    ops.paged_prefill(qkv[nd:], attn[nd:], pool, si.page_table[nd:nd + np_], si.ctx_len[nd:nd + np_],
                                      si.cu_q, si.tile_seq, si.tile_q0, si.num_tiles, self.hq, self.hkv, self.d, self.scale,
                                      cfg.sliding_window, kv_scales=kv.scales[li] if kv.scales is not None else None, sink=cfg.sink_len)
                lw.quant["o"].fused(attn, x, residual=x)
                gu = self.gate_up[:t, : 2 * lw.quant["gate"].n]
                lw.quant["gate_up"].fused(x, gu, norm_weight=lw.ln2, eps=cfg.rms_eps)
                lw.quant["down"].fused(gu, x, silu_mul=True, residual=x)
                continue
            self._norm(x, lw.ln1, pending, h)
            if tapping and li in self.taps:       # the norm has just folded the previous layer's output into x
                torch.index_select(x, 0, si.logit_rows[:si.num_logit_rows].long(), out=self.taps[li][:si.num_logit_rows])
            if lw.quant:
                c0 = 0
                for proj in lw.quant["qkv"]:          # q, k, v MatMulNBits write adjacent column slices
                    proj(h, out=qkv[:, c0:c0 + proj.n])
                    c0 += proj.n
            else:
                self._gemm(h, lw.qkv_w, out=qkv, bias=lw.qkv_b)
            ops.rope_kv_append(qkv, si.positions[:t], si.slots[:t], self.cos_sin, pool, self.hq, self.hkv, self.d,
                               self.rotary_dim, cfg.rotary_interleaved,
                               kv_scales=kv.scales[li] if kv.scales is not None else None)
            if nd > 0:
                ops.paged_decode(qkv[:nd], attn[:nd], pool, si.page_table[:nd], si.ctx_len[:nd], self.hq, self.hkv,
                                 self.d, self.scale, self.decode_splits, self.part_o, self.part_ml, cfg.sliding_window,
                                 kv_scales=kv.scales[li] if kv.scales is not None else None, sink=cfg.sink_len)
            if si.num_prefill_seqs > 0 and si.verify_table is not None:
                nv = si.verify_ctx.numel()
                ops.paged_decode(qkv[nd:nd + nv], attn[nd:nd + nv], pool, si.verify_table, si.verify_ctx, self.hq, self.hkv,
                                 self.d, self.scale, si.verify_splits, self.part_o, self.part_ml, cfg.sliding_window,
                                 kv_scales=kv.scales[li] if kv.scales is not None else None, sink=cfg.sink_len)
            elif si.num_prefill_seqs > 0:
                np_ = si.num_prefill_seqs
                ops.paged_prefill(qkv[nd:], attn[nd:], pool, si.page_table[nd:nd + np_], si.ctx_len[nd:nd + np_],
                                  si.cu_q, si.tile_seq, si.tile_q0, si.num_tiles, self.hq, self.hkv, self.d, self.scale,
                                  cfg.sliding_window, kv_scales=kv.scales[li] if kv.scales is not None else None, sink=cfg.sink_len)
            if lw.quant:
                pending = lw.quant["o"](attn, out=self.partial[:t])
                self._norm(x, lw.ln2, pending, h)
                inter = lw.quant["gate"].n
                gu = self.gate_up[:t, : 2 * inter]
                if lw.quant.get("gate_up") is not None:
                    lw.quant["gate_up"](h, out=gu)
                else:
                    lw.quant["gate"](h, out=gu[:, :inter])
                    lw.quant["up"](h, out=gu[:, inter:])
                act = ops.silu_mul(gu, out=self.act_q[:t]) if x.is_cuda else ops.silu_mul(gu)
                pending = lw.quant["down"](act, out=self.partial[:t])
                continue
            pending = self._row_parallel(attn, lw.o_w, x, 0)
            self._norm(x, lw.ln2, pending, h)
            if lw.gate_up_w is not None:
                act = self.act[:t]
                if x.is_cuda:
                    ops.gemm(h, lw.gate_up_w, epilogue="swiglu", swiglu_half=w.swiglu_half, out=act)
                else:
                    act = ops.gemm(h, lw.gate_up_w, epilogue="swiglu", swiglu_half=w.swiglu_half)
                pending = self._row_parallel(act, lw.down_w, x, 1)
            else:
                pending = self._moe(h, lw, x)
        r = si.num_logit_rows
        if pending is not None:   # fold the last partial sum into the residual before selecting rows
            x.add_(pending)
        if stage < stages - 1:
            self.comm.send(x, stage + 1)
            return None                                  # the last stage computes the logits and samples
        xl = self.x_last[:r]
        torch.index_select(x, 0, si.logit_rows[:r].long(), out=xl)
        hl = self.h_last[:r]
        self._norm(xl, w.final_norm, None, hl)
        logits = self.logits[:r]
        self._gemm(hl, w.lm_head, out=logits)
        return logits

    def _attention(self, si, kv, li, qkv, attn):
        """Rotary embedding + KV append + paged attention of one layer over the step's rows."""
        cfg = self.cfg
        t, nd = si.num_tokens, si.num_decode
        pool = kv.pools[li]
        scales = kv.scales[li] if kv.scales is not None else None
        ops.rope_kv_append(qkv, si.positions[:t], si.slots[:t], self.cos_sin, pool, self.hq, self.hkv, self.d,
                           self.rotary_dim, cfg.rotary_interleaved, kv_scales=scales)
        if nd > 0:
            ops.paged_decode(qkv[:nd], attn[:nd], pool, si.page_table[:nd], si.ctx_len[:nd], self.hq, self.hkv,
                             self.d, self.scale, self.decode_splits, self.part_o, self.part_ml, cfg.sliding_window,
                             kv_scales=scales, sink=cfg.sink_len)
        if si.num_prefill_seqs > 0 and si.verify_table is not None:
            nv = si.verify_ctx.numel()
            ops.paged_decode(qkv[nd:nd + nv], attn[nd:nd + nv], pool, si.verify_table, si.verify_ctx, self.hq, self.hkv,
                             self.d, self.scale, si.verify_splits, self.part_o, self.part_ml, cfg.sliding_window,
                             kv_scales=scales, sink=cfg.sink_len)
        elif si.num_prefill_seqs > 0:
            np_ = si.num_prefill_seqs
            ops.paged_prefill(qkv[nd:], attn[nd:], pool, si.page_table[nd:nd + np_], si.ctx_len[nd:nd + np_],
                              si.cu_q, si.tile_seq, si.tile_q0, si.num_tiles, self.hq, self.hkv, self.d, self.scale,
                              cfg.sliding_window, kv_scales=scales, sink=cfg.sink_len)

    def _forward_tp_fused(self, si: StepInputs, kv: "KVCache") -> torch.Tensor:
        """The step under fused tensor parallelism, driven op by op (the C++ executor runs the same sequence).

        The residual stream is owned by rows; every row-parallel projection ends in one exchange kernel that
        reduce-scatters the partial products, adds the owner's residual rows, applies the *next* RMSNorm and
        all-gathers the normed rows into ``h`` on every rank.  The column-parallel GEMM that follows waits for ``h``
        tile by tile inside its TMA producer."""
        cfg, w, fc = self.cfg, self.w, self.fused_comm
        t = si.num_tokens
        x, h, qkv, attn = self.x[:t], self.h[:t], self.qkv[:t], self.attn[:t]
        ops.embedding(si.token_ids[:t], w.embed, out=x)
        ops.rmsnorm(x, w.layers[0].ln1, cfg.rms_eps, out=h)       # all rows once; owners keep their rows current from here on
        ready = None
        n_layers = len(w.layers)
        for li, lw in enumerate(w.layers):
            ops.gemm(h, lw.qkv_w, bias=lw.qkv_b, out=qkv, a_ready=ready)
            self._attention(si, kv, li, qkv, attn)
            fc.row_parallel_norm(attn, lw.o_w, t, 0, lw.ln2, cfg.rms_eps)
            ready = fc.ready_ptrs(0)
            next_norm = w.layers[li + 1].ln1 if li + 1 < n_layers else w.final_norm
            if lw.gate_up_w is not None:
                act = self.act[:t]
                ops.gemm(h, lw.gate_up_w, epilogue="swiglu", swiglu_half=w.swiglu_half, out=act, a_ready=ready)
                fc.row_parallel_norm(act, lw.down_w, t, 1, next_norm, cfg.rms_eps)
            else:
                from . import moe

                moe.moe_forward_fused(self, h, lw, ready, next_norm)
            ready = fc.ready_ptrs(1)
        r = si.num_logit_rows
        fc.wait_ready(1, t)                                      # the last exchange applied the final norm
        hl = self.h_last[:r]
        torch.index_select(h, 0, si.logit_rows[:r].long(), out=hl)
        logits = self.logits[:r]
        self._gemm(hl, w.lm_head, out=logits)
        return logits

    # --------------------------------------------------------------------------------------
    def _norm(self, x, weight, delta, out):
        if x.is_cuda:
            ops.rmsnorm(x, weight, self.cfg.rms_eps, delta=delta, out=out)
        else:
            out.copy_(ops.rmsnorm(x, weight, self.cfg.rms_eps, delta=delta))

    def _gemm(self, a, wt, out, bias=None):
        if a.is_cuda:
            ops.gemm(a, wt, bias=bias, out=out)
        else:
            out.copy_(ops.gemm(a, wt, bias=bias))

    def _row_parallel(self, a, wt, x, slot=0):
        """x += a @ wt^T.  TP=1: fused residual epilogue.  TP>1: partial sum -> all-reduce -> returned as
        a pending delta that the next RMSNorm adds."""
        if self.tp == 1:
            if a.is_cuda:
                ops.gemm(a, wt, residual=x, epilogue="residual", out=x)
            else:
                x.copy_(ops.gemm(a, wt, residual=x, epilogue="residual"))
            return None
        if self.fused_comm is not None:
            # GEMM epilogue scatters partial tiles to the owner ranks; the owners reduce, add the
            # residual and write the new rows into every rank's x.  Nothing is left pending.
            self.fused_comm.row_parallel(a, wt, a.shape[0], slot)
            return None
        part = self.partial[: a.shape[0]]
        self._gemm(a, wt, out=part)
        self.comm.all_reduce(part)
        return part

    def _moe(self, h, lw, x):
        from . import moe

        return moe.moe_forward(self, h, lw, x)
