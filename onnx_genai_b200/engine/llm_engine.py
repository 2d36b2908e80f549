"""Continuous-batching engine: C++ scheduler core + fused decoder executor + device sampler.

Role of `Engine` + `ContinuousBatchManager` in the reference
(crates/onnx-genai-engine/src/engine/runtime.rs:340-1524, src/batched.rs:189-749).  One
``step()`` is:

    core.build_step  -> packed plan in pinned host memory          (C++)
    one H2D copy of the plan, CoW / swap page moves if the plan asks for them
    DecoderModel.forward over the mixed batch (decode rows + prefill chunks)
    fused sampler (or argmax when every row is greedy) -> int32 tokens
    one D2H copy of the tokens, core.commit_step -> token / finish events

Differences from the reference by design: prompts are prefilled in multi-token chunks inside the
same step as decode rows (the reference feeds one prompt token per row per step,
batched.rs:663-749), batched rows can be preempted (swap or recompute), and attention reads KV
pages in place.  Under tensor parallelism every rank runs an identical scheduler replica on the
same request stream, so no per-step control message crosses ranks.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..models.config import DecoderConfig
from ..models.decoder import DecoderModel, DecoderWeights, KVCache, StepInputs, random_weights
from ..parallel.sharding import shard_heads
from ..utils.trace import TRACER
from .core import HDR, Core, CoreConfig


@dataclass
class EngineConfig:
    model: DecoderConfig
    num_pages: int = 0                 # 0: size from free device memory
    host_allocator_plugin: str = ""    # shared library implementing the memory plugin ABI: the host swap space comes from it
    kv_max_pages: int = 0              # > num_pages (CUDA, TP=1): reserve address space for this many pages, back num_pages now
                                       # and more on demand when the scheduler runs low (the pool grows in place)
    gpu_memory_utilization: float = 0.85
    num_host_pages: int = 0
    max_seqs: int = 256
    max_tokens_per_step: int = 2048
    max_seq_len: int = 4096
    prefill_chunk: int = 2048
    token_multiple: int = 1
    policy: str = "fcfs"
    preempt: str = "recompute"
    enable_prefix_cache: bool = True
    release_window_pages: bool = True  # sliding-window models: give back the KV pages no later query can see (sinks are kept)
    kv_dtype: str = "bf16"
    decode_splits: int = 0             # 0: pick from batch shape
    sync_sampled_tokens: bool = True   # TP: broadcast rank 0's tokens so replicas cannot diverge
    max_draft_tokens: int = 0          # speculative decoding: drafts verified per sequence per step
    native_executor: bool = True       # launch the layer stack from the C++ step executor when possible
    cuda_graphs: bool = False          # replay decode-only steps (forward + sampler) from captured CUDA graphs
    allocator: object | None = None    # engine/allocator.py Allocator for KV pools and swap space (torch's allocator when None)
    max_tree_branches: int = 4         # root-to-leaf paths of a speculation tree verified per step (one forked sequence each)
    weight_offload_layers: int = 0     # keep the matrices of the last N layers in pinned host memory and stream them per step
    shard_sampling: bool = True        # TP: each rank runs lm_head + sampler for 1/tp of the rows, tokens are all-gathered
    vram_limit: str | None = None      # "8GiB" | "0.9" | "auto": cap on device bytes (weights + activations + KV pool)
    seed: int = 0


@dataclass
class RequestStats:
    arrival: float = 0.0
    first_token: float = 0.0
    finished: float = 0.0
    prompt_tokens: int = 0
    output_tokens: int = 0
    finish_reason: str | None = None


@dataclass
class StepOutput:
    events: list = field(default_factory=list)    # (seq_id, token, finish_reason | None)
    num_tokens: int = 0
    num_decode: int = 0
    num_prefill_tokens: int = 0


class LLMEngine:
    def __init__(self, cfg: EngineConfig, weights: DecoderWeights | None = None, device="cuda", tp: int = 1,
                 rank: int = 0, comm=None, pp: int = 1):
        """``tp`` > 1: this process is rank ``rank`` of a tensor-parallel group.  ``pp`` > 1 (with tp = 1): this process is
        stage ``rank`` of a pipeline over the layers -- every stage runs the same scheduler, the residual stream moves
        stage to stage by send / recv, the last stage samples and broadcasts the tokens."""
        self.cfg, self.device = cfg, torch.device(device)
        self.tp, self.rank, self.comm = tp, rank, comm
        self.pp = int(pp)
        if self.pp > 1 and (tp != 1 or comm is None or cfg.weight_offload_layers):
            raise ValueError("pipeline parallelism needs tp = 1, a communicator, and no weight paging")
        m = cfg.model
        is_cuda = self.device.type == "cuda"
        shard_rank = 0 if self.pp > 1 else rank       # a pipeline stage holds whole layers: nothing is sharded within one
        if weights is None:
            dtype = torch.bfloat16 if is_cuda else torch.float32
            weights = random_weights(m, self.device, tp, shard_rank, seed=cfg.seed, dtype=dtype)
        self.weights = weights
        max_pages_per_seq = (cfg.max_seq_len + ops.PAGE - 1) // ops.PAGE
        hs = shard_heads(m.num_heads, m.num_kv_heads, tp, shard_rank)
        max_rows = cfg.max_seqs * (1 + max(0, cfg.max_draft_tokens))
        self.model = DecoderModel(m, weights, self.device, cfg.max_tokens_per_step, max_rows, tp, shard_rank, comm)
        own_layers = None
        if self.pp > 1:
            from ..parallel.pipeline import plan_stages

            # the first stage also embeds and the last one runs the LM head: weigh them like the layers they displace
            head = 2.0 * m.vocab * m.hidden / max(1.0, 2.0 * m.hidden * (m.num_heads + 2 * m.num_kv_heads) * m.head_dim + 2.0 * m.hidden * m.hidden
                                                  + 6.0 * m.hidden * max(m.intermediate, 1))
            self.stage_plan = plan_stages(m.num_layers, self.pp, head_cost=head)
            self.model.set_pipeline(rank, self.pp, self.stage_plan.ranges)
            own_layers = range(*self.stage_plan.ranges[rank])
        # memory ledger: bytes come from the tensors that exist, the KV pool gets what the limit leaves
        from .memory import MemoryLedger, parse_limit, tensor_bytes

        tier = "vram" if is_cuda else "host"
        self.memory = MemoryLedger()
        if is_cuda and cfg.vram_limit:
            self.memory.limits["vram"] = parse_limit(cfg.vram_limit, torch.cuda.mem_get_info(self.device)[1])
        w_bytes = tensor_bytes(weights)
        self.weights_lease = self.memory.lease("weights", tier, w_bytes, m.name)
        try:
            act_bytes = max(0, tensor_bytes(self.model) - w_bytes)
        except Exception:            # accounting must never stop an engine from starting
            act_bytes = 0
        self.memory.lease("activations", tier, act_bytes, "step buffers")
        num_pages = cfg.num_pages
        if num_pages <= 0:
            kv_bytes = 1 if cfg.kv_dtype in ("fp8", "int8", "fp8_e5m2") else 2
            page_bytes = m.num_layers * len(hs.kv_heads) * 2 * ops.PAGE * m.head_dim * kv_bytes
            if is_cuda:
                free, total = torch.cuda.mem_get_info(self.device)
                budget = int(free - (1.0 - cfg.gpu_memory_utilization) * total)
                ledger_budget = self.memory.kv_budget("vram", reserve=256 << 20)   # headroom for sampler scratch and graphs
                if ledger_budget is not None:
                    budget = min(budget, ledger_budget)
                if self.comm is not None:   # every replica must agree on the pool size
                    budget = self.comm.min_int(budget)
                num_pages = max(64, budget // page_bytes)
                # no more pages than max_seqs full-length sequences can ever use
                num_pages = min(num_pages, cfg.max_seqs * max_pages_per_seq + 64)
            else:
                num_pages = min(4096, cfg.max_seqs * max_pages_per_seq + 16)
        self.num_pages = int(num_pages)
        kv_max = cfg.kv_max_pages if (is_cuda and self.tp == 1 and self.pp == 1 and cfg.kv_max_pages > self.num_pages) else 0
        from .allocator import DeferredReleaseQueue

        self.allocator = cfg.allocator
        self.release_queue = DeferredReleaseQueue()
        self.kv = KVCache(m, self.num_pages, self.device, len(hs.kv_heads), cfg.kv_dtype, max_pages=kv_max, layers=own_layers,
                          allocator=self.allocator)
        self.kv_lease = self.memory.lease("kv", tier, self.kv.mapped_bytes(), f"pages of 16 tokens, {cfg.kv_dtype}")
        self.kv_grows, self.kv_grow_error = 0, None
        self.core = Core(CoreConfig(num_pages=self.num_pages, num_host_pages=cfg.num_host_pages, max_seqs=cfg.max_seqs,
                                    max_tokens_per_step=cfg.max_tokens_per_step, max_pages_per_seq=max_pages_per_seq,
                                    prefill_chunk=cfg.prefill_chunk, token_multiple=cfg.token_multiple,
                                    policy=cfg.policy, preempt=cfg.preempt,
                                    enable_prefix_cache=cfg.enable_prefix_cache, eos_token=m.eos_token,
                                    max_draft_tokens=cfg.max_draft_tokens))
        if m.sliding_window > 0 and cfg.release_window_pages:
            self.core.set_window(m.sliding_window, m.attention_sinks)
        L = self.core.layout
        self.L = L
        self.plan_host = torch.zeros(L.total_words, dtype=torch.int32, pin_memory=is_cuda)
        self.plan_np = self.plan_host.numpy()
        self.dev_words = L.swap_out_dev      # sections after this offset cross to the device only in steps that swap pages
        self.plan_dev_full = torch.zeros(L.total_words, dtype=torch.int32, device=self.device) if is_cuda else self.plan_host
        self.plan_dev = self.plan_dev_full[: self.dev_words] if is_cuda else self.plan_host     # what every step copies
        self.status_host = torch.zeros(1, dtype=torch.int32, pin_memory=is_cuda)
        self.sampled_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=is_cuda)
        self.sampled_dev = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.sample_work = (torch.empty(max_rows * m.vocab, dtype=torch.int32, device=self.device)
                            if is_cuda else None)
        self.host_kv = None
        self.host_scales = None
        self.direct_swap = False
        self.swap_moves = 0                # page-move launches issued for swap / copy-on-write
        if cfg.num_host_pages > 0:
            own_pools, own_scales = self.kv.own_pools, self.kv.own_scales
            shape = (cfg.num_host_pages,) + tuple(own_pools[0].shape[1:])
            if cfg.host_allocator_plugin:
                # swap space from a third-party allocator (memory plugin ABI); copies to it are synchronous, as for any
                # host memory the CUDA driver has not pinned
                from ..utils.mem_plugin import PluginAllocator

                self.host_allocator = PluginAllocator(cfg.host_allocator_plugin, purpose="kv-swap")
                self.host_kv = [self.host_allocator.tensor(shape, own_pools[0].dtype) for _ in own_pools]
            else:
                self.host_kv = [torch.zeros(shape, dtype=own_pools[0].dtype, pin_memory=is_cuda) for _ in own_pools]
            try:
                self.memory.lease("kv", "host", sum(t.numel() * t.element_size() for t in self.host_kv), "swap space")
            except Exception:
                pass
            if self.kv.scales is not None:     # one-byte pages: the per-(page, head, K|V) scales travel with their page
                sshape = (cfg.num_host_pages,) + tuple(own_scales[0].shape[1:])
                self.host_scales = [torch.zeros(sshape, dtype=torch.float32, pin_memory=is_cuda and not cfg.host_allocator_plugin)
                                    for _ in own_pools]
            # Pinned host memory is addressable from the device: swap kernels on a side stream read and write it in
            # place, so a swap needs no staging buffer and never blocks the host.  Memory from an allocator plugin is
            # not pinned by the driver and keeps the synchronous copy path.
            self.direct_swap = is_cuda and not cfg.host_allocator_plugin
        if is_cuda:
            addr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=self.device)
            self._kv_bases = addr(self.kv.own_pools)
            self._scale_bases = addr(self.kv.own_scales) if self.kv.scales is not None else None
            if self.direct_swap:
                self._host_bases = addr(self.host_kv)
                self._host_scale_bases = addr(self.host_scales) if self.host_scales is not None else None
                self.swap_stream = torch.cuda.Stream(device=self.device)
        p = self.plan_dev
        S, T, MP = cfg.max_seqs, cfg.max_tokens_per_step, max_pages_per_seq
        self.si = StepInputs(
            0, 0, 0, 0, 0,
            token_ids=p[L.token_ids:L.token_ids + T], positions=p[L.positions:L.positions + T],
            slots=p[L.slots:L.slots + T], ctx_len=p[L.ctx_len:L.ctx_len + S],
            page_table=p[L.page_table:L.page_table + S * MP].view(S, MP), cu_q=p[L.cu_q:L.cu_q + S + 1],
            tile_seq=p[L.tile_seq:L.tile_seq + L.max_tiles], tile_q0=p[L.tile_q0:L.tile_q0 + L.max_tiles],
            logit_rows=p[L.logit_rows:L.logit_rows + max_rows])
        f32 = lambda off: p[off:off + max_rows].view(torch.float32)
        self.temperature, self.top_p, self.min_p, self.uniform = (f32(L.temperature), f32(L.top_p), f32(L.min_p),
                                                                  f32(L.uniform))
        self.top_k = p[L.top_k:L.top_k + max_rows]
        self.model.weight_offload_layers = cfg.weight_offload_layers if is_cuda else 0
        self.native_executor = cfg.native_executor and self.pp == 1 and self.model.bind_native(self.kv, max_pages_per_seq)
        if cfg.weight_offload_layers > 0:
            if not (self.native_executor and getattr(self.model, "weight_packs", None)):
                raise ValueError("weight_offload_layers needs the C++ step executor (CUDA, dense bf16 layers, bf16 KV pages)")
            self.memory.lease("weights", "host", self.model.paged_weight_bytes, f"{cfg.weight_offload_layers} paged layer(s)")
            slots = sum(s.numel() for s in self.model.weight_slots)
            self.weights_lease.resize(max(0, self.weights_lease.nbytes - self.model.paged_weight_bytes + slots))   # two slots stay on the device
        self.host_samplers: dict = {}     # seq id -> fn(logits_row fp32 numpy, uniform) -> token id
        self.proposers: dict = {}         # seq id -> SpeculativeProposer
        self.stats: dict[int, RequestStats] = {}
        self.steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # CUDA graphs of decode-only steps, keyed by (row bucket, KV splits, sampler kind).  A capture that
        # fails is a decline, not an error: the bucket is marked and the step runs eagerly from then on.
        self.hidden_taps: dict = {}       # seq id -> None until the request's first logits row exists, then its final hidden state
        self.graphs: dict = {}
        self.graph_replays = 0
        self.tree_groups: dict = {}         # sequence id -> ids of the forks verifying the other paths of its speculation tree
        self.tree_branches = self.tree_branch_wins = 0
        self.verify_on_decode_kernel = 0   # steps whose draft rows ran on the split-KV decode kernel
        self.graph_declines: list = []
        self.device_faults = 0            # steps that ended with a non-zero device status word

    # --------------------------------------------------------------------------------------
    def add_request(self, prompt_ids, max_new_tokens=256, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0,
                    priority=0, tenant=0, ignore_eos=False, stop_ids=()) -> int:
        sid = self.core.add_request(prompt_ids, max_new_tokens, temperature, top_k, top_p, min_p, seed, priority, tenant,
                                    ignore_eos, stop_ids)
        self.stats[sid] = RequestStats(arrival=time.perf_counter(), prompt_tokens=len(prompt_ids))
        return sid

    @property
    def has_work(self) -> bool:
        return self.core.has_work

    def _page_moves(self, hdr):
        """Copy-on-write copies, swap-outs and swap-ins of the step, in the order the scheduler decided them (a page
        freed by a swap-out can be the target of a later copy, and the target of a copy can be swapped out later in
        the same step).  On a GPU with pinned swap space every run is one kernel launch per table (KV pages, scale
        rows) over all layers on a side stream; the step's own kernels wait for that stream, the host does not."""
        L, pn = self.L, self.plan_np
        nruns = int(hdr[HDR["num_move_runs"]])
        runs = pn[L.move_runs:L.move_runs + 2 * nruns].reshape(-1, 2)
        lists = {0: (L.copy_src, L.copy_dst), 1: (L.swap_out_dev, L.swap_out_host), 2: (L.swap_in_host, L.swap_in_dev)}
        offs = {0: 0, 1: 0, 2: 0}
        kv = self.kv
        is_cuda = self.device.type == "cuda"
        fast = is_cuda and (self.direct_swap or not (hdr[HDR["num_swap_out"]] or hdr[HDR["num_swap_in"]]))
        if fast:
            if hdr[HDR["num_swap_out"]] or hdr[HDR["num_swap_in"]]:      # the swap lists sit past the per-step copy
                tail = slice(self.dev_words, L.total_words)
                self.plan_dev_full[tail].copy_(self.plan_host[tail], non_blocking=True)
                self.h2d_bytes += (L.total_words - self.dev_words) * 4
            main = torch.cuda.current_stream()
            side = self.swap_stream if self.direct_swap else main
            if side is not main:
                side.wait_stream(main)       # earlier steps wrote the pages that leave; the index lists were just copied
            page_bytes = kv.own_pools[0].stride(0) * kv.own_pools[0].element_size()
            scale_bytes = kv.own_scales[0].stride(0) * 4 if kv.scales is not None else 0
            n_host = self.cfg.num_host_pages
            with torch.cuda.stream(side):
                for kind, count in runs:
                    kind, count, o = int(kind), int(count), offs[int(kind)]
                    src_off, dst_off = lists[kind]
                    src_idx = self.plan_dev_full[src_off + o:src_off + o + count]
                    dst_idx = self.plan_dev_full[dst_off + o:dst_off + o + count]
                    if kind == 0:
                        tables = [(self._kv_bases, self._kv_bases, page_bytes), (self._scale_bases, self._scale_bases, scale_bytes)]
                        sc, dc = kv.num_pages, kv.num_pages
                    elif kind == 1:
                        tables = [(self._host_bases, self._kv_bases, page_bytes),
                                  (self._host_scale_bases, self._scale_bases, scale_bytes)]
                        sc, dc = kv.num_pages, n_host
                    else:
                        tables = [(self._kv_bases, self._host_bases, page_bytes),
                                  (self._scale_bases, self._host_scale_bases, scale_bytes)]
                        sc, dc = n_host, kv.num_pages
                    for dst_b, src_b, nbytes in tables:
                        if dst_b is None or src_b is None or nbytes == 0:
                            continue
                        ops.kv_move_pages(dst_b, src_b, len(kv.own_layers), src_idx, dst_idx, count, nbytes, sc, dc)
                        self.swap_moves += 1
                    offs[kind] += count
            if side is not main:
                main.wait_stream(side)
            return
        # CPU tensors, or swap space the device cannot address (allocator plugin): indexed copies, same order
        for kind, count in runs:
            kind, count, o = int(kind), int(count), offs[int(kind)]
            src_off, dst_off = lists[kind]
            src = torch.from_numpy(pn[src_off + o:src_off + o + count].astype(np.int64))
            dst = torch.from_numpy(pn[dst_off + o:dst_off + o + count].astype(np.int64))
            for li, pool in enumerate(kv.own_pools):             # li also indexes the swap space, which holds the own layers only
                scales = kv.own_scales[li] if kv.scales is not None else None
                if kind == 0:
                    sd, dd = src.to(self.device), dst.to(self.device)
                    pool[dd] = pool[sd]
                    if scales is not None:
                        scales[dd] = scales[sd]
                elif kind == 1:
                    sd = src.to(self.device)
                    self.host_kv[li][dst] = pool[sd].cpu()
                    if scales is not None:
                        self.host_scales[li][dst] = scales[sd].cpu()
                else:
                    dd = dst.to(self.device)
                    pool[dd] = self.host_kv[li][src].to(self.device)
                    if scales is not None:
                        scales[dd] = self.host_scales[li][src].to(self.device)
            offs[kind] += count

    def _maybe_grow_kv(self) -> None:
        """Back more KV pages when the allocator runs low and the pool has address space left.  Addresses do not move,
        so page tables, captured graphs and cached descriptors stay valid; a failure (device memory or the VRAM limit)
        ends growth for good and the scheduler falls back to preemption as with a fixed pool."""
        kv = self.kv
        if not kv.growable:
            return
        low_water = self.cfg.max_tokens_per_step // ops.PAGE + self.cfg.max_seqs
        if self.core.num_free_pages >= low_water:
            return
        before = kv.num_pages
        target = min(kv.max_pages, max(before + 2 * low_water, before + before // 2))
        old_bytes = self.kv_lease.nbytes
        try:
            self.kv_lease.resize(old_bytes // before * target)
            kv.grow(target)
        except Exception as exc:
            self.kv_lease.resize(kv.mapped_bytes())
            kv.max_pages = kv.num_pages                    # not growable any more
            self.kv_grow_error = str(exc)
        if kv.num_pages > before:
            self.core.add_pages(kv.num_pages - before)
            self.num_pages = kv.num_pages
            self.model.set_backed_pages(kv.num_pages)    # kernels bound page ids by the backed count
            self.graphs.clear()                          # captured launches carry the old bound
            self.kv_lease.resize(kv.mapped_bytes())
            self.kv_grows += 1

    def _pick_splits(self, nd: int, max_ctx: int) -> int:
        if self.cfg.decode_splits > 0:
            return self.cfg.decode_splits
        ctas = nd * self.model.hkv
        target = 2 * (ops.num_sms() if self.device.type == "cuda" else 148)
        if ctas >= target or max_ctx < 256:
            return 1
        s = 1
        while ctas * s < target and s < 32 and max_ctx // (s * 2) >= 128:
            s *= 2
        return s

    # ---- CUDA graphs for decode-only steps -------------------------------------------------
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)

    def _graph_eligible(self, si, r, hdr) -> bool:
        return (self.cfg.cuda_graphs and self.device.type == "cuda" and self.tp == 1 and self.pp == 1 and not getattr(self.model, "tap_layers", None)
                and not self.cfg.weight_offload_layers
                and si.num_prefill_seqs == 0 and si.num_tiles == 0 and si.num_decode == si.num_tokens == r and r > 0
                and r <= min(self.cfg.max_seqs, self.GRAPH_BUCKETS[-1]))

    def _graph_step(self, si, r) -> bool:
        """Run a decode-only step of r rows as a graph replay over the next row bucket.  Rows r..bucket are
        padding: token 0 at position 0, no KV slot, context length 0 (idle in attention), greedy."""
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= r)
        if bucket > self.cfg.max_seqs or bucket > self.cfg.max_tokens_per_step:
            return False
        L, pn = self.L, self.plan_np
        temps = pn[L.temperature:L.temperature + r].view(np.float32)
        greedy = bool((temps <= 0).all())
        key = (bucket, self.model.decode_splits, greedy)
        entry = self.graphs.get(key)
        if entry is False:
            return False
        if bucket > r:
            pn[L.token_ids + r:L.token_ids + bucket] = 0
            pn[L.positions + r:L.positions + bucket] = 0
            pn[L.slots + r:L.slots + bucket] = -1
            pn[L.ctx_len + r:L.ctx_len + bucket] = 0
            pn[L.logit_rows + r:L.logit_rows + bucket] = np.arange(r, bucket, dtype=np.int32)
            pn[L.temperature + r:L.temperature + bucket] = 0          # 0.0f: padded rows take the argmax path
            self.plan_dev.copy_(self.plan_host[: self.dev_words], non_blocking=True)
            self.h2d_bytes += self.dev_words * 4
        saved = (si.num_tokens, si.num_decode, si.num_logit_rows)
        si.num_tokens = si.num_decode = si.num_logit_rows = bucket

        def body():
            logits = self.model.forward(si, self.kv)
            if greedy:
                ops.argmax(logits, out=self.sampled_dev[:bucket])
            else:
                ops.sample(logits, self.temperature[:bucket], self.top_k[:bucket], self.top_p[:bucket], self.min_p[:bucket],
                           self.uniform[:bucket], work=self.sample_work, out=self.sampled_dev[:bucket])

        try:
            if entry is None:
                body()                                   # eager warm-up: one-time setup must not land in the capture
                torch.cuda.current_stream().synchronize()
                g = torch.cuda.CUDAGraph()
                try:
                    with torch.cuda.graph(g, capture_error_mode="thread_local"):
                        body()
                except Exception as exc:                 # decline: remember why, fall back to eager for this bucket
                    self.graphs[key] = False
                    self.graph_declines.append((key, repr(exc)))
                    return False
                self.graphs[key] = g
                # the warm-up already produced this step's tokens
                return True
            entry.replay()
            self.graph_replays += 1
            ops.launch_counts["graph_replay"] += 1
            return True
        finally:
            si.num_tokens, si.num_decode, si.num_logit_rows = saved

    # ---- speculative verification rows on the split-KV decode kernel ------------------------------
    VERIFY_MIN_CTX = 2048

    def _plan_verify_rows(self, si) -> None:
        """When every non-decode sequence of the step is a short run of draft rows over a long context, describe
        each query row as a decode row (own context length, the sequence's page-table row).  The prefill kernel
        gives one CTA per (64-row tile, head) the whole context to walk; the decode kernel splits the context
        across CTAs, which is what a 32k-token verification needs.  Such a step is driven from Python even when the
        C++ step executor is bound (it has no per-row page tables)."""
        si.verify_table = si.verify_ctx = None
        si.force_python = False
        np_ = si.num_prefill_seqs
        if np_ == 0 or self.device.type != "cuda" or si.max_ctx < self.VERIFY_MIN_CTX:
            return
        nd, L, pn = si.num_decode, self.L, self.plan_np
        cu = pn[L.cu_q:L.cu_q + np_ + 1].astype(np.int64)
        qlen = cu[1:] - cu[:-1]
        if qlen.max() > max(8, self.cfg.max_draft_tokens + 1):
            return                                        # a real prefill chunk is in the step
        # (also taken by a draft engine: after a rejection it is fed one or two corrected tokens over the whole context)
        si.force_python = bool(self.native_executor)      # the C++ step executor has no per-row page tables
        ctx_end = pn[L.ctx_len + nd:L.ctx_len + nd + np_].astype(np.int64)
        seq_of_row = np.repeat(np.arange(np_), qlen)
        within = np.arange(int(cu[-1])) - np.repeat(cu[:-1], qlen)
        ctx_rows = (ctx_end[seq_of_row] - qlen[seq_of_row] + within + 1).astype(np.int32)
        rows = int(cu[-1])
        if rows > self.sampled_dev.numel():
            return
        idx = torch.from_numpy(seq_of_row.astype(np.int64)).to(self.device, non_blocking=True)
        si.verify_table = si.page_table[nd:nd + np_].index_select(0, idx).contiguous()
        si.verify_ctx = torch.from_numpy(ctx_rows).to(self.device, non_blocking=True)
        splits = self._pick_splits(rows, int(si.max_ctx))
        if self.model.ensure_split_scratch(splits):
            self.graphs.clear()
        si.verify_splits = splits
        self.verify_on_decode_kernel += 1

    # ---- speculation trees verified as forked branches --------------------------------------------
    def _fork_tree_branches(self, sid, tree) -> None:
        """Verify a speculation tree with the linear machinery: the sequence drafts the tree's first root-to-leaf path
        and every other path is drafted by a copy-on-write fork of the sequence (the context's pages are shared; a
        branch writes only its own tail).  All branches run in the same step; `_settle_tree_branches` keeps the one that
        got furthest.  Shared prefixes of paths are recomputed per branch -- what a tree-masked attention pass would
        save -- but rows of a step are cheap next to the weights they share.  Greedy requests only: branches of a
        sampled request would draw different tokens for the same position."""
        if tree is None or len(tree) == 0 or sid in self.tree_groups:
            return
        if self.core.seq_computed(sid) < self.core.seq_len(sid) - 1:
            return                                            # still prefilling: a fork would repeat the prefill
        k = self.cfg.max_draft_tokens
        paths = []
        for leaf in tree.leaves():
            toks = [tree.nodes[i].token for i in tree.path_to(leaf)][:k]
            if toks and toks not in paths:
                paths.append(toks)
        paths.sort(key=len, reverse=True)
        room = max(0, self.cfg.max_seqs - (self.core.num_running + self.core.num_waiting + self.core.num_swapped))
        paths = paths[: max(1, min(self.cfg.max_tree_branches, 1 + room))]
        self.core.set_draft(sid, np.asarray(paths[0], dtype=np.int32))
        forks = []
        for path in paths[1:]:
            fid = self.core.fork(sid)
            if fid < 0:
                break
            self.core.set_draft(fid, np.asarray(path, dtype=np.int32))
            forks.append(fid)
        if forks:
            self.tree_groups[sid] = forks
            self.tree_branches += len(forks)

    def _settle_tree_branches(self, events):
        """After the commit: per tree, the branch that committed the most tokens becomes the sequence (its state moves
        under the caller's id), the other branches are released, and only the winner's events are reported."""
        committed: dict = {}
        for ev_sid, _tok, _fin in events:
            committed[ev_sid] = committed.get(ev_sid, 0) + 1
        relabel, dropped = {}, set()
        for sid, forks in self.tree_groups.items():
            members = [sid] + forks
            if not any(m in committed for m in members):
                continue                                      # the tree's rows were not scheduled this step: settle at the next
            winner = max(members, key=lambda m: (committed.get(m, 0), m == sid))
            if winner != sid:
                self.core.swap_state(sid, winner)
                self.tree_branch_wins += 1
            relabel[winner] = sid
            dropped.update(m for m in members if m != winner)
            for f in forks:                                   # after the swap the fork ids hold the losing states
                self.core.cancel(f)
                self.core.release(f)
            self.tree_groups[sid] = None
        self.tree_groups = {k: v for k, v in self.tree_groups.items() if v is not None}
        out = []
        for ev_sid, tok, fin in events:
            if ev_sid in relabel:
                out.append((relabel[ev_sid], tok, fin))
            elif ev_sid not in dropped:
                out.append((ev_sid, tok, fin))
        return out

    # ---- TP: rows of the logits/sampling stage split over the ranks -------------------------------
    def _shard_rows(self, r: int) -> bool:
        """With a replicated lm_head every rank would compute and sample all r rows.  Instead rank k takes rows
        [k*chunk, (k+1)*chunk): its lm_head GEMM and sampler see 1/tp of the rows and one all-gather of the token
        ids (4 bytes per row) replaces the broadcast that kept replicas in step.  Steps whose logits are needed on
        the host (custom samplers, log-probabilities, embeddings, speculative verification) keep all rows."""
        return (self.tp > 1 and self.cfg.shard_sampling and r >= self.tp
                and not self.host_samplers and not self.hidden_taps and self.cfg.max_draft_tokens == 0)

    def forward_and_sample_sharded(self, si, r: int, greedy: bool) -> None:
        """Run the step with this rank's share of the sampling rows; leaves all r token ids in sampled_dev[:r]."""
        tp, rank = self.tp, self.rank
        chunk = (r + tp - 1) // tp
        r0 = min(r, rank * chunk)
        n_loc = max(0, min(r, r0 + chunk) - r0)
        if getattr(self, "_shard_buf", None) is None or self._shard_buf.numel() < chunk:
            cap = (self.sampled_dev.numel() + tp - 1) // tp + 1
            self._shard_buf = torch.zeros(cap, dtype=torch.int32, device=self.device)
            self._gather_buf = torch.zeros(cap * tp, dtype=torch.int32, device=self.device)
        saved_rows, saved_n = si.logit_rows, si.num_logit_rows
        # a rank whose share is empty (r not a multiple of tp) still runs the layers; it samples one throw-away row
        lo = r0 if n_loc > 0 else 0
        n_run = max(n_loc, 1)
        si.logit_rows, si.num_logit_rows = saved_rows[lo:], n_run
        try:
            logits = self.model.forward(si, self.kv)
        finally:
            si.logit_rows, si.num_logit_rows = saved_rows, saved_n
        out = self._shard_buf[:n_run]
        if self.device.type != "cuda":
            toks = (ops.argmax(logits) if greedy else
                    ops.sample(logits, self.temperature[lo:lo + n_run], self.top_k[lo:lo + n_run], self.top_p[lo:lo + n_run],
                               self.min_p[lo:lo + n_run], self.uniform[lo:lo + n_run]))
            out.copy_(toks)
        elif greedy:
            ops.argmax(logits, out=out)
        else:
            ops.sample(logits, self.temperature[lo:lo + n_run], self.top_k[lo:lo + n_run], self.top_p[lo:lo + n_run],
                       self.min_p[lo:lo + n_run], self.uniform[lo:lo + n_run], work=self.sample_work, out=out)
        self.comm.all_gather(self._gather_buf[: tp * chunk], self._shard_buf[:chunk])
        self.sampled_dev[:r].copy_(self._gather_buf[:r])

    def _finish_device_step(self, r: int) -> None:
        """The step's one synchronisation: the sampled tokens and the device status word cross to pinned host memory
        behind the step's kernels, the host waits once, and a non-zero word (a bounded wait that ran out, a bad page or
        token id, a peer that never signalled) becomes an exception *before* any token is committed -- the caller
        fails the in-flight requests instead of streaming garbage."""
        if r > 0:
            self.sampled_host[:r].copy_(self.sampled_dev[:r], non_blocking=True)
            self.d2h_bytes += r * 4
        self.status_host.copy_(ops.status_word(self.device), non_blocking=True)
        self.d2h_bytes += 4
        torch.cuda.current_stream().synchronize()
        v = int(self.status_host[0])
        if v:
            ops.status_word(self.device).zero_()
            self.device_faults += 1
            self.graphs.clear()
            fc = getattr(self.model, "fused_comm", None)
            if fc is not None and (v & (ops.STATUS_PEER_TIMEOUT | ops.STATUS_WAIT_TIMEOUT)):
                fc.poison("device status word %d" % v)      # its counters are part-consumed: the group must be rebuilt
            raise ops.status_error(v)

    def step(self) -> StepOutput:
        """Schedule, run and commit one engine step."""
        tracing = TRACER.enabled or TRACER.want_gpu or TRACER.nvtx is not None
        if not tracing:
            return self._step()
        with TRACER.span("loop.step"):        # with its parts (loop.schedule / loop.forward / loop.commit) recorded inside
            return self._step(True)

    def _step(self, tracing: bool = False) -> StepOutput:
        out = StepOutput()
        t_begin = time.perf_counter() if tracing else 0.0
        batches: dict = {}
        for sid, proposer in list(self.proposers.items()):   # speculative drafts for the coming step
            toks = self.core.seq_tokens(sid) if self.core.seq_len(sid) > 0 else None
            if toks is None:
                continue
            if getattr(proposer, "wants_sequence", False):   # proposers that read this sequence's KV pages
                proposer.bind(self, sid)
            if hasattr(proposer, "propose_tree"):            # a tree of candidates: one forked sequence per root-to-leaf path
                self._fork_tree_branches(sid, proposer.propose_tree(toks, self.cfg.max_draft_tokens))
                continue
            key = getattr(proposer, "batch_key", None)
            if key is not None:                              # proposers that can answer together (one draft engine)
                batches.setdefault(key, []).append((sid, proposer, toks))
                continue
            draft = proposer.propose(toks, self.cfg.max_draft_tokens)
            if len(draft):
                self.core.set_draft(sid, draft)
        for items in batches.values():
            drafts = type(items[0][1]).propose_many([p for _, p, _ in items], [t for _, _, t in items], self.cfg.max_draft_tokens)
            for (sid, _, _), draft in zip(items, drafts):
                if len(draft):
                    self.core.set_draft(sid, draft)
        self._maybe_grow_kv()
        t = self.core.build_step(self.plan_host.data_ptr())
        if tracing:
            t_sched = time.perf_counter()
            TRACER.add("loop.schedule", t_begin, t_sched)
        if t <= 0:
            return out
        hdr = self.plan_np[:32]
        si = self.si
        si.num_tokens, si.num_decode = t, int(hdr[HDR["num_decode"]])
        si.num_prefill_seqs, si.num_tiles = int(hdr[HDR["num_prefill_seqs"]]), int(hdr[HDR["num_tiles"]])
        si.num_logit_rows, si.max_ctx = int(hdr[HDR["num_logit_rows"]]), int(hdr[HDR["max_ctx"]])
        r = si.num_logit_rows
        if self.device.type == "cuda":
            self.plan_dev.copy_(self.plan_host[: self.dev_words], non_blocking=True)
            self.h2d_bytes += self.dev_words * 4
        if hdr[HDR["num_move_runs"]]:
            self._page_moves(hdr)
        self._plan_verify_rows(si)
        if si.num_decode:
            splits = self._pick_splits(si.num_decode, si.max_ctx)
            if splits != self.model.decode_splits and self.model.set_decode_splits(splits):
                self.graphs.clear()          # split scratch was reallocated: captured pointers are stale
        graphed = self._graph_step(si, r) if self._graph_eligible(si, r, hdr) else False
        sharded = (not graphed) and self._shard_rows(r)
        if graphed:
            logits = self.model.logits[:r]
        elif sharded:
            logits = None
        else:
            logits = self.model.forward(si, self.kv)
        if r > 0:
            temps = self.plan_np[self.L.temperature:self.L.temperature + r].view(np.float32)
            if graphed:
                self._finish_device_step(r)
            elif sharded:
                self.forward_and_sample_sharded(si, r, bool((temps <= 0).all()))
                if self.device.type == "cuda":
                    self._finish_device_step(r)
                else:
                    self.sampled_host[:r].copy_(self.sampled_dev[:r])
            elif self.device.type == "cuda":
                if logits is None:
                    pass                                      # an earlier pipeline stage: the last stage samples
                elif (temps <= 0).all():
                    ops.argmax(logits, out=self.sampled_dev[:r])
                else:
                    ops.sample(logits, self.temperature[:r], self.top_k[:r], self.top_p[:r], self.min_p[:r],
                               self.uniform[:r], work=self.sample_work, out=self.sampled_dev[:r])
                if self.tp > 1 and self.cfg.sync_sampled_tokens:
                    self.comm.broadcast(self.sampled_dev[:r], src=0)
                if self.pp > 1:
                    self.comm.broadcast(self.sampled_dev[:r], src=self.pp - 1)
                self._finish_device_step(r)
            else:
                if logits is None:
                    pass
                elif (temps <= 0).all():
                    self.sampled_host[:r] = ops.argmax(logits)
                else:
                    self.sampled_host[:r] = ops.sample(logits, self.temperature[:r], self.top_k[:r], self.top_p[:r], self.min_p[:r],
                                                       self.uniform[:r])
                if self.pp > 1:
                    self.comm.broadcast(self.sampled_host[:r], src=self.pp - 1)
        elif self.device.type == "cuda":
            self._finish_device_step(0)
        if tracing:                       # launches of the forward pass and the sampler, and the read-back of the sampled tokens
            t_fwd = time.perf_counter()
            TRACER.add("loop.forward", t_sched, t_fwd)
        if self.hidden_taps and r > 0:
            # embeddings: the final-normed hidden state of a tapped request's last prompt token
            seq_of_row = self.plan_np[self.L.logit_seq:self.L.logit_seq + r]
            for row in range(r):
                key = int(seq_of_row[row])
                if key in self.hidden_taps and self.hidden_taps[key] is None:
                    self.hidden_taps[key] = self.model.h_last[row].float().cpu().numpy().copy()
        if self.host_samplers and r > 0:
            # rows whose request cannot use the device sampler: logits cross to the host, the request's
            # processor chain and sampler pick the token, and the device's choice for that row is replaced
            seq_of_row = self.plan_np[self.L.logit_seq:self.L.logit_seq + r]
            unis = self.plan_np[self.L.uniform:self.L.uniform + r].view(np.float32)
            for row in range(r):
                fn = self.host_samplers.get(int(seq_of_row[row]))
                if fn is not None:
                    row_logits = logits[row].float().cpu().numpy()
                    self.d2h_bytes += row_logits.nbytes
                    self.sampled_host[row] = int(fn(row_logits, float(unis[row])))
        events = self.core.commit_step(self.sampled_host.data_ptr(), r)
        if self.tree_groups:
            events = self._settle_tree_branches(events)
        if r > 0 and any(getattr(p, "wants_hidden", False) for p in self.proposers.values()):
            # proposers that draft from the target's hidden state get the row that produced the last committed token:
            # a sequence's rows are consecutive, and it committed (accepted drafts + 1) tokens
            seq_of_row = self.plan_np[self.L.logit_seq:self.L.logit_seq + r]
            first, committed = {}, {}
            for row in range(r):
                first.setdefault(int(seq_of_row[row]), row)
            for sid, _tok, _fin in events:
                committed[sid] = committed.get(sid, 0) + 1
            for sid, proposer in self.proposers.items():
                key = sid & 0x7FFFFFFF                       # the plan carries sequence ids as int32
                if getattr(proposer, "wants_hidden", False) and key in first and committed.get(sid):
                    row = first[key] + committed[sid] - 1
                    if getattr(proposer, "tap_layers", None):
                        proposer.observe(self.model.h_last[row].clone(), {l: self.model.taps[l][row].clone() for l in proposer.tap_layers})
                    else:
                        proposer.observe(self.model.h_last[row].clone())
        now = time.perf_counter()
        for sid, tok, fin in events:
            st = self.stats.get(sid)
            if st is None:
                continue
            st.output_tokens += 1
            if st.output_tokens == 1:
                st.first_token = now
            if fin is not None:
                st.finished, st.finish_reason = now, fin
        self.steps += 1
        if tracing:
            TRACER.add("loop.commit", t_fwd, time.perf_counter())
        out.events, out.num_tokens, out.num_decode = events, t, si.num_decode
        out.num_prefill_tokens = int(hdr[HDR["num_prefill_tokens"]])
        return out

    def close(self) -> dict:
        """Give the KV pools back to the engine's allocator.  The releases are parked behind an event on the current
        stream (steps still in flight may touch the pages) and completed once it has passed; returns the queue's
        figures.  The engine must not step afterwards."""
        allocs = self.kv.allocations()
        stream = torch.cuda.current_stream() if self.device.type == "cuda" else None
        self.kv.pools = [None] * len(self.kv.pools)
        if self.kv.scales is not None:
            self.kv.scales = [None] * len(self.kv.scales)
        for a in allocs:
            self.release_queue.enqueue(a, stream, "engine closed")
        self.release_queue.flush()
        self.kv_lease.release()
        return self.release_queue.stats()

    # --------------------------------------------------------------------------------------
    def generate(self, prompts, max_new_tokens=64, **sampling):
        """Run a batch of token-id prompts to completion; returns the generated ids per prompt."""
        ids = [self.add_request(p, max_new_tokens, **sampling) for p in prompts]
        outs = {i: [] for i in ids}
        done = set()
        while len(done) < len(ids) and self.core.has_work:
            for sid, tok, fin in self.step().events:
                if sid in outs:
                    outs[sid].append(tok)
                    if fin is not None:
                        done.add(sid)
        for sid in ids:
            self.core.release(sid)
        return [outs[i] for i in ids]

    def check_device_status(self):
        if self.device.type == "cuda":
            ops.check_status()
