"""Fused ops of the decoder step.

Each function takes torch tensors.  CUDA tensors run the hand-written sm_100a kernels from
``libogb_cuda.so`` (a missing library is an error, never a silent fallback); fp32 CPU tensors run
the C++ kernels of :mod:`onnx_genai_b200.ops.cpu` and other CPU tensors the PyTorch statements in
:mod:`onnx_genai_b200.ops.reference`, which are also the oracle the GPU tests compare against.  Launch counters per op (``launch_counts``) let callers and tests
prove which path ran, like the reference's dispatch hit counters (dispatch_manifest.toml:1-35).
"""
from __future__ import annotations

import collections
import math
import os

import torch

from . import _native, cpu, reference

PAGE = reference.PAGE


def _cpu_native(t) -> bool:
    """True when a CPU tensor should go to the C++ kernels (fp32 and the library is built)."""
    return t.dtype == torch.float32 and cpu.available()

launch_counts: collections.Counter = collections.Counter()
_status_words: dict[int, torch.Tensor] = {}

STATUS_WAIT_TIMEOUT = 1
STATUS_INDEX_OUT_OF_RANGE = 2
STATUS_BAD_ARGUMENT = 4
STATUS_PEER_TIMEOUT = 8


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word kernels OR error bits into (wait timeout, index out of range...)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_words[idx] = w
    return w


def status_error(v: int) -> "_native.KernelError":
    """The exception for a non-zero status word, with its bits decoded."""
    names = [n for b, n in ((1, "wait timeout"), (2, "index out of range"), (4, "bad argument"),
                            (8, "peer wait timeout")) if v & b]
    return _native.KernelError("device status word = %d (%s)" % (v, ", ".join(names)))


def check_status(reset: bool = True) -> None:
    """Synchronising read of the status word; raises with the decoded bits when non-zero."""
    w = status_word()
    v = int(w.item())
    if v:
        if reset:
            w.zero_()
        raise status_error(v)


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def backed_pages(pool) -> int:
    """Pages of a KV pool that kernels may touch.  A growable pool is a view over a reserved address range whose tail
    is not mapped yet; its owner records the mapped count on the tensor (``pool.backed_pages``) and every kernel
    bounds page ids and slots by it, so an id inside the reserve but beyond the backing raises the status bit
    instead of reaching unmapped memory."""
    return int(getattr(pool, "backed_pages", pool.shape[0]))


# ------------------------------------------------------------------------------------------
# per-op device timing (stage profiler: role of ONNX_GENAI_PROFILE / prof_span! in the reference,
# crates/onnx-genai-ort/src/profile.rs:1-52).  Disabled path = one global load.
# ------------------------------------------------------------------------------------------
_PROFILE: list | None = None


def profile_start() -> None:
    global _PROFILE
    _PROFILE = []


def profile_stop() -> dict:
    """Stops profiling; returns {op: (total_ms, calls)} measured with CUDA events."""
    global _PROFILE
    rec, _PROFILE = _PROFILE or [], None
    torch.cuda.synchronize()
    agg: dict = {}
    for name, e0, e1 in rec:
        t, c = agg.get(name, (0.0, 0))
        agg[name] = (t + e0.elapsed_time(e1), c + 1)
    return agg


def _timed(name):
    def deco(fn):
        import functools

        @functools.wraps(fn)
        def wrapper(*a, **kw):
            if _PROFILE is None:
                return fn(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            tag = name
            if name == "gemm":
                tag = "gemm[%s N=%d K=%d]" % (kw.get("epilogue", "none"), a[1].shape[0], a[1].shape[1])
            _PROFILE.append((tag, e0, e1))
            return out

        return wrapper

    return deco


class timed_region:
    """``with ops.timed_region("name"):`` records a CUDA-event pair when the op profiler is on."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _PROFILE is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _PROFILE is not None and hasattr(self, "e0"):
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _PROFILE.append((self.name, self.e0, e1))
        return False


def num_sms() -> int:
    return _native.load().ogb_num_sms()


# ------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------
_EPI = {"none": 0, "residual": 1, "swiglu": 2}
_BASELINE = False


def set_baseline(on: bool) -> None:
    """Route GEMMs to the library path (torch.matmul -> cuBLAS) with unfused epilogues.

    This is the labelled same-machine *baseline* the hand-written kernels are compared with;
    it is never selected implicitly.
    """
    global _BASELINE
    _BASELINE = bool(on)


def set_stream_k(on: bool) -> bool:
    """Switch the stream-K work decomposition of the GEMM kernel on or off (it is on by default); returns the old
    setting.  With it, the k-block iterations of all output tiles are cut into one equal range per SM, so a tile count
    that is not a multiple of the SM count no longer leaves SMs idle in the last wave."""
    return bool(_native.load().ogb_gemm_set_stream_k(1 if on else 0))


def set_tp_pdl(on: bool) -> bool:
    """Programmatic dependent launch along scatter GEMM -> exchange kernel -> consuming GEMM of the tensor-parallel path (off by
    default; ``OGB_TP_PDL=1`` enables it at start-up).  Returns the old setting."""
    return bool(_native.load().ogb_tp_set_pdl(1 if on else 0))


def set_e4m3_mma(mode: int) -> int:
    """Pick the decode kernel for e4m3 KV pages (query groups of at most 8 heads): 2 = tcgen05 kernel that feeds the raw
    bytes to the tensor cores (default), 1 = the ``mma.sync`` e4m3 kernel, 0 = the kernel that expands pages to bf16 in
    shared memory first.  Returns the old setting."""
    return int(_native.load().ogb_attn_set_e4m3_mma(int(mode)))


def _baseline_gemm(a, w, bias, residual, epilogue, out, out_f32, swiglu_half):
    y = torch.matmul(a, w.t())
    launch_counts["baseline_cublas_gemm"] += 1
    if bias is not None:
        y = y + bias
    if epilogue == "residual":
        y = y + residual
    elif epilogue == "swiglu":
        half = swiglu_half or 128
        m, n = y.shape
        y4 = y.view(m, n // (2 * half), 2, half)
        y = (torch.nn.functional.silu(y4[:, :, 0, :]) * y4[:, :, 1, :]).reshape(m, n // 2)
    if out_f32:
        y = y.float()
    if out is not None:
        out.copy_(y)
        return out
    return y


@_timed("gemm")
def gemm(a, w, bias=None, residual=None, epilogue="none", out=None, out_f32=False, bn=0, swiglu_half=None, a_ready=None):
    """out[M,N] = a[M,K] @ w[N,K]^T (+bias)(+residual) or SwiGLU over a :func:`pack_gate_up` weight.

    For ``epilogue="swiglu"`` ``w`` must have been packed with half-width ``swiglu_half`` and the
    kernel tile width is ``2*swiglu_half``; the output is [M, N/2].

    ``a_ready`` = (address of per-128-row-tile ready counters, address of a zeroed word, wait limit in ns): the rows of
    ``a`` are being delivered by other GPUs (a tensor-parallel exchange bumps a tile's counter once per 8 rows); the
    kernel's TMA producer waits for each tile before loading it and the last CTA clears the counters.
    """
    m, k = a.shape
    n = w.shape[0]
    if _BASELINE and a.is_cuda:
        return _baseline_gemm(a, w, bias, residual, epilogue, out, out_f32, swiglu_half)
    if not a.is_cuda:
        if epilogue == "swiglu":
            return reference.swiglu_packed(a, w, swiglu_half or 128)
        return reference.gemm(a, w, bias, residual, epilogue, torch.float32 if out_f32 else None)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    lib = _native.load()
    if epilogue == "swiglu":
        bn = 2 * (swiglu_half or 128)
        n_out = n // 2
    else:
        n_out = n
    if out is None:
        out = torch.empty(m, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    c_bf16 = 0 if out_f32 else out.data_ptr()
    c_f32 = out.data_ptr() if out_f32 else 0
    if a_ready is not None:
        rc = lib.ogb_gemm_bf16_wait(a.data_ptr(), w.data_ptr(), c_bf16, _ptr(bias), _ptr(residual), c_f32, m, n, k,
                                    a.stride(0), w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                                    _EPI[epilogue], bn, a_ready[0], a_ready[1], a_ready[2], status_word().data_ptr(), _stream())
    else:
        rc = lib.ogb_gemm_bf16(a.data_ptr(), w.data_ptr(), c_bf16, _ptr(bias), _ptr(residual), c_f32, m, n, k,
                               a.stride(0), w.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                               _EPI[epilogue], bn, status_word().data_ptr(), _stream())
    _native.check(rc, "ogb_gemm_bf16")
    launch_counts["gemm_bf16_tcgen05"] += 1
    return out


pack_gate_up = reference.pack_gate_up


# ------------------------------------------------------------------------------------------
# glue
# ------------------------------------------------------------------------------------------
@_timed("rmsnorm")
def rmsnorm(x, weight, eps, delta=None, out=None):
    """Returns normed x; with ``delta`` the residual x is updated in place first (x += delta)."""
    if not x.is_cuda:
        if _cpu_native(x):
            y, new_x = cpu.rmsnorm(x, weight, eps, delta)
        else:
            y, new_x = reference.rmsnorm(x, weight, eps, delta)
        if delta is not None:
            x.copy_(new_x)
        return y
    rows, hidden = x.shape
    if out is None:
        out = torch.empty(rows, hidden, dtype=x.dtype, device=x.device)
    rc = _native.load().ogb_rmsnorm_bf16(x.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), rows, hidden,
                                         x.stride(0), out.stride(0), float(eps), _stream())
    _native.check(rc, "ogb_rmsnorm_bf16")
    launch_counts["rmsnorm"] += 1
    return out


@_timed("embedding")
def embedding(ids, table, out=None):
    if not table.is_cuda:
        return table[ids.long()]
    t = ids.numel()
    vocab, hidden = table.shape
    if out is None:
        out = torch.empty(t, hidden, dtype=table.dtype, device=table.device)
    rc = _native.load().ogb_embedding_bf16(ids.data_ptr(), table.data_ptr(), out.data_ptr(), t, hidden, vocab,
                                           status_word().data_ptr(), _stream())
    _native.check(rc, "ogb_embedding_bf16")
    launch_counts["embedding"] += 1
    return out


@_timed("silu_mul")
def silu_mul(gate_up, out=None):
    if not gate_up.is_cuda:
        return cpu.silu_mul(gate_up) if _cpu_native(gate_up) else reference.silu_mul(gate_up)
    rows, two_inter = gate_up.shape
    if out is None:
        out = torch.empty(rows, two_inter // 2, dtype=gate_up.dtype, device=gate_up.device)
    rc = _native.load().ogb_silu_mul_bf16(gate_up.data_ptr(), out.data_ptr(), rows, two_inter // 2, _stream())
    _native.check(rc, "ogb_silu_mul_bf16")
    launch_counts["silu_mul"] += 1
    return out


@_timed("rope_kv_append")
def kv_format(pool) -> int:
    """One-byte page pools say their format by dtype: uint8 holds e4m3 bit patterns (0), int8 holds symmetric int8 (1),
    float8_e5m2 holds e5m2 (2)."""
    return 1 if pool.dtype == torch.int8 else (2 if pool.dtype == torch.float8_e5m2 else 0)


def rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim=None, interleaved=False,
                   kv_scales=None):
    """Rotate q,k in place inside qkv and append k,v to the paged pool (bf16; with kv_scales e4m3 or int8 by the pool's dtype)."""
    rotary_dim = rotary_dim or d
    if not qkv.is_cuda:
        if kv_scales is not None:
            return reference.rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim, interleaved, kv_scales)
        if _cpu_native(qkv) and qkv.is_contiguous() and pool.dtype == torch.float32 and pool.is_contiguous():
            return cpu.rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim, interleaved)
        return reference.rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim, interleaved)
    t = qkv.shape[0]
    assert qkv.is_contiguous() and positions.dtype == torch.int32 and slots.dtype == torch.int32
    num_slots = backed_pages(pool) * PAGE
    lib = _native.load()
    if kv_scales is None:
        rc = lib.ogb_rope_kv_append_bf16(qkv.data_ptr(), positions.data_ptr(), slots.data_ptr(), cos_sin.data_ptr(),
                                         pool.data_ptr(), t, hq, hkv, d, rotary_dim, int(interleaved), PAGE, num_slots,
                                         cos_sin.shape[0], status_word().data_ptr(), _stream())
    else:
        rc = lib.ogb_rope_kv_append_q8(qkv.data_ptr(), positions.data_ptr(), slots.data_ptr(), cos_sin.data_ptr(),
                                       pool.data_ptr(), kv_scales.data_ptr(), kv_format(pool), t, hq, hkv, d, rotary_dim,
                                       int(interleaved), PAGE, num_slots, cos_sin.shape[0],
                                       status_word().data_ptr(), _stream())
    _native.check(rc, "ogb_rope_kv_append")
    launch_counts["rope_kv_append"] += 1
    return qkv


# ------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------
# OGB_PREFILL_TC=0 keeps prefill attention on the mma.sync kernel (comparison runs); default is the tcgen05 kernel
PREFILL_TC = os.environ.get("OGB_PREFILL_TC", "1") != "0"


def prefill_tiles(q_lens, block_m=64):
    """Host-side tile list for the prefill kernel: (tile_seq, tile_q0) int32 lists."""
    seqs, q0s = [], []
    for s, n in enumerate(q_lens):
        for q0 in range(0, int(n), block_m):
            seqs.append(s)
            q0s.append(q0)
    return seqs, q0s


@_timed("paged_prefill")
def paged_prefill(q, out, pool, page_table, ctx_len, cu_q, tile_seq, tile_q0, num_tiles, hq, hkv, d, scale=None,
                  window=0, kv_scales=None, sink=0):
    """Causal varlen GQA over paged KV for chunks of new tokens.  q: packed qkv rows (first hq*d cols).
    ``kv_scales`` selects the e4m3 page kernels."""
    scale = scale or 1.0 / math.sqrt(d)
    if not q.is_cuda:
        if kv_scales is None and _cpu_native(q) and pool.dtype == torch.float32 and pool.is_contiguous():
            out.copy_(cpu.paged_attention(q, pool, page_table, ctx_len, cu_q, hq, hkv, d, scale, window, sink))
            return out
        out.copy_(reference.paged_attention(q, pool, page_table, ctx_len, cu_q, hq, hkv, d, scale, window, kv_scales, sink))
        return out
    if kv_scales is not None:
        rc = _native.load().ogb_paged_prefill_q8(
            q.data_ptr(), out.data_ptr(), pool.data_ptr(), kv_scales.data_ptr(), kv_format(pool), page_table.data_ptr(), ctx_len.data_ptr(),
            cu_q.data_ptr(), tile_seq.data_ptr(), tile_q0.data_ptr(), int(num_tiles), ctx_len.numel(), page_table.shape[1],
            backed_pages(pool), hq, hkv, d, q.stride(0), out.stride(0), float(scale), int(window), int(sink), status_word().data_ptr(),
            _stream())
        _native.check(rc, "ogb_paged_prefill_q8")
        launch_counts["paged_prefill_fp8"] += 1
        return out
    if PREFILL_TC and d in (64, 128) and out.stride(0) % 8 == 0:
        # tcgen05 / TMEM kernel: S and O accumulators in tensor memory, K/V pages fed by TMA
        rc = _native.load().ogb_paged_prefill_tc_bf16(
            q.data_ptr(), out.data_ptr(), pool.data_ptr(), page_table.data_ptr(), ctx_len.data_ptr(), cu_q.data_ptr(),
            tile_seq.data_ptr(), tile_q0.data_ptr(), int(num_tiles), ctx_len.numel(), q.shape[0], page_table.shape[1],
            backed_pages(pool), hq, hkv, d, q.stride(0), out.stride(0), float(scale), int(window), int(sink),
            status_word().data_ptr(), _stream())
        _native.check(rc, "ogb_paged_prefill_tc_bf16")
        launch_counts["paged_prefill_tc"] += 1
        launch_counts["paged_prefill"] += 1
        return out
    rc = _native.load().ogb_paged_prefill_bf16(
        q.data_ptr(), out.data_ptr(), pool.data_ptr(), page_table.data_ptr(), ctx_len.data_ptr(), cu_q.data_ptr(),
        tile_seq.data_ptr(), tile_q0.data_ptr(), int(num_tiles), ctx_len.numel(), page_table.shape[1], backed_pages(pool),
        hq, hkv, d, q.stride(0), out.stride(0), float(scale), int(window), int(sink), status_word().data_ptr(), _stream())
    _native.check(rc, "ogb_paged_prefill_bf16")
    launch_counts["paged_prefill"] += 1
    return out


@_timed("paged_decode")
def paged_decode(q, out, pool, page_table, ctx_len, hq, hkv, d, scale=None, num_splits=1, part_o=None, part_ml=None,
                 window=0, kv_scales=None, sink=0):
    """One query token per sequence (row s of q) over paged KV; ctx_len[s] <= 0 marks an idle row.
    ``kv_scales`` selects the e4m3 page kernels."""
    scale = scale or 1.0 / math.sqrt(d)
    n = ctx_len.numel()
    if not q.is_cuda:
        cu = torch.arange(n + 1, dtype=torch.int32)
        if kv_scales is None and _cpu_native(q) and pool.dtype == torch.float32 and pool.is_contiguous():
            out[:n].copy_(cpu.paged_attention(q[:n], pool, page_table, ctx_len, cu, hq, hkv, d, scale, window, sink))
            return out
        out[:n].copy_(reference.paged_attention(q[:n], pool, page_table, ctx_len, cu, hq, hkv, d, scale, window, kv_scales, sink))
        return out
    if num_splits > 1 and part_o is None:
        part_o = torch.empty(n * hq * num_splits * d, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n * hq * num_splits * 2, dtype=torch.float32, device=q.device)
    if kv_scales is not None:
        rc = _native.load().ogb_paged_decode_q8(
            q.data_ptr(), out.data_ptr(), pool.data_ptr(), kv_scales.data_ptr(), kv_format(pool), page_table.data_ptr(), ctx_len.data_ptr(), n,
            page_table.shape[1], backed_pages(pool), hq, hkv, d, q.stride(0), out.stride(0), float(scale), int(num_splits),
            _ptr(part_o), _ptr(part_ml), int(window), int(sink), status_word().data_ptr(), _stream())
        _native.check(rc, "ogb_paged_decode_q8")
        launch_counts["paged_decode_fp8"] += 1
        return out
    rc = _native.load().ogb_paged_decode_bf16(
        q.data_ptr(), out.data_ptr(), pool.data_ptr(), page_table.data_ptr(), ctx_len.data_ptr(), n,
        page_table.shape[1], backed_pages(pool), hq, hkv, d, q.stride(0), out.stride(0), float(scale), int(num_splits),
        _ptr(part_o), _ptr(part_ml), int(window), int(sink), status_word().data_ptr(), _stream())
    _native.check(rc, "ogb_paged_decode_bf16")
    launch_counts["paged_decode"] += 1
    return out


# ------------------------------------------------------------------------------------------
# token selection
# ------------------------------------------------------------------------------------------
@_timed("argmax")
def argmax(logits, out=None):
    if not logits.is_cuda:
        return cpu.argmax(logits) if _cpu_native(logits) else reference.argmax(logits)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    rc = _native.load().ogb_argmax_bf16(logits.data_ptr(), out.data_ptr(), rows, vocab, logits.stride(0), _stream())
    _native.check(rc, "ogb_argmax_bf16")
    launch_counts["argmax"] += 1
    return out


@_timed("sample")
def sample(logits, temperature, top_k, top_p, min_p, uniform, work=None, out=None):
    """Fused temperature/top-k/top-p/min-p sampler; per-row parameter tensors; ``uniform`` in [0,1)."""
    if not logits.is_cuda:
        if _cpu_native(logits):
            return cpu.sample(logits, temperature, top_k, top_p, min_p, uniform)
        return reference.sample(logits, temperature, top_k, top_p, min_p, uniform)
    rows, vocab = logits.shape
    if work is None:
        work = torch.empty(rows * vocab, dtype=torch.int32, device=logits.device)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    rc = _native.load().ogb_sample_bf16(logits.data_ptr(), out.data_ptr(), temperature.data_ptr(), top_k.data_ptr(),
                                        top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(), work.data_ptr(), rows,
                                        vocab, logits.stride(0), _stream())
    _native.check(rc, "ogb_sample_bf16")
    launch_counts["sample"] += 1
    return out


@_timed("spec_verify_greedy")
def spec_verify_greedy(logits, draft, k):
    if not logits.is_cuda:
        return reference.spec_verify_greedy(logits, draft, k)
    s = draft.shape[0]
    accept = torch.empty(s, dtype=torch.int32, device=logits.device)
    out = torch.empty(s, k + 1, dtype=torch.int32, device=logits.device)
    rc = _native.load().ogb_spec_verify_greedy(logits.data_ptr(), draft.data_ptr(), accept.data_ptr(), out.data_ptr(),
                                               s, k, logits.shape[1], logits.stride(0), _stream())
    _native.check(rc, "ogb_spec_verify_greedy")
    launch_counts["spec_verify_greedy"] += 1
    return accept, out


# ------------------------------------------------------------------------------------------
# KV page utilities (pool: one layer [P, hkv, 2, PAGE, d])
# ------------------------------------------------------------------------------------------
def _page_bytes(pool):
    return pool.stride(0) * pool.element_size()


def kv_page_copy(pool, src_pages, dst_pages):
    if not pool.is_cuda:
        pool[dst_pages.long()] = pool[src_pages.long()]
        return
    rc = _native.load().ogb_kv_page_copy(pool.data_ptr(), src_pages.data_ptr(), dst_pages.data_ptr(),
                                         src_pages.numel(), _page_bytes(pool), _stream())
    _native.check(rc, "ogb_kv_page_copy")
    launch_counts["kv_page_copy"] += 1


def kv_gather_pages(pool, staging, pages):
    if not pool.is_cuda:
        staging[: pages.numel()] = pool[pages.long()]
        return
    rc = _native.load().ogb_kv_gather_pages(pool.data_ptr(), staging.data_ptr(), pages.data_ptr(), pages.numel(),
                                            _page_bytes(pool), _stream())
    _native.check(rc, "ogb_kv_gather_pages")
    launch_counts["kv_gather_pages"] += 1


def kv_scatter_pages(pool, staging, pages):
    if not pool.is_cuda:
        pool[pages.long()] = staging[: pages.numel()]
        return
    rc = _native.load().ogb_kv_scatter_pages(pool.data_ptr(), staging.data_ptr(), pages.data_ptr(), pages.numel(),
                                             _page_bytes(pool), _stream())
    _native.check(rc, "ogb_kv_scatter_pages")
    launch_counts["kv_scatter_pages"] += 1


def kv_move_pages(dst_bases, src_bases, layers, src_pages, dst_pages, n, page_bytes, src_count, dst_count):
    """Move ``n`` pages of every layer in one launch: ``dst_bases[l] + dst_pages[i]*page_bytes <- src_bases[l] +
    src_pages[i]*page_bytes``.  The base tables are int64 device tensors of addresses (device memory or pinned host
    memory), the index lists int32 device tensors (views of the step plan).  Ids outside ``[0, count)`` raise the
    status bit and are skipped."""
    lib = _native.load()
    done = 0
    while done < n:
        m = min(n - done, 65535)
        rc = lib.ogb_kv_move_pages(dst_bases.data_ptr(), src_bases.data_ptr(), int(layers),
                                   src_pages.data_ptr() + 4 * done, dst_pages.data_ptr() + 4 * done, m, int(page_bytes),
                                   int(src_count), int(dst_count), status_word().data_ptr(), _stream())
        _native.check(rc, "ogb_kv_move_pages")
        launch_counts["kv_move_pages"] += 1
        done += m
