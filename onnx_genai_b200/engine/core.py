"""ctypes binding of the C++ runtime core (scheduler + paged-KV block pool + step builder).

The reference splits this across `onnx-genai-scheduler` and `onnx-genai-kv`
(crates/onnx-genai-scheduler/src/lib.rs:199-760, crates/onnx-genai-kv/src/paged_cache.rs:57-1085);
the C++ restatement lives in csrc/runtime/core.{h,cpp}.  A step is exchanged as one packed int32
plan written straight into pinned host memory, so the per-step host work is one C call plus one
host-to-device copy.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_LIB = None

POLICIES = {"fcfs": 0, "priority": 1, "fair_share": 2}
PREEMPT = {"recompute": 0, "swap": 1}
FINISH = {0: None, 1: "length", 2: "stop", 3: "cancelled", 4: "error"}

HDR = dict(num_tokens=0, num_decode=1, num_prefill_seqs=2, num_tiles=3, num_logit_rows=4, num_copies=5,
           num_swap_out=6, num_swap_in=7, num_prefill_tokens=8, max_ctx=9, num_preempted=10, step_id=11, num_move_runs=12)

_LAYOUT_FIELDS = ["header", "token_ids", "positions", "slots", "seq_slot", "ctx_len", "cu_q", "page_table", "tile_seq",
                  "tile_q0", "logit_rows", "temperature", "top_k", "top_p", "min_p", "uniform", "copy_src", "copy_dst",
                  "swap_out_dev", "swap_out_host", "swap_in_dev", "swap_in_host", "total_words", "max_tiles", "max_swap",
                  "logit_seq", "max_rows", "move_runs", "max_runs"]


def load_runtime():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = Path(__file__).resolve().parent.parent / "_lib" / "libogb_runtime.so"
    try:
        from .. import build as _build

        path = _build.build_runtime()
    except Exception as exc:
        if not path.exists():
            raise RuntimeError(f"runtime library {path} is missing and could not be built: {exc}") from exc
    lib = ctypes.CDLL(str(path))
    P = c_void_p
    I32P = POINTER(c_int32)
    lib.ogb_core_create.argtypes = [c_int] * 12
    lib.ogb_core_create.restype = P
    lib.ogb_core_destroy.argtypes = [P]
    lib.ogb_core_layout.argtypes = [P, I32P, c_int]
    lib.ogb_core_layout.restype = c_int
    lib.ogb_core_add_request.argtypes = [P, I32P, c_int, c_int, c_float, c_int, c_float, c_float, c_uint64, c_int, c_int,
                                         c_int, I32P, c_int]
    lib.ogb_core_add_request.restype = c_int64
    lib.ogb_core_build_step.argtypes = [P, c_void_p]
    lib.ogb_core_build_step.restype = c_int
    lib.ogb_core_commit_step.argtypes = [P, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int]
    lib.ogb_core_commit_step.restype = c_int
    for name in ("ogb_core_cancel",):
        getattr(lib, name).argtypes = [P, c_int64]
        getattr(lib, name).restype = c_int
    lib.ogb_core_add_pages.argtypes = [P, c_int]
    lib.ogb_core_add_pages.restype = None
    lib.ogb_core_fork.argtypes = [P, c_int64]
    lib.ogb_core_fork.restype = c_int64
    lib.ogb_core_seq_computed.argtypes = [P, c_int64]
    lib.ogb_core_seq_computed.restype = c_int
    lib.ogb_core_swap_state.argtypes = [P, c_int64, c_int64]
    lib.ogb_core_swap_state.restype = c_int
    lib.ogb_core_rewind.argtypes = [P, c_int64, c_int]
    lib.ogb_core_rewind.restype = c_int
    lib.ogb_core_set_window.argtypes = [P, c_int, c_int]
    lib.ogb_core_set_window.restype = None
    lib.ogb_core_released_pages.argtypes = [P, c_int64]
    lib.ogb_core_released_pages.restype = c_int
    lib.ogb_core_set_draft.argtypes = [P, c_int64, I32P, c_int]
    lib.ogb_core_set_draft.restype = c_int
    lib.ogb_core_append_tokens.argtypes = [P, c_int64, I32P, c_int]
    lib.ogb_core_append_tokens.restype = c_int
    lib.ogb_core_seq_pages.argtypes = [P, c_int64, I32P, c_int]
    lib.ogb_core_seq_pages.restype = c_int
    lib.ogb_core_prefix_adopt.argtypes = [P, I32P, c_int, I32P, c_int]
    lib.ogb_core_prefix_adopt.restype = c_int
    lib.ogb_core_prefix_unpublish.argtypes = [P, I32P, c_int]
    lib.ogb_core_prefix_unpublish.restype = c_int
    lib.ogb_core_prefix_peek.argtypes = [P, I32P, c_int, I32P, c_int]
    lib.ogb_core_prefix_peek.restype = c_int
    lib.ogb_core_seq_len.argtypes = [P, c_int64]
    lib.ogb_core_seq_len.restype = c_int
    lib.ogb_core_seq_tokens.argtypes = [P, c_int64, I32P, c_int]
    lib.ogb_core_seq_tokens.restype = c_int
    lib.ogb_core_release.argtypes = [P, c_int64]
    lib.ogb_core_stat.argtypes = [P, c_int]
    lib.ogb_core_stat.restype = c_int64
    _LIB = lib
    return lib


@dataclass
class CoreConfig:
    num_pages: int
    num_host_pages: int = 0
    max_seqs: int = 256
    max_tokens_per_step: int = 2048
    max_pages_per_seq: int = 256
    prefill_chunk: int = 2048
    token_multiple: int = 1
    policy: str = "fcfs"
    preempt: str = "recompute"
    enable_prefix_cache: bool = True
    eos_token: int = -1
    max_draft_tokens: int = 0


class Layout:
    def __init__(self, values):
        for k, v in zip(_LAYOUT_FIELDS, values):
            setattr(self, k, int(v))


class Core:
    """Owner of all sequence / page bookkeeping.  Not thread-safe: one driver thread owns it."""

    def __init__(self, cfg: CoreConfig):
        self.cfg = cfg
        self.lib = load_runtime()
        self.h = self.lib.ogb_core_create(cfg.num_pages, cfg.num_host_pages, cfg.max_seqs, cfg.max_tokens_per_step,
                                          cfg.max_pages_per_seq, cfg.prefill_chunk, cfg.token_multiple,
                                          POLICIES[cfg.policy], PREEMPT[cfg.preempt], int(cfg.enable_prefix_cache),
                                          cfg.eos_token, cfg.max_draft_tokens)
        buf = (c_int32 * 32)()
        n = self.lib.ogb_core_layout(self.h, buf, 32)
        self.layout = Layout(list(buf)[:n])
        self._ev_seq = np.zeros(self.layout.max_rows, dtype=np.int64)
        self._ev_tok = np.zeros(self.layout.max_rows, dtype=np.int32)
        self._ev_fin = np.zeros(self.layout.max_rows, dtype=np.int32)

    def __del__(self):
        try:
            if self.h:
                self.lib.ogb_core_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def add_request(self, prompt, max_new_tokens, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0, priority=0,
                    tenant=0, ignore_eos=False, stop_ids=()):
        arr = np.ascontiguousarray(prompt, dtype=np.int32)
        stop = np.ascontiguousarray(stop_ids, dtype=np.int32)
        sid = self.lib.ogb_core_add_request(
            self.h, arr.ctypes.data_as(POINTER(c_int32)), len(arr), int(max_new_tokens), float(temperature), int(top_k),
            float(top_p), float(min_p), int(seed) & 0xFFFFFFFFFFFFFFFF, int(priority), int(tenant), int(ignore_eos),
            stop.ctypes.data_as(POINTER(c_int32)), len(stop))
        if sid == -1:
            raise ValueError("empty prompt or negative max_new_tokens")
        if sid == -2:
            raise ValueError(f"prompt of {len(arr)} tokens does not fit max_pages_per_seq={self.cfg.max_pages_per_seq} "
                             f"({self.cfg.max_pages_per_seq * 16} tokens); raise it or shorten the prompt")
        return int(sid)

    def build_step(self, plan_ptr: int) -> int:
        return self.lib.ogb_core_build_step(self.h, plan_ptr)

    def commit_step(self, sampled_ptr: int, n: int):
        ne = self.lib.ogb_core_commit_step(self.h, sampled_ptr, n, self._ev_seq.ctypes.data, self._ev_tok.ctypes.data,
                                           self._ev_fin.ctypes.data, len(self._ev_seq))
        return [(int(self._ev_seq[i]), int(self._ev_tok[i]), FINISH[int(self._ev_fin[i])]) for i in range(ne)]

    def cancel(self, sid):
        return bool(self.lib.ogb_core_cancel(self.h, sid))

    def add_pages(self, n: int) -> None:
        """The KV buffers grew in place: ``n`` more page ids become allocatable."""
        self.lib.ogb_core_add_pages(self.h, int(n))

    def fork(self, sid):
        return int(self.lib.ogb_core_fork(self.h, sid))

    def swap_state(self, a, b) -> bool:
        """The two sequences exchange everything but their ids (between steps only)."""
        return bool(self.lib.ogb_core_swap_state(self.h, a, b))

    def rewind(self, sid, new_len):
        return bool(self.lib.ogb_core_rewind(self.h, sid, new_len))

    def set_window(self, window: int, sink_tokens: int = 0):
        """Sliding-window retention: pages that no later query can see -- all of them lie between the first
        ceil(sink_tokens / 16) pages and the window -- are released as sequences advance (their page-table entries
        become -1); a rewind that would need them again is refused.  ``window`` <= 0 turns it off."""
        self.lib.ogb_core_set_window(self.h, int(window), int(sink_tokens))

    def released_pages(self, sid) -> int:
        return int(self.lib.ogb_core_released_pages(self.h, sid))

    def set_draft(self, sid, tokens):
        """Propose tokens to follow the sequence's last token; verified (and rewound) by the next step."""
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        return bool(self.lib.ogb_core_set_draft(self.h, sid, arr.ctypes.data_as(POINTER(c_int32)), len(arr)))

    def append_tokens(self, sid, tokens):
        """Extend a live sequence with caller-chosen tokens (computed as a prefill chunk by the next steps)."""
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        return bool(self.lib.ogb_core_append_tokens(self.h, sid, arr.ctypes.data_as(POINTER(c_int32)), len(arr)))

    def seq_pages(self, sid):
        """Device pages of a live sequence that hold computed tokens (in order)."""
        out = np.zeros(self.cfg.max_pages_per_seq, dtype=np.int32)
        n = int(self.lib.ogb_core_seq_pages(self.h, sid, out.ctypes.data_as(POINTER(c_int32)), len(out)))
        return out[:max(n, 0)].copy()

    def prefix_adopt(self, tokens):
        """Register cached pages for every full page of ``tokens`` the prefix cache does not serve yet.  Returns an
        int32 array with one entry per served page: the adopted page id to fill, or -1 where a page existed."""
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.full(len(arr) // 16 + 1, -1, dtype=np.int32)
        n = int(self.lib.ogb_core_prefix_adopt(self.h, arr.ctypes.data_as(POINTER(c_int32)), len(arr),
                                               out.ctypes.data_as(POINTER(c_int32)), len(out)))
        return out[:max(n, 0)].copy()

    def prefix_unpublish(self, pages) -> int:
        """Take adopted pages that were never filled out of the prefix cache again; returns how many were removed."""
        arr = np.ascontiguousarray([p for p in pages if p >= 0], dtype=np.int32)
        if len(arr) == 0:
            return 0
        return int(self.lib.ogb_core_prefix_unpublish(self.h, arr.ctypes.data_as(POINTER(c_int32)), len(arr)))

    def prefix_peek(self, tokens):
        """Pages that currently serve the leading full pages of ``tokens`` in the prefix cache (no reference taken)."""
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.full(len(arr) // 16 + 1, -1, dtype=np.int32)
        n = int(self.lib.ogb_core_prefix_peek(self.h, arr.ctypes.data_as(POINTER(c_int32)), len(arr),
                                              out.ctypes.data_as(POINTER(c_int32)), len(out)))
        return out[:max(n, 0)].copy()

    def seq_len(self, sid):
        return int(self.lib.ogb_core_seq_len(self.h, sid))

    def seq_computed(self, sid):
        """Tokens of the sequence whose K/V are in the cache."""
        return int(self.lib.ogb_core_seq_computed(self.h, sid))

    def seq_tokens(self, sid):
        n = self.seq_len(sid)
        if n < 0:
            raise KeyError(sid)
        out = np.zeros(n, dtype=np.int32)
        self.lib.ogb_core_seq_tokens(self.h, sid, out.ctypes.data_as(POINTER(c_int32)), n)
        return out

    def release(self, sid):
        self.lib.ogb_core_release(self.h, sid)

    def _stat(self, i):
        return int(self.lib.ogb_core_stat(self.h, i))

    num_waiting = property(lambda self: self._stat(0))
    num_running = property(lambda self: self._stat(1))
    num_swapped = property(lambda self: self._stat(2))
    num_free_pages = property(lambda self: self._stat(3))
    prefix_hits = property(lambda self: self._stat(4))
    prefix_lookups = property(lambda self: self._stat(5))
    num_preemptions = property(lambda self: self._stat(6))
    has_work = property(lambda self: bool(self._stat(7)))
    spec_proposed = property(lambda self: self._stat(8))
    spec_accepted = property(lambda self: self._stat(9))
    spec_steps = property(lambda self: self._stat(10))
    num_pages = property(lambda self: self._stat(11))
