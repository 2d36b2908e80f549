"""Chrome Trace Event (Perfetto) timeline export and a small span collector.

Role of the reference's runtime trace (crates/onnx-genai-engine/src/runtime_trace.rs:1-107,
`ONNX_GENAI_TRACE=path`): engine spans and per-op device spans on one clock, written as JSON that
https://ui.perfetto.dev opens directly.
"""
from __future__ import annotations

import json
import os
import threading
import time


def chrome_trace_events(spans=None, pid: int = 1) -> dict:
    """The collected spans (default: the process-wide tracer's) as a Chrome Trace Event document."""
    if spans is None:
        with TRACER.lock:
            spans = list(TRACER.spans)
    events = []
    tids = {}
    for name, a, b, cat in spans:
        tid = tids.setdefault(cat, len(tids) + 1)
        events.append({"name": name, "cat": cat, "ph": "X", "ts": a * 1e6, "dur": max(0.0, (b - a) * 1e6), "pid": pid, "tid": tid})
    for cat, tid in tids.items():
        events.append({"name": "thread_name", "ph": "M", "pid": pid, "tid": tid, "args": {"name": cat}})
    return {"traceEvents": events, "displayTimeUnit": "ms"}


def write_chrome_trace(path: str, spans, pid: int = 1) -> None:
    """spans: iterable of (name, t_start_s, t_end_s, category)."""
    events = []
    tids = {}
    for name, a, b, cat in spans:
        tid = tids.setdefault(cat, len(tids) + 1)
        events.append({"name": name, "cat": cat, "ph": "X", "ts": a * 1e6, "dur": max(0.0, (b - a) * 1e6), "pid": pid, "tid": tid})
    for cat, tid in tids.items():
        events.append({"name": "thread_name", "ph": "M", "pid": pid, "tid": tid, "args": {"name": cat}})
    with open(path, "w", encoding="utf-8") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)


class Tracer:
    """Process-wide span collector; enabled by ONNX_GENAI_TRACE=<path> or start()."""

    def __init__(self):
        self.lock = threading.Lock()
        self.spans = []
        from .runtime_config import runtime_config

        self.path = runtime_config().trace_path or None      # ONNX_GENAI_TRACE
        self.enabled = self.path is not None
        # ONNX_GENAI_TRACE_NVTX=1: every span also opens an NVTX range, so an external profiler that records NVTX
        # (Nsight Systems, a CUPTI-based collector) sees the engine's stages on the same timeline as the kernels.  This
        # is the hand-off to vendor collectors that the reference does through its ITT tracer back end
        # (crates/onnx-runtime-tracer/src/itt.rs).
        import os

        self.nvtx = None
        if os.environ.get("ONNX_GENAI_TRACE_NVTX", "0") not in ("", "0"):
            self.enable_nvtx()
        # ONNX_GENAI_TRACE_CUPTI=1 (with ONNX_GENAI_TRACE): device activity (kernels, copies) is collected through CUPTI
        # from the first span on and written as one track per GPU stream beside the host spans (utils/gpu_activity.py).
        self.gpu = None
        self.gpu_error = ""
        self.want_gpu = os.environ.get("ONNX_GENAI_TRACE_CUPTI", "0") not in ("", "0")
        if self.enabled:                     # ONNX_GENAI_TRACE=<path>: the file is written when the process exits
            self._flush_at_exit()

    def _start_gpu(self):
        self.want_gpu = False
        try:
            from .gpu_activity import GpuActivityCollector

            self.gpu = GpuActivityCollector().start()
        except Exception as exc:            # no CUPTI here: the host spans are still worth having
            self.gpu, self.gpu_error = None, str(exc)

    def enable_nvtx(self, push=None, pop=None):
        """Mirror spans as NVTX ranges (``push(name)`` / ``pop()`` default to torch.cuda.nvtx; tests pass fakes)."""
        if push is None or pop is None:
            try:
                import torch

                push, pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
            except Exception:        # no CUDA build: ranges have nowhere to go
                self.nvtx = None
                return False
        self.nvtx = (push, pop)
        return True

    def start(self, path):
        self.path, self.enabled = path, True
        self._flush_at_exit()

    def add(self, name, t0, t1, cat="engine"):
        """Record a span whose ends the caller timed itself (``time.perf_counter()`` seconds)."""
        if self.enabled:
            with self.lock:
                self.spans.append((name, t0, t1, cat))

    def _flush_at_exit(self):
        if not getattr(self, "_exit_hook", False):
            import atexit

            atexit.register(self.flush)
            self._exit_hook = True

    def span(self, name, cat="engine"):
        tracer = self

        class _Span:
            def __enter__(self):
                if tracer.want_gpu and tracer.enabled:
                    tracer._start_gpu()
                self.t0 = time.perf_counter()
                self.ranged = False
                if tracer.nvtx is not None:
                    try:
                        tracer.nvtx[0](f"{cat}:{name}")
                        self.ranged = True
                    except Exception:
                        tracer.nvtx = None           # NVTX is not usable in this process: stop trying
                return self

            def __exit__(self, *exc):
                if self.ranged and tracer.nvtx is not None:
                    tracer.nvtx[1]()
                if tracer.enabled:
                    with tracer.lock:
                        tracer.spans.append((name, self.t0, time.perf_counter(), cat))
                return False

        return _Span()

    def flush(self):
        if self.enabled and self.path:
            spans = list(self.spans)
            if self.gpu is not None:
                try:
                    self.gpu.poll()
                    spans += self.gpu.spans()
                except Exception as exc:
                    self.gpu_error = str(exc)
            write_chrome_trace(self.path, spans)


TRACER = Tracer()
