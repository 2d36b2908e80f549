"""Device-side activity on the trace timeline: kernels, copies and memsets with their GPU timestamps.

:class:`GpuActivityCollector` drives the CUPTI activity collector of the runtime library
(csrc/runtime/cupti_collector.cpp).  Between ``start()`` and ``stop()`` CUPTI records every kernel launch (and, if asked,
every memcpy / memset) of the process asynchronously; ``stop()`` flushes its buffers and returns the records.  CUPTI's clock
is sampled against ``time.perf_counter()`` at both ends, so the records land on the same axis as the engine's host spans
and :func:`merge_into_trace` can lay them out as one track per GPU stream beside them.

    with GpuActivityCollector() as gpu:
        engine.generate(...)
    print(gpu.table())                              # per-kernel count / total / mean, slowest first
    merge_into_trace("trace.json", gpu)             # host spans + one track per stream, opens in ui.perfetto.dev

``ONNX_GENAI_TRACE_CUPTI=1`` together with ``ONNX_GENAI_TRACE=<path>`` does the same for a whole process through the
process-wide tracer.  Collecting costs time per launch: numbers taken while it runs are for reading a timeline, not for
reporting throughput.

Same role as the reference's CUPTI tracer back end (crates/onnx-runtime-tracer/src/cupti.rs:1-60).
"""
from __future__ import annotations

import ctypes
import glob
import os
import time
from collections import defaultdict
from dataclasses import dataclass

KINDS = ("kernel", "memcpy", "memset")
COPY_KINDS = {1: "host to device", 2: "device to host", 8: "device to device", 10: "peer to peer"}


class _Record(ctypes.Structure):
    _fields_ = [("start_ns", ctypes.c_uint64), ("end_ns", ctypes.c_uint64), ("bytes", ctypes.c_uint64), ("kind", ctypes.c_uint32),
                ("device", ctypes.c_uint32), ("stream", ctypes.c_uint32), ("correlation", ctypes.c_uint32),
                ("grid", ctypes.c_int32 * 3), ("block", ctypes.c_int32 * 3), ("detail", ctypes.c_uint32), ("name_id", ctypes.c_uint32)]


@dataclass
class GpuActivity:
    kind: str                  # kernel | memcpy | memset
    name: str
    start_s: float             # on the time.perf_counter() axis
    end_s: float
    device: int
    stream: int
    correlation: int
    grid: tuple = (0, 0, 0)
    block: tuple = (0, 0, 0)
    bytes: int = 0             # copies: size; kernels: static + dynamic shared memory
    detail: int = 0            # copies: CUPTI copy kind; kernels: registers per thread

    @property
    def duration_us(self) -> float:
        return (self.end_s - self.start_s) * 1e6


def short_name(name: str) -> str:
    """A demangled kernel signature cut down for a table: no return type, no namespace of this package, no parameter list
    (template arguments stay: they tell instantiations apart)."""
    depth, cut = 0, len(name)
    for i, ch in enumerate(name):                        # the parameter list opens at the first '(' outside <...>
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif ch == "(" and depth == 0:
            cut = i
            break
    head = name[:cut]
    depth = 0
    for i in range(len(head) - 1, -1, -1):               # drop a leading return type: the last space outside <...>
        ch = head[i]
        if ch == ">":
            depth += 1
        elif ch == "<":
            depth -= 1
        elif ch == " " and depth == 0:
            head = head[i + 1:]
            break
    return head[5:] if head.startswith("ogb::") else head


class GpuActivityError(RuntimeError):
    pass


def _lib():
    from ..engine.core import load_runtime

    lib = load_runtime()
    if not getattr(lib, "_ogb_cupti_bound", False):
        lib.ogb_cupti_start.argtypes = [ctypes.c_char_p, ctypes.c_int]
        lib.ogb_cupti_start.restype = ctypes.c_int
        lib.ogb_cupti_drain.argtypes = [ctypes.POINTER(_Record), ctypes.c_int]
        lib.ogb_cupti_drain.restype = ctypes.c_int
        lib.ogb_cupti_name.argtypes = [ctypes.c_uint32]
        lib.ogb_cupti_name.restype = ctypes.c_char_p
        lib.ogb_cupti_last_error.restype = ctypes.c_char_p
        lib.ogb_cupti_now.restype = ctypes.c_uint64
        lib.ogb_cupti_dropped.restype = ctypes.c_uint64
        for fn in ("ogb_cupti_stop", "ogb_cupti_flush", "ogb_cupti_pending", "ogb_cupti_headers"):
            getattr(lib, fn).restype = ctypes.c_int
        lib._ogb_cupti_bound = True
    return lib


def find_cupti_library() -> str:
    """The CUPTI shared library to open: ``ONNX_GENAI_CUPTI_LIB``, else the one shipped with the CUDA wheels torch uses
    (so that a profiler inside torch and this collector talk to one CUPTI), else '' (the loader's search path decides)."""
    explicit = os.environ.get("ONNX_GENAI_CUPTI_LIB", "")
    if explicit:
        return explicit
    try:
        import nvidia.cuda_cupti as pkg                      # the wheel torch depends on

        for base in list(getattr(pkg, "__path__", [])):
            hits = sorted(glob.glob(os.path.join(base, "lib", "libcupti.so*")))
            if hits:
                return hits[0]
    except Exception:
        pass
    for base in (os.environ.get("CUDA_HOME", ""), "/usr/local/cuda"):
        for sub in ("lib64", os.path.join("extras", "CUPTI", "lib64")):
            hits = sorted(glob.glob(os.path.join(base, sub, "libcupti.so*"))) if base else []
            if hits:
                return hits[0]
    return ""


class GpuActivityCollector:
    """Start / stop CUPTI activity collection and turn its records into :class:`GpuActivity` rows (see module docstring)."""

    def __init__(self, library: str | None = None, copies: bool = True):
        self.library = library if library is not None else find_cupti_library()
        self.copies = bool(copies)
        self.records: list[GpuActivity] = []
        self.running = False
        self._clock = None           # (cupti ns, perf_counter s) pairs at start and at the latest drain

    # -- control ------------------------------------------------------------------------------------------
    def start(self) -> "GpuActivityCollector":
        lib = _lib()
        if lib.ogb_cupti_start(self.library.encode() if self.library else None, int(self.copies)) != 0:
            raise GpuActivityError(lib.ogb_cupti_last_error().decode())
        self._clock = [self._sample(lib), None]
        self.running = True
        return self

    def stop(self) -> list[GpuActivity]:
        if not self.running:
            return self.records
        lib = _lib()
        rc = lib.ogb_cupti_stop()
        self.running = False
        self._drain(lib)
        if rc != 0:
            raise GpuActivityError(lib.ogb_cupti_last_error().decode())
        return self.records

    def poll(self) -> list[GpuActivity]:
        """Flush what CUPTI holds so far and return every record since start (collection goes on)."""
        lib = _lib()
        if self.running and lib.ogb_cupti_flush() != 0:
            raise GpuActivityError(lib.ogb_cupti_last_error().decode())
        self._drain(lib)
        return self.records

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False

    @property
    def dropped(self) -> int:
        """Records CUPTI or the collector had to discard (buffers not drained in time)."""
        return int(_lib().ogb_cupti_dropped())

    # -- records ------------------------------------------------------------------------------------------
    @staticmethod
    def _sample(lib):
        a = time.perf_counter()
        t = int(lib.ogb_cupti_now())
        b = time.perf_counter()
        return t, 0.5 * (a + b)

    def _to_host(self, ns: int) -> float:
        (t0, h0), end = self._clock
        if end is None or end[0] == t0:
            return h0 + (ns - t0) * 1e-9
        t1, h1 = end                                     # two samples: correct the drift between the two clocks as well
        return h0 + (ns - t0) * (h1 - h0) / (t1 - t0)

    def _drain(self, lib) -> None:
        self._clock[1] = self._sample(lib)
        buf = (_Record * 4096)()
        names: dict[int, str] = {}
        while True:
            n = lib.ogb_cupti_drain(buf, len(buf))
            for r in buf[:n]:
                if r.name_id not in names:
                    names[r.name_id] = lib.ogb_cupti_name(r.name_id).decode(errors="replace")
                self.records.append(GpuActivity(KINDS[r.kind] if r.kind < len(KINDS) else "other", names[r.name_id],
                                                self._to_host(r.start_ns), self._to_host(r.end_ns), r.device, r.stream, r.correlation,
                                                tuple(r.grid), tuple(r.block), int(r.bytes), int(r.detail)))
            if n < len(buf):
                break
        self.records.sort(key=lambda a: a.start_s)

    # -- views --------------------------------------------------------------------------------------------
    def spans(self):
        """(name, start_s, end_s, track) rows for the trace writer: one track per device stream."""
        out = []
        for a in self.records:
            name = short_name(a.name) if a.kind == "kernel" else f"{a.kind} {COPY_KINDS.get(a.detail, '')} {a.bytes} B".replace("  ", " ")
            out.append((name, a.start_s, a.end_s, f"gpu{a.device} stream {a.stream}"))
        return out

    def summary(self) -> list[dict]:
        """Per-name totals, largest total first: ``{"name", "kind", "count", "total_us", "mean_us", "max_us", "bytes"}``."""
        acc = defaultdict(lambda: {"count": 0, "total_us": 0.0, "max_us": 0.0, "bytes": 0})
        for a in self.records:
            e = acc[(a.kind, a.name)]
            e["count"] += 1
            e["total_us"] += a.duration_us
            e["max_us"] = max(e["max_us"], a.duration_us)
            e["bytes"] += a.bytes if a.kind != "kernel" else 0
        rows = [{"name": name, "kind": kind, **e, "mean_us": e["total_us"] / e["count"]} for (kind, name), e in acc.items()]
        return sorted(rows, key=lambda r: -r["total_us"])

    def busy_fraction(self) -> float:
        """Share of the span from the first start to the last end during which at least one activity ran on the device."""
        if not self.records:
            return 0.0
        busy, cur_a, cur_b = 0.0, None, None
        for a in self.records:                            # sorted by start
            if cur_b is None or a.start_s > cur_b:
                if cur_b is not None:
                    busy += cur_b - cur_a
                cur_a, cur_b = a.start_s, a.end_s
            else:
                cur_b = max(cur_b, a.end_s)
        busy += cur_b - cur_a
        total = max(a.end_s for a in self.records) - self.records[0].start_s
        return busy / total if total > 0 else 1.0

    def table(self, top: int = 25) -> str:
        rows = self.summary()[:top]
        shown = [short_name(r["name"])[:72] for r in rows]
        width = max([len(n) for n in shown] + [4])
        lines = [f"{'name':<{width}}  {'count':>7}  {'total us':>11}  {'mean us':>9}  {'max us':>9}"]
        for n, r in zip(shown, rows):
            lines.append(f"{n:<{width}}  {r['count']:>7}  {r['total_us']:>11.1f}  {r['mean_us']:>9.2f}  {r['max_us']:>9.2f}")
        lines.append(f"device busy {100 * self.busy_fraction():.1f} % of the recorded span; {self.dropped} records dropped")
        return "\n".join(lines)


def merge_into_trace(path: str, collector: GpuActivityCollector, host_spans=None) -> int:
    """Write host spans (default: the process-wide tracer's) and the collector's device activity as one Chrome Trace
    document; returns the number of events written."""
    from . import trace as _trace

    if host_spans is None:
        with _trace.TRACER.lock:
            host_spans = list(_trace.TRACER.spans)
    spans = list(host_spans) + collector.spans()
    _trace.write_chrome_trace(path, spans)
    return len(spans)
