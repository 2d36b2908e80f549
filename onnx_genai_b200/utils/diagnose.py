"""Automatic diagnosis of a trace or of a per-operator profile: findings instead of timelines.

Counterpart of the reference's trace diagnosis and roofline analyser (crates/onnx-runtime-tracer/src/diagnose.rs:1-60):
every finding says **what** is wrong, **why** (the evidence, in numbers) and **how** to fix it; a kernel whose FLOPs and
bytes are unknown is reported as indeterminate rather than classified from invented figures.

Two inputs are understood:

* a Chrome Trace Event document (what ``ONNX_GENAI_TRACE`` / ``/v1/debug/trace/perfetto`` produce; ``args.flops`` /
  ``args.bytes`` on an event feed the roofline), and
* the per-operator table of ``ops.profile_stop()`` (``{op: (total_ms, calls)}``), optionally with the model
  configuration and the step's shape, from which :mod:`cost_model` supplies each part's roofline time.

``python -m onnx_genai_b200.utils.diagnose trace.json`` prints the report; ``bench.py --profile-ops`` and the CLI's
``--profile`` append it to their output.
"""
from __future__ import annotations

import json
import os
import re
import sys
from dataclasses import dataclass, field


@dataclass
class KernelSample:
    name: str
    duration_s: float               # total over `calls`
    calls: int = 1
    flops: float | None = None      # total over `calls`
    bytes: float | None = None
    category: str = "compute"


@dataclass
class RooflineResult:
    name: str
    bound: str                      # "compute" | "memory" | "latency" | "indeterminate"
    ceiling_s: float | None         # roofline time of the sample
    efficiency: float | None        # ceiling / measured (1.0 = at the roofline)
    intensity: float | None         # FLOP per byte
    achieved_tflops: float | None
    achieved_gbs: float | None


@dataclass
class Issue:
    severity: str                   # "high" | "medium" | "low"
    title: str
    description: str                # what
    evidence: str                   # why, in numbers
    root_cause: str
    suggestion: str                 # how

    def render(self) -> str:
        return (f"[{self.severity}] {self.title}\n  what : {self.description}\n  why  : {self.evidence}\n  cause: {self.root_cause}\n"
                f"  fix  : {self.suggestion}")


class RooflineAnalyzer:
    """Classifies a sample against ``max(FLOPs / peak, bytes / bandwidth)``; a sample whose roofline time is below
    ``latency_floor_s`` per call is latency-bound whatever its intensity."""

    def __init__(self, peak_tflops: float = 1376.4, hbm_gbs: float = 6446.6, latency_floor_s: float = 4e-6, name: str = "NVIDIA B200"):
        self.peak_tflops, self.hbm_gbs, self.latency_floor_s, self.name = peak_tflops, hbm_gbs, latency_floor_s, name

    @classmethod
    def measured(cls, path: str | None = None) -> "RooflineAnalyzer":
        """Denominators from a measured-peaks file (keys hbm_gbs, bf16_tflops_sustained) when one is found."""
        path = path or os.environ.get("OGB_MEASURED_PEAKS") or os.path.join(os.getcwd(), "MEASURED_PEAKS.json")
        try:
            with open(path, encoding="utf-8") as f:
                m = json.load(f)
            return cls(float(m.get("bf16_tflops_sustained", m.get("bf16_tflops", 1376.4))), float(m.get("hbm_gbs", 6446.6)),
                       name=str(m.get("gpu_name", "measured device")))
        except (OSError, ValueError):
            return cls()

    def analyze(self, s: KernelSample) -> RooflineResult:
        if s.duration_s <= 0 or (s.flops is None and s.bytes is None):
            return RooflineResult(s.name, "indeterminate", None, None, None, None, None)
        t_c = (s.flops or 0.0) / (self.peak_tflops * 1e12)
        t_m = (s.bytes or 0.0) / (self.hbm_gbs * 1e9)
        ceiling = max(t_c, t_m)
        per_call = ceiling / max(1, s.calls)
        bound = "latency" if per_call < self.latency_floor_s else ("compute" if t_c >= t_m else "memory")
        return RooflineResult(s.name, bound, ceiling, ceiling / s.duration_s,
                              (s.flops / s.bytes) if s.flops and s.bytes else None,
                              (s.flops / s.duration_s / 1e12) if s.flops else None, (s.bytes / s.duration_s / 1e9) if s.bytes else None)


@dataclass
class Diagnosis:
    issues: list = field(default_factory=list)
    rooflines: list = field(default_factory=list)
    total_s: float = 0.0
    notes: list = field(default_factory=list)

    def report(self) -> str:
        lines = [f"diagnosis over {self.total_s * 1e3:.3f} ms of device time: {len(self.issues)} finding(s)"]
        order = {"high": 0, "medium": 1, "low": 2}
        for i in sorted(self.issues, key=lambda x: order.get(x.severity, 3)):
            lines.append(i.render())
        if self.rooflines:
            lines.append("roofline (share of device time, bound, efficiency against the measured ceilings):")
            for r, share in self.rooflines:
                eff = "n/a" if r.efficiency is None else f"{r.efficiency:.2f}"
                lines.append(f"  {r.name:36s} {100 * share:5.1f}%  {r.bound:13s} {eff}")
        lines += [f"note: {n}" for n in self.notes]
        return "\n".join(lines)


_COMM = ("tp_", "exchange", "all_reduce", "nccl", "scatter")


def diagnose_samples(samples, analyzer: RooflineAnalyzer | None = None, wall_s: float | None = None, steps: int = 1,
                     preemptions: int = 0, graph_replays: int = 0, device_busy_s: float | None = None) -> Diagnosis:
    """``samples``: KernelSample list covering ``steps`` engine steps; ``wall_s``: host wall-clock time of the same steps
    (to find host-side gaps); ``device_busy_s``: time with at least one device event running, when the samples come from
    several streams whose events overlap (default: the sum of the samples)."""
    analyzer = analyzer or RooflineAnalyzer.measured()
    d = Diagnosis()
    d.total_s = sum(s.duration_s for s in samples)
    if d.total_s <= 0:
        d.notes.append("no device time recorded: was profiling enabled?")
        return d
    results = [(analyzer.analyze(s), s) for s in samples]
    d.rooflines = sorted(((r, s.duration_s / d.total_s) for r, s in results), key=lambda x: -x[1])
    for r, s in results:
        share = s.duration_s / d.total_s
        mean_us = s.duration_s / max(1, s.calls) * 1e6
        if r.bound in ("compute", "memory") and share >= 0.05 and r.efficiency is not None and r.efficiency < 0.5:
            what = "tensor-core rate" if r.bound == "compute" else "HBM bandwidth"
            got = f"{r.achieved_tflops:.0f} TFLOP/s of {analyzer.peak_tflops:.0f}" if r.bound == "compute" else f"{r.achieved_gbs:.0f} GB/s of {analyzer.hbm_gbs:.0f}"
            d.issues.append(Issue(
                "high" if share >= 0.15 else "medium", f"{s.name} runs at {r.efficiency:.2f} of its {r.bound} roofline",
                f"{s.name} takes {100 * share:.1f}% of device time and reaches {r.efficiency:.0%} of the {what} it is bound by.",
                f"{s.calls} call(s), {mean_us:.1f} us each; {got}; arithmetic intensity {r.intensity:.1f} FLOP/B." if r.intensity else
                f"{s.calls} call(s), {mean_us:.1f} us each; {got}.",
                "tile shape or wave quantisation for a contraction (few tiles per SM, short K), scattered or narrow accesses for a streaming pass",
                "check the tile count against 148 SMs (stream-K covers tail waves), batch more rows per launch, or fuse the pass into its producer" if r.bound == "compute"
                else "widen the loads to 16 bytes, keep pages contiguous, fuse the pass into the kernel that produces its input"))
        if s.calls / max(1, steps) >= 16 and mean_us < 5.0 and share >= 0.03:
            d.issues.append(Issue(
                "medium", f"{s.name} is launch-bound", f"{s.calls // max(1, steps)} launches of {s.name} per step last {mean_us:.1f} us on average.",
                f"{100 * share:.1f}% of device time in kernels shorter than the ~4 us a launch costs in a stream of launches.",
                "per-launch overhead, not work, sets the time", "replay the step from a CUDA graph (EngineConfig.cuda_graphs) or fuse the op into its neighbour (norm and activation prologues, residual epilogues exist for the GEMM and GEMV)"))
    comm = sum(s.duration_s for s in samples if any(k in s.name.lower() for k in _COMM) and "gemm" not in s.name.lower())
    if comm / d.total_s >= 0.2:
        d.issues.append(Issue("high", "tensor-parallel exchange dominates", f"Exchange kernels take {100 * comm / d.total_s:.1f}% of device time.",
                              f"{comm * 1e3 / max(1, steps):.3f} ms per step in reduce / broadcast kernels.",
                              "fixed fence-and-signal latency per exchange (two per layer), not bytes",
                              "use push mode (OGB_TP_PUSH=1) so the reduce reads local memory, enable OGB_TP_PDL=1 so the consumer GEMM starts under the exchange, or lower the TP degree (cost_model.pick_tp)"))
    busy_s = d.total_s if device_busy_s is None else device_busy_s
    if wall_s is not None and wall_s > 0 and busy_s / wall_s < 0.85:
        sev = "high" if busy_s / wall_s < 0.6 else "medium"
        d.issues.append(Issue(sev, "the GPU waits for the host", f"Device kernels cover {100 * busy_s / wall_s:.0f}% of the wall-clock time of the profiled steps.",
                              f"{wall_s * 1e3 / max(1, steps):.3f} ms per step on the wall clock against {busy_s * 1e3 / max(1, steps):.3f} ms of kernels"
                              + (f"; {graph_replays} graph replays" if graph_replays else "; no graph replays"),
                              "scheduling, plan packing or Python between steps is not overlapped with device work",
                              "enable CUDA-graph replay for decode steps, raise max_tokens_per_step so each step carries more work, or move per-step host work off the critical path"))
    if preemptions > 0:
        d.issues.append(Issue("medium", "sequences were preempted", f"{preemptions} preemption(s) during the profiled steps.",
                              "the scheduler ran out of free KV pages and evicted running sequences",
                              "the KV pool is smaller than the working set of the admitted batch",
                              "raise --kv-max-pages / gpu_memory_utilization, use one-byte KV pages (--kv-cache-dtype fp8_e4m3fn), enable swap preemption, or lower max_seqs"))
    unknown = [s.name for r, s in results if r.bound == "indeterminate" and s.duration_s / d.total_s >= 0.05]
    if unknown:
        d.notes.append("no FLOP / byte counts for " + ", ".join(sorted(unknown)) + ": their roofline is indeterminate, not assumed")
    return d


def samples_from_profile(agg: dict, cfg=None, shape=None, tp: int = 1, steps: int = 1) -> list:
    """``agg``: ``ops.profile_stop()``'s ``{op: (total_ms, calls)}``.  With a model configuration and a step shape the
    cost model's per-part FLOPs and bytes are attached to the operators that make up each part."""
    flops_bytes: dict = {}
    if cfg is not None and shape is not None:
        t = shape.decode_rows + shape.prefill_tokens
        hq, hkv = max(1, cfg.num_heads // tp), max(1, -(-cfg.num_kv_heads // tp))
        d, hid, L = cfg.head_dim, cfg.hidden, cfg.num_layers
        inter = cfg.intermediate // tp
        wb = 2.0 if cfg.weight_format == "bf16" else 0.5 + 2.0 / cfg.int4_block

        def gemm(n, k):
            return 2.0 * t * n * k * L * steps, (n * k * wb + 2.0 * t * (n + k)) * L * steps

        flops_bytes["gemm:qkv"] = gemm((hq + 2 * hkv) * d, hid)
        flops_bytes["gemm:o"] = gemm(hid, hq * d)
        flops_bytes["gemm:gate_up"] = gemm(2 * inter, hid)
        flops_bytes["gemm:down"] = gemm(hid, inter)
        kvb = shape.decode_rows * shape.mean_context * hkv * 2 * d * shape.kv_bytes * L * steps
        flops_bytes["paged_decode"] = (4.0 * shape.decode_rows * shape.mean_context * hq * d * L * steps, kvb)
        flops_bytes["paged_prefill"] = (4.0 * shape.prefill_tokens * shape.prefill_context * hq * d * L * steps, None)
        flops_bytes["rmsnorm"] = (None, 2.0 * t * hid * 2 * (2 * L + 1) * steps)
    out = []
    for name, (ms, calls) in agg.items():
        fb = flops_bytes.get(name)
        if fb is None:
            for key, v in flops_bytes.items():
                if name.startswith(key) or key.split(":")[-1] in name:
                    fb = v
                    break
        out.append(KernelSample(name, ms / 1e3, calls, fb[0] if fb else None, fb[1] if fb else None))
    return out


def samples_from_trace(doc: dict, category: str | None = None) -> tuple:
    """Chrome Trace Event document -> (samples aggregated by event name, wall-clock seconds the events span)."""
    agg: dict = {}
    t0, t1 = None, None
    for ev in doc.get("traceEvents", []):
        if ev.get("ph") != "X" or (category and ev.get("cat") != category):
            continue
        dur = float(ev.get("dur", 0.0)) / 1e6
        ts = float(ev.get("ts", 0.0)) / 1e6
        t0 = ts if t0 is None else min(t0, ts)
        t1 = ts + dur if t1 is None else max(t1, ts + dur)
        a = ev.get("args") or {}
        rec = agg.setdefault(ev["name"], [0.0, 0, None, None, ev.get("cat", "compute")])
        rec[0] += dur
        rec[1] += 1
        for i, key in ((2, "flops"), (3, "bytes")):
            if a.get(key) is not None:
                rec[i] = (rec[i] or 0.0) + float(a[key])
    samples = [KernelSample(n, r[0], r[1], r[2], r[3], r[4]) for n, r in agg.items()]
    return samples, (0.0 if t0 is None else t1 - t0)


_DEVICE_TRACK = re.compile(r"gpu\d+ stream \d+$")


def device_view(doc: dict):
    """A trace that carries device tracks (one category per GPU stream, written by the CUPTI activity collector of
    utils/gpu_activity.py): the device events inside the longest host span, aggregated by kernel (copies by direction),
    with that span's wall-clock length and the time during which at least one device event ran.  None when the trace has
    no device track.  Returns ``(samples, wall_s, busy_s, window_name)``."""
    from .gpu_activity import short_name

    host, device = [], []
    for ev in doc.get("traceEvents", []):
        if ev.get("ph") != "X":
            continue
        ts, dur = float(ev.get("ts", 0.0)) / 1e6, float(ev.get("dur", 0.0)) / 1e6
        (device if _DEVICE_TRACK.match(str(ev.get("cat", ""))) else host).append((ts, ts + dur, ev["name"]))
    if not device:
        return None
    if host:
        w0, w1, window = max(host, key=lambda e: e[1] - e[0])
    else:
        w0, w1, window = min(e[0] for e in device), max(e[1] for e in device), "device events"
    inside = sorted(e for e in device if w0 <= e[0] <= w1)
    agg: dict = {}
    busy, cur = 0.0, None
    for a, b, name in inside:
        if name.startswith("memcpy") or name.startswith("memset"):
            key, cat = " ".join(name.split()[:-2]) if name.endswith(" B") else name, "copy"     # drop the byte count: one row per direction
        else:
            key, cat = short_name(name), "compute"
        rec = agg.setdefault(key, [0.0, 0, cat])
        rec[0] += b - a
        rec[1] += 1
        if cur is None or a > cur[1]:
            if cur is not None:
                busy += cur[1] - cur[0]
            cur = [a, b]
        else:
            cur[1] = max(cur[1], b)
    if cur is not None:
        busy += cur[1] - cur[0]
    samples = [KernelSample(n, r[0], r[1], None, None, r[2]) for n, r in agg.items()]
    return samples, w1 - w0, busy, window


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="diagnose a Chrome-trace JSON written by ONNX_GENAI_TRACE or /v1/debug/trace/perfetto")
    ap.add_argument("trace")
    ap.add_argument("--category", default=None, help="only events of this category (for instance 'op' for device spans)")
    ap.add_argument("--peaks", default=None, help="measured-peaks JSON (hbm_gbs, bf16_tflops_sustained)")
    args = ap.parse_args(argv)
    with open(args.trace, encoding="utf-8") as f:
        doc = json.load(f)
    view = device_view(doc) if args.category is None else None
    if view is not None:                 # device tracks present: judge device time against the host span that encloses it
        samples, wall, busy, window = view
        d = diagnose_samples(samples, RooflineAnalyzer.measured(args.peaks), wall_s=wall, device_busy_s=busy)
        d.notes.append(f"device events inside the host span '{window}' ({wall * 1e3:.3f} ms); the device was busy {busy * 1e3:.3f} ms of it")
        print(d.report())
        return 0
    samples, wall = samples_from_trace(doc, args.category)
    nested = args.category is None and len({s.category for s in samples}) > 1
    d = diagnose_samples(samples, RooflineAnalyzer.measured(args.peaks), wall_s=None if nested else wall)
    if nested:
        d.notes.append("events of several categories overlap on the timeline; pass --category to compare device time with the wall clock")
    print(d.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
