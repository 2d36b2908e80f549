"""Prometheus text exposition of the serving counters.

Same metric families as the reference's atomic registry (crates/onnx-genai-server/src/metrics.rs:
13-115): per-endpoint x status request counts, prompt / completion tokens, TTFT and end-to-end
histograms over 14 buckets from 5 ms to 5 s, rejections; gauges are passed in at render time.
"""
from __future__ import annotations

import threading

BUCKETS = [0.005, 0.01, 0.02, 0.035, 0.05, 0.075, 0.1, 0.15, 0.25, 0.5, 1.0, 2.0, 3.5, 5.0]


class _Hist:
    def __init__(self):
        self.counts = [0] * (len(BUCKETS) + 1)
        self.sum = 0.0
        self.n = 0

    def observe(self, v):
        self.sum += v
        self.n += 1
        for i, b in enumerate(BUCKETS):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def render(self, name):
        out, cum = [f"# TYPE {name} histogram"], 0
        for b, c in zip(BUCKETS, self.counts):
            cum += c
            out.append(f'{name}_bucket{{le="{b}"}} {cum}')
        out.append(f'{name}_bucket{{le="+Inf"}} {self.n}')
        out.append(f"{name}_sum {self.sum:.6f}")
        out.append(f"{name}_count {self.n}")
        return out


class Metrics:
    def __init__(self):
        self.lock = threading.Lock()
        self.requests: dict = {}
        self.prompt = 0
        self.completion = 0
        self.rejections = 0
        self.h_ttft, self.h_e2e = _Hist(), _Hist()

    def request(self, path, status, seconds):
        with self.lock:
            self.requests[(path, status)] = self.requests.get((path, status), 0) + 1

    def prompt_tokens(self, n):
        with self.lock:
            self.prompt += n

    def completion_tokens(self, n):
        with self.lock:
            self.completion += n

    def rejected(self):
        with self.lock:
            self.rejections += 1

    def ttft(self, s):
        with self.lock:
            self.h_ttft.observe(s)

    def e2e(self, s):
        with self.lock:
            self.h_e2e.observe(s)

    def render(self, extra=None) -> str:
        with self.lock:
            lines = ["# TYPE onnx_genai_requests_total counter"]
            for (path, status), n in sorted(self.requests.items()):
                lines.append(f'onnx_genai_requests_total{{endpoint="{path}",status="{status}"}} {n}')
            lines += ["# TYPE onnx_genai_prompt_tokens_total counter", f"onnx_genai_prompt_tokens_total {self.prompt}",
                      "# TYPE onnx_genai_completion_tokens_total counter", f"onnx_genai_completion_tokens_total {self.completion}",
                      "# TYPE onnx_genai_rejections_total counter", f"onnx_genai_rejections_total {self.rejections}"]
            lines += self.h_ttft.render("onnx_genai_ttft_seconds")
            lines += self.h_e2e.render("onnx_genai_e2e_seconds")
            for k, v in (extra or {}).items():
                kind = "counter" if k.endswith("_total") else "gauge"
                lines += [f"# TYPE {k} {kind}", f"{k} {v}"]
        return "\n".join(lines) + "\n"
