"""Typed registry of the ``ONNX_GENAI_*`` environment knobs, read once.

Counterpart of `onnx-genai-runtime-config` (crates/onnx-genai-runtime-config/src/lib.rs:118-...).
Precedence everywhere: command-line flag > environment > model metadata default > built-in.
Knobs that named execution providers or NVRTC options in the reference have no meaning here and
are accepted but ignored with a note in ``ignored``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field


def _bool(v, default):
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")


@dataclass
class RuntimeConfig:
    cuda_device: int = 0
    cuda_graph: bool = True
    require_cuda: bool = False
    profile: bool = False
    trace_path: str | None = None
    trace_verbosity: str = "decisions"
    backend: str = "native"
    kv_min_bucket: int = 256
    device_token_loop_k: int = 1
    spec_tokens: int = 4
    decode_splits: int = 0
    baseline_gemm: bool = False
    ignored: dict = field(default_factory=dict)

    @classmethod
    def from_env(cls, env=None) -> "RuntimeConfig":
        env = os.environ if env is None else env
        g = lambda k: env.get("ONNX_GENAI_" + k)
        cfg = cls(cuda_device=int(g("CUDA_DEVICE") or 0), cuda_graph=_bool(g("CUDA_GRAPH"), True),
                  require_cuda=_bool(g("REQUIRE_CUDA"), False), profile=_bool(g("PROFILE"), False), trace_path=g("TRACE"),
                  trace_verbosity=g("TRACE_VERBOSITY") or "decisions", backend=g("BACKEND") or "native",
                  kv_min_bucket=int(g("KV_MIN_BUCKET") or 256), device_token_loop_k=int(g("DEVICE_TOKEN_LOOP_K") or 1),
                  spec_tokens=int(g("SPEC_TOKENS") or 4), decode_splits=int(g("CUDA_GQA_SPLITS") or 0),
                  baseline_gemm=_bool(g("BASELINE_GEMM"), False))
        if cfg.trace_verbosity not in ("decisions", "ops", "full"):
            raise ValueError(f"ONNX_GENAI_TRACE_VERBOSITY={cfg.trace_verbosity!r}: expected decisions | ops | full")
        for k in ("EP", "ORT_LIB", "ORT_LIB_DIR", "INTRA_OP_THREADS", "MARLIN_M_GT_1", "GEMV_PIPELINE", "DOWN_COLS", "CUDA_KV_LAYOUT"):
            if g(k) is not None:
                cfg.ignored["ONNX_GENAI_" + k] = "no execution-provider / NVRTC layer exists in this runtime"
        return cfg


    def describe(self) -> dict:
        """What the engine loader will do with the environment (served by ``/v1/debug/config`` and ``show``)."""
        return {"cuda_device": self.cuda_device, "cuda_graph": self.cuda_graph, "require_cuda": self.require_cuda,
                "profile": self.profile, "trace_path": self.trace_path, "trace_verbosity": self.trace_verbosity,
                "backend": self.backend, "spec_tokens": self.spec_tokens, "decode_splits": self.decode_splits,
                "baseline_gemm": self.baseline_gemm, "ignored": dict(self.ignored)}

    def default_device(self, cuda_available: bool) -> str:
        """The device an engine loads on when the caller names none: ``cuda:<ONNX_GENAI_CUDA_DEVICE>`` when CUDA is there,
        else the CPU -- unless ``ONNX_GENAI_REQUIRE_CUDA`` forbids that fallback."""
        if cuda_available:
            return f"cuda:{self.cuda_device}"
        if self.require_cuda:
            raise RuntimeError("ONNX_GENAI_REQUIRE_CUDA is set but no CUDA device is available; unset it to run on the CPU")
        return "cpu"

    def apply_engine_defaults(self, engine_kw: dict, on_cuda: bool) -> dict:
        """Fill engine options the caller left open from the environment (a caller's explicit value always wins)."""
        engine_kw.setdefault("cuda_graphs", bool(on_cuda and self.cuda_graph))
        if self.decode_splits > 0:
            engine_kw.setdefault("decode_splits", self.decode_splits)
        return engine_kw


_CACHED = None


def runtime_config(refresh: bool = False) -> RuntimeConfig:
    global _CACHED
    if _CACHED is None or refresh:
        _CACHED = RuntimeConfig.from_env()
    return _CACHED
