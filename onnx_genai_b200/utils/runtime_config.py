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


_CACHED = None


def runtime_config() -> RuntimeConfig:
    global _CACHED
    if _CACHED is None:
        _CACHED = RuntimeConfig.from_env()
    return _CACHED
