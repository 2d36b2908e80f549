"""ctypes bindings of ``libogb_cuda.so`` (the sm_100a kernel library).

The library exposes a plain C ABI taking raw device pointers and a stream handle, so the Python
side passes ``tensor.data_ptr()`` and ``torch.cuda.current_stream().cuda_stream``.  On a machine
with a GPU a missing library is an error (there is no silent PyTorch fallback for CUDA tensors);
on a CPU-only machine the library is simply never loaded.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None

P = c_void_p
I = c_int
L = c_int64
F = c_float

_SIGNATURES = {
    "ogb_num_sms": ([], I),
    "ogb_gemm_bf16": ([P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P], I),
    "ogb_gemm_bf16_wait": ([P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P, ctypes.c_uint64, P, P], I),
    "ogb_gemm_set_stream_k": ([I], I),
    "ogb_tp_set_pdl": ([I], I),
    "ogb_attn_set_e4m3_mma": ([I], I),
    "ogb_rmsnorm_bf16": ([P, P, P, P, I, I, I, I, F, P], I),
    "ogb_embedding_bf16": ([P, P, P, I, I, I, P, P], I),
    "ogb_silu_mul_bf16": ([P, P, I, I, P], I),
    "ogb_rope_kv_append_bf16": ([P, P, P, P, P, I, I, I, I, I, I, I, L, I, P, P], I),
    "ogb_rope_kv_append_fp8": ([P, P, P, P, P, P, I, I, I, I, I, I, I, L, I, P, P], I),
    "ogb_paged_prefill_bf16": ([P, P, P, P, P, P, P, P, I, I, I, L, I, I, I, I, I, F, I, I, P, P], I),
    "ogb_paged_prefill_tc_bf16": ([P, P, P, P, P, P, P, P, I, I, I, I, L, I, I, I, I, I, F, I, I, P, P], I),
    "ogb_paged_decode_bf16": ([P, P, P, P, P, I, I, L, I, I, I, I, I, F, I, P, P, I, I, P, P], I),
    "ogb_paged_decode_fp8": ([P, P, P, P, P, P, I, I, L, I, I, I, I, I, F, I, P, P, P, P], I),
    "ogb_paged_prefill_fp8": ([P, P, P, P, P, P, P, P, P, I, I, I, L, I, I, I, I, I, F, P, P], I),
    "ogb_rope_kv_append_q8": ([P, P, P, P, P, P, I, I, I, I, I, I, I, I, L, I, P, P], I),
    "ogb_paged_decode_q8": ([P, P, P, P, I, P, P, I, I, L, I, I, I, I, I, F, I, P, P, I, I, P, P], I),
    "ogb_paged_prefill_q8": ([P, P, P, P, I, P, P, P, P, P, I, I, I, L, I, I, I, I, I, F, I, I, P, P], I),
    "ogb_argmax_bf16": ([P, P, I, I, I, P], I),
    "ogb_sample_bf16": ([P, P, P, P, P, P, P, P, I, I, I, P], I),
    "ogb_spec_verify_greedy": ([P, P, P, P, I, I, I, I, P], I),
    "ogb_kv_page_copy": ([P, P, P, I, L, P], I),
    "ogb_kv_gather_pages": ([P, P, P, I, L, P], I),
    "ogb_kv_scatter_pages": ([P, P, P, I, L, P], I),
    "ogb_kv_move_pages": ([P, P, I, P, P, I, L, L, L, P, P], I),
}


def lib_path() -> Path:
    return Path(__file__).resolve().parent.parent / "_lib" / "libogb_cuda.so"


def load() -> ctypes.CDLL:
    """Load (building first when the sources are newer and nvcc exists) the CUDA kernel library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        try:
            from .. import build as _build

            path = _build.build_cuda()
        except Exception as exc:  # nvcc missing on the run machine: fall back to the shipped .so
            if not path.exists():
                raise RuntimeError(
                    f"CUDA kernel library {path} is missing and could not be built ({exc}). "
                    "Run `python -m onnx_genai_b200.build` on a machine with nvcc."
                ) from exc
        lib = ctypes.CDLL(str(path))
        for name, (argtypes, restype) in _SIGNATURES.items():
            if hasattr(lib, name):
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = restype
        _LIB = lib
        return lib


def register(name: str, argtypes, restype=I) -> None:
    """Declare the signature of an extra exported symbol (used by optional kernel families)."""
    _SIGNATURES[name] = (list(argtypes), restype)
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.argtypes = list(argtypes)
        fn.restype = restype


class KernelError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        kind = "CUDA error" if rc > 0 else "argument rejected"
        raise KernelError(f"{what}: {kind} (code {rc})")
