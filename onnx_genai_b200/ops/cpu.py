"""ctypes bindings for the C++ CPU kernels (``csrc/cpu_ref/cpu_ref.cpp``, built into ``libogb_runtime.so``).

These kernels are the executor of the CPU-only configuration and an oracle for the CUDA kernels that is
independent of PyTorch.  Every function takes fp32 CPU tensors; ``available()`` is False when the
library could not be built, and the callers in :mod:`onnx_genai_b200.ops` then use the PyTorch statements
in :mod:`onnx_genai_b200.ops.reference`.  ``OGB_CPU_KERNELS=torch`` forces that fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

_LIB = None
_TRIED = False
calls: dict = {}


def _lib():
    global _LIB, _TRIED
    if _TRIED:
        return _LIB
    _TRIED = True
    if os.environ.get("OGB_CPU_KERNELS", "native") == "torch":
        return None
    try:
        from ..engine.core import load_runtime

        lib = load_runtime()
        P, I, L, F = c_void_p, c_int, c_int64, c_float
        sigs = {
            "ogb_cpu_matmul_nbits": [P, L, P, P, P, P, P, L, I, I, I],
            "ogb_cpu_gemm": [P, L, P, L, P, P, L, P, L, I, I, I],
            "ogb_cpu_rmsnorm": [P, P, P, P, I, I, F],
            "ogb_cpu_silu_mul": [P, L, P, I, I],
            "ogb_cpu_rope_kv_append": [P, P, P, P, I, P, L, I, I, I, I, I, I],
            "ogb_cpu_paged_attention": [P, L, P, P, P, I, P, P, I, I, I, I, F, I, I],
            "ogb_cpu_argmax": [P, L, P, I, I],
            "ogb_cpu_sample": [P, L, P, P, P, P, P, P, I, I],
            "ogb_cpu_dequant_nbits": [P, P, P, P, I, I],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        _LIB = lib
    except Exception:   # the PyTorch statements stay available
        _LIB = None
    return _LIB


def available() -> bool:
    return _lib() is not None


def _f32(t: torch.Tensor) -> torch.Tensor:
    assert t.device.type == "cpu"
    return t if t.dtype == torch.float32 else t.float()


def _rows(t: torch.Tensor) -> torch.Tensor:
    """fp32 tensor whose last dimension is contiguous (row stride may be anything)."""
    t = _f32(t)
    return t if t.stride(-1) == 1 else t.contiguous()


def _count(name):
    calls[name] = calls.get(name, 0) + 1


def matmul_nbits(x, qweight, scales, zero_points=None, bias=None, k=None, out=None):
    """y = x @ dequant(W)^T (+ bias) for MatMulNBits int4 block-32 weights [N, ceil(K/32), 16]."""
    lib = _lib()
    x = _rows(x)
    m = x.shape[0]
    n = qweight.shape[0]
    k = k or x.shape[1]
    scales = _f32(scales).contiguous()
    qweight = qweight.contiguous()
    y = out if (out is not None and out.dtype == torch.float32 and out.stride(-1) == 1) else torch.empty(m, n)
    bias_f = _f32(bias).contiguous() if bias is not None else None
    zp = zero_points.contiguous() if zero_points is not None else None
    rc = lib.ogb_cpu_matmul_nbits(x.data_ptr(), x.stride(0), qweight.data_ptr(), scales.data_ptr(),
                                  zp.data_ptr() if zp is not None else None, bias_f.data_ptr() if bias_f is not None else None,
                                  y.data_ptr(), y.stride(0), m, n, k)
    if rc != 0:
        raise RuntimeError(f"ogb_cpu_matmul_nbits failed ({rc})")
    _count("matmul_nbits")
    if out is not None and y is not out:
        out.copy_(y)
        return out
    return y


def gemm(x, w, bias=None, residual=None):
    lib = _lib()
    x, w = _rows(x), _rows(w)
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty(m, n)
    b = _f32(bias).contiguous() if bias is not None else None
    r = _rows(residual) if residual is not None else None
    rc = lib.ogb_cpu_gemm(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), b.data_ptr() if b is not None else None,
                          r.data_ptr() if r is not None else None, r.stride(0) if r is not None else 0, y.data_ptr(), y.stride(0),
                          m, n, k)
    if rc != 0:
        raise RuntimeError(f"ogb_cpu_gemm failed ({rc})")
    _count("gemm")
    return y


def rmsnorm(x, weight, eps, delta=None):
    """Returns (normed, new_residual); x is not modified."""
    lib = _lib()
    xr = _f32(x).contiguous().clone()
    d = _f32(delta).contiguous() if delta is not None else None
    w = _f32(weight).contiguous()
    y = torch.empty_like(xr)
    lib.ogb_cpu_rmsnorm(xr.data_ptr(), d.data_ptr() if d is not None else None, w.data_ptr(), y.data_ptr(), xr.shape[0],
                        xr.shape[1], float(eps))
    _count("rmsnorm")
    return y, xr


def silu_mul(gate_up):
    lib = _lib()
    g = _rows(gate_up)
    rows, two = g.shape
    out = torch.empty(rows, two // 2)
    lib.ogb_cpu_silu_mul(g.data_ptr(), g.stride(0), out.data_ptr(), rows, two // 2)
    _count("silu_mul")
    return out


def rope_kv_append(qkv, positions, slots, cos_sin, pool, hq, hkv, d, rotary_dim=None, interleaved=False):
    """In place on fp32 contiguous ``qkv`` and ``pool``."""
    lib = _lib()
    assert qkv.dtype == torch.float32 and qkv.is_contiguous() and pool.dtype == torch.float32 and pool.is_contiguous()
    pos = positions.to(torch.int32).contiguous()
    sl = slots.to(torch.int32).contiguous()
    cs = _f32(cos_sin).contiguous()
    rc = lib.ogb_cpu_rope_kv_append(qkv.data_ptr(), pos.data_ptr(), sl.data_ptr(), cs.data_ptr(), cs.shape[0], pool.data_ptr(),
                                    pool.shape[0], qkv.shape[0], hq, hkv, d, rotary_dim or d, int(bool(interleaved)))
    if rc != 0:
        raise IndexError("rope_kv_append: a position or KV slot is out of range")
    _count("rope_kv_append")
    return qkv


def paged_attention(q, pool, page_table, ctx_len, cu_q, hq, hkv, d, scale=None, window=0, sink=0):
    lib = _lib()
    q = _rows(q)
    assert pool.dtype == torch.float32 and pool.is_contiguous()
    t = q.shape[0]
    out = torch.empty(t, hq * d)
    table = page_table.to(torch.int32).contiguous()
    if table.dim() == 1:
        table = table.view(1, -1)
    ctx = ctx_len.to(torch.int32).contiguous()
    cu = cu_q.to(torch.int32).contiguous()
    n = ctx.numel()
    lib.ogb_cpu_paged_attention(q.data_ptr(), q.stride(0), out.data_ptr(), pool.data_ptr(), table.data_ptr(), table.stride(0),
                                ctx.data_ptr(), cu.data_ptr(), n, hq, hkv, d, float(scale or d ** -0.5), int(window), int(sink))
    _count("paged_attention")
    return out


def argmax(logits):
    lib = _lib()
    l = _rows(logits)
    out = torch.empty(l.shape[0], dtype=torch.int32)
    lib.ogb_cpu_argmax(l.data_ptr(), l.stride(0), out.data_ptr(), l.shape[0], l.shape[1])
    _count("argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, uniform):
    lib = _lib()
    l = _rows(logits)
    rows, vocab = l.shape
    out = torch.empty(rows, dtype=torch.int32)
    t, p, mp, u = (_f32(v).contiguous() for v in (temperature, top_p, min_p, uniform))
    k = top_k.to(torch.int32).contiguous()
    lib.ogb_cpu_sample(l.data_ptr(), l.stride(0), out.data_ptr(), t.data_ptr(), k.data_ptr(), p.data_ptr(), mp.data_ptr(),
                       u.data_ptr(), rows, vocab)
    _count("sample")
    return out


def dequant_nbits(qweight, scales, zero_points=None, k=None):
    lib = _lib()
    n, kb, _ = qweight.shape
    k = k or kb * 32
    w = torch.empty(n, k)
    s = _f32(scales).contiguous()
    zp = zero_points.contiguous() if zero_points is not None else None
    lib.ogb_cpu_dequant_nbits(qweight.contiguous().data_ptr(), s.data_ptr(), zp.data_ptr() if zp is not None else None,
                              w.data_ptr(), n, k)
    return w
