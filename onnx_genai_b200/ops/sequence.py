"""CUDA kernels behind the graph executor's hybrid / sparse decoder operators (csrc/kernels/sequence_ops.cu): recurrent
linear attention, the causal convolution with a rolling state, attention over selected cache positions and the checked
sparse row gather.  Each wrapper returns ``None`` when the kernel does not take the call (CPU tensors, a dtype or width
outside its range), and the executor then runs its torch statement of the same operator."""
from __future__ import annotations

import ctypes

import torch

from . import _native, launch_counts, status_word, timed_region

_native.register("ogb_linear_attention", [_native.P] * 8 + [_native.I] * 11 + [_native.F, _native.I, _native.P])
_native.register("ogb_causal_conv_state", [_native.P] * 6 + [_native.I] * 6 + [_native.P])
_native.register("ogb_index_share_attention", [_native.P] * 6 + [_native.I] * 8 + [_native.P, _native.F, _native.I, _native.P, _native.P])
_native.register("ogb_sparse_kv_gather", [_native.P] * 4 + [_native.I] * 6 + [_native.P] * 2)

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _ok(*tensors) -> bool:
    first = next(t for t in tensors if t is not None)
    return (first.is_cuda and first.dtype in _DT
            and all(t is None or (t.is_cuda and t.dtype == first.dtype) for t in tensors))


def _ptr(t):
    return t.data_ptr() if t is not None else 0


def _stream():
    return torch.cuda.current_stream().cuda_stream


def linear_attention(q, k, v, past, decay, beta, hq: int, hkv: int, rule: str, scale: float):
    """(out [B, T, max(hq, hkv) * dv], state [B, hkv, dk, dv]) or None."""
    if not _ok(q, k, v, past, decay, beta):
        return None
    b, t = q.shape[0], q.shape[1]
    dk, dv = q.shape[2] // hq, v.shape[2] // hkv
    nk = k.shape[2] // dk
    group = hq // hkv if hq >= hkv else 1
    if dk not in (32, 64, 128) or group > 8:
        return None
    use_decay, use_delta = rule in ("gated", "gated_delta"), rule in ("delta", "gated_delta")
    decay_per_dim = 0
    if use_decay:
        per = decay.numel() // max(1, b * t * hkv)
        if per not in (1, dk):
            return None
        decay_per_dim = int(per == dk)
    beta_heads = hkv
    if use_delta:
        beta_heads = beta.numel() // max(1, b * t)
        if beta_heads not in (1, hkv):
            return None
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    past = past.contiguous() if past is not None else None
    decay = decay.contiguous() if decay is not None else None
    beta = beta.contiguous() if beta is not None else None
    out = torch.empty(b, t, max(hq, hkv) * dv, dtype=q.dtype, device=q.device)
    state = torch.empty(b, hkv, dk, dv, dtype=q.dtype, device=q.device)
    with timed_region("linear_attention"):
        rc = _native.load().ogb_linear_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(past), _ptr(decay) if use_decay else 0,
                                                 _ptr(beta) if use_delta else 0, _ptr(out), _ptr(state), b, t, hq, nk, hkv, dk, dv,
                                                 decay_per_dim, beta_heads, int(use_decay), int(use_delta), float(scale), _DT[q.dtype], _stream())
    if rc == -2:
        return None
    _native.check(rc, "ogb_linear_attention")
    launch_counts["linear_attention"] += 1
    return out, state


def causal_conv_state(x, w, bias, past, silu: bool):
    """(y [B, C, L], state [B, C, K-1]) of the depthwise causal convolution, or None."""
    if not _ok(x, w, bias, past) or x.dim() != 3 or w.dim() != 3 or w.shape[1] != 1:
        return None
    b, c, l = x.shape
    k = w.shape[2]
    x, w = x.contiguous(), w.contiguous()
    bias = bias.contiguous() if bias is not None else None
    past = past.contiguous() if past is not None else None
    y = torch.empty_like(x)
    state = torch.empty(b, c, k - 1, dtype=x.dtype, device=x.device)
    with timed_region("causal_conv_state"):
        rc = _native.load().ogb_causal_conv_state(_ptr(x), _ptr(w), _ptr(bias), _ptr(past), _ptr(y), _ptr(state), b, c, l, k, int(silu),
                                                  _DT[x.dtype], _stream())
    _native.check(rc, "ogb_causal_conv_state")
    launch_counts["causal_conv_state"] += 1
    return y, state


def index_share_attention(q, k, v, sel, bias, scale: float):
    """q [B, N, Sq, D] over the selected rows of k / v [B, Nkv, total, D]; ``sel`` int64 [B, 1 or N, Sq, K] (validated by
    the caller), ``bias`` broadcastable to [B, N, Sq, total].  Returns out [B, N, Sq, D] or None."""
    if not _ok(q, k, v) or sel.dtype != torch.int64 or not sel.is_cuda:
        return None
    b, n, sq, d = q.shape
    nkv, total = k.shape[1], k.shape[2]
    if d % 32 or d > 256 or v.shape[3] != d:
        return None
    strides = None
    if bias is not None:
        if bias.dtype != q.dtype or not bias.is_cuda:
            return None
        view = bias.expand(b, n, sq, total)                  # broadcast dimensions get stride 0
        strides = (ctypes.c_longlong * 4)(*view.stride())
        bias = view
    q, k, v, sel = q.contiguous(), k.contiguous(), v.contiguous(), sel.contiguous()
    out = torch.empty_like(q)
    with timed_region("index_share_attention"):
        rc = _native.load().ogb_index_share_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(sel), _ptr(bias), _ptr(out), b, n, nkv, sq, total, d,
                                                      sel.shape[3], sel.shape[1], ctypes.cast(strides, ctypes.c_void_p) if strides is not None else 0,
                                                      float(scale), _DT[q.dtype], status_word(q.device).data_ptr(), _stream())
    if rc == -2:
        return None
    _native.check(rc, "ogb_index_share_attention")
    launch_counts["index_share_attention"] += 1
    return out


def sparse_kv_gather(cache, idx, lengths):
    """cache [B, G, C, D], idx int64 [B, G, Q, K], optional lengths int64 [B] -> [B, G, Q, K, D] or None.  Indices outside
    a row's valid range raise the device status word (the caller decides when to read it)."""
    if not (cache.is_cuda and idx.is_cuda and idx.dtype == torch.int64):
        return None
    b, g, c, d = cache.shape
    qn, kn = idx.shape[2], idx.shape[3]
    cache, idx = cache.contiguous(), idx.contiguous()
    lengths = lengths.to(torch.int64).contiguous() if lengths is not None else None
    out = torch.empty(b, g, qn, kn, d, dtype=cache.dtype, device=cache.device)
    with timed_region("sparse_kv_gather"):
        rc = _native.load().ogb_sparse_kv_gather(_ptr(cache), _ptr(idx), _ptr(lengths), _ptr(out), b, g, c, qn, kn, d * cache.element_size(),
                                                 status_word(cache.device).data_ptr(), _stream())
    _native.check(rc, "ogb_sparse_kv_gather")
    launch_counts["sparse_kv_gather"] += 1
    return out
