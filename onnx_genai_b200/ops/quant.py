"""MatMulNBits int4 projections on the GPU: GEMV with in-kernel dequant for decode-sized M, above that a tcgen05
GEMM whose B tiles are dequantised in shared memory (the weights stay int4 in device memory).  CPU tensors use the C++ block-wise kernel (ops.cpu), or the fp32 statement in
ops.reference when the runtime library is not built."""
from __future__ import annotations

import torch

from . import _native, launch_counts, reference, status_word, timed_region
from . import gemm as _gemm

GEMV_MAX_M = 8          # rows the GEMV kernels accept
FUSED_MAX_M = 4         # above this the tensor-core GEMM is faster than the row-specialised GEMV (measured: 8 rows 2.2 ms/step vs 16 rows 2.1 ms/step on the 0.5B shape)
_native.register("ogb_w4a16_gemv", [_native.P] * 6 + [_native.I] * 6 + [_native.P])
_native.register("ogb_w4a16_dequant", [_native.P] * 4 + [_native.I] * 3 + [_native.P])
_native.register("ogb_w4a16_gemm", [_native.P] * 6 + [_native.I] * 6 + [_native.P] * 2)
_native.register("ogb_w4a16_gemv_fused", [_native.P] * 8 + [_native.I] * 6 + [_native.F] + [_native.I] * 2 + [_native.P])
PRO_NONE, PRO_RMSNORM, PRO_SILU_MUL = 0, 1, 2
_LEGACY_GEMV = __import__("os").environ.get("OGB_W4A16_LEGACY", "0") == "1"   # A/B switch: the unspecialised 8-row GEMV


class QuantLinear:
    """y = x @ dequant(W)^T (+ bias); W in MatMulNBits layout [N, ceil(K/32), 16] uint8."""

    def __init__(self, qweight, scales, zero_points=None, bias=None, k=None, block=32, device=None):
        assert block == 32, "the GPU kernels implement block_size 32"
        dev = device or qweight.device
        self.n = qweight.shape[0]
        self.k = k or qweight.shape[1] * block
        self.qweight = qweight.contiguous().to(dev)
        self.scales_fp32 = scales.dtype == torch.float32
        self.scales = (scales.float() if self.scales_fp32 else scales.to(torch.bfloat16)).contiguous().to(dev)
        self.zp = zero_points.contiguous().to(dev) if zero_points is not None else None
        self.bias = bias.to(torch.bfloat16).contiguous().to(dev) if bias is not None else None
        self._scratch = None

    # "int4": the tensor-core GEMM with in-kernel dequant (device memory holds the int4 weights only).  "dense": the
    # earlier path, a bf16 copy of the weights built once per projection and multiplied by the bf16 GEMM; kept as the
    # A/B arm of the kernel benchmark (4x the weight bytes).
    large_m = __import__("os").environ.get("OGB_W4A16_LARGE_M", "int4")

    @classmethod
    def merge(cls, parts):
        """One projection that computes the concatenation of ``parts`` along N (same K, same quantisation form)."""
        parts = list(parts)
        first = parts[0]
        if len(parts) == 1:
            return first
        if any(p.k != first.k or (p.zp is None) != (first.zp is None) or p.scales.dtype != first.scales.dtype for p in parts):
            return None
        bias = None
        if any(p.bias is not None for p in parts):
            bias = torch.cat([p.bias if p.bias is not None else torch.zeros(p.n, dtype=torch.bfloat16, device=p.qweight.device)
                              for p in parts])
        zp = torch.cat([p.zp for p in parts]) if first.zp is not None else None
        return cls(torch.cat([p.qweight for p in parts]), torch.cat([p.scales for p in parts]), zp, bias, first.k, 32,
                   first.qweight.device)

    def dense(self, dtype=torch.float32):
        return reference.dequant_w4(self.qweight.cpu(), self.scales.float().cpu(), self.zp.cpu() if self.zp is not None else None,
                                    32, self.k).to(dtype)

    def fused(self, x, out, norm_weight=None, eps=0.0, silu_mul=False, residual=None):
        """Decode-size rows (M <= 8) on the GPU in one launch: ``out = prologue(x) @ W^T (+ bias) (+ residual)``
        with prologue = RMSNorm(x, norm_weight, eps), or SiLU(x[:, :K]) * x[:, K:], or nothing."""
        m = x.shape[0]
        assert x.is_cuda and m <= GEMV_MAX_M and x.stride(1) == 1 and out.stride(1) == 1
        pro = PRO_RMSNORM if norm_weight is not None else (PRO_SILU_MUL if silu_mul else PRO_NONE)
        if silu_mul:
            assert x.shape[1] == 2 * self.k
        lib = _native.load()
        with timed_region("w4a16_gemv_fused"):
            rc = lib.ogb_w4a16_gemv_fused(
                x.data_ptr(), self.qweight.data_ptr(), self.scales.data_ptr(), self.zp.data_ptr() if self.zp is not None else 0,
                self.bias.data_ptr() if self.bias is not None else 0, norm_weight.data_ptr() if norm_weight is not None else 0,
                residual.data_ptr() if residual is not None else 0, out.data_ptr(), m, self.n, self.k, x.stride(0), out.stride(0),
                residual.stride(0) if residual is not None else 0, float(eps), pro, int(self.scales_fp32),
                torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ogb_w4a16_gemv_fused")
        launch_counts["w4a16_gemv_fused"] += 1
        return out

    def __call__(self, x, out=None):
        m = x.shape[0]
        if not x.is_cuda:
            from . import cpu

            if cpu.available():
                return cpu.matmul_nbits(x, self.qweight, self.scales, self.zp, self.bias, self.k, out=out)
            y = x.float() @ self.dense().t()
            if self.bias is not None:
                y = y + self.bias.float()
            y = y.to(x.dtype)
            if out is not None:
                out.copy_(y)
                return out
            return y
        if out is None:
            out = torch.empty(m, self.n, dtype=torch.bfloat16, device=x.device)
        lib = _native.load()
        stream = torch.cuda.current_stream().cuda_stream
        if m <= FUSED_MAX_M and not _LEGACY_GEMV and x.stride(1) == 1:
            return self.fused(x, out)
        # shapes the tensor-core GEMM does not take (N or K not a multiple of 32) stay on the generic GEMV up to 8 rows
        if m <= GEMV_MAX_M and (_LEGACY_GEMV or self.n % 32 or self.k % 32):
            with timed_region("w4a16_gemv"):
                rc = lib.ogb_w4a16_gemv(x.data_ptr(), self.qweight.data_ptr(), self.scales.data_ptr(),
                                        self.zp.data_ptr() if self.zp is not None else 0,
                                        self.bias.data_ptr() if self.bias is not None else 0, out.data_ptr(), m, self.n, self.k,
                                        x.stride(0), out.stride(0), int(self.scales_fp32), stream)
            _native.check(rc, "ogb_w4a16_gemv")
            launch_counts["w4a16_gemv"] += 1
            return out
        if self.large_m == "int4" and self.k % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and out.stride(0) % 8 == 0:
            with timed_region("w4a16_gemm"):
                rc = lib.ogb_w4a16_gemm(x.data_ptr(), self.qweight.data_ptr(), self.scales.data_ptr(),
                                        self.zp.data_ptr() if self.zp is not None else 0,
                                        self.bias.data_ptr() if self.bias is not None else 0, out.data_ptr(), m, self.n, self.k,
                                        x.stride(0), out.stride(0), int(self.scales_fp32), status_word(x.device).data_ptr(), stream)
            _native.check(rc, "ogb_w4a16_gemm")
            launch_counts["w4a16_gemm"] += 1
            return out
        if self._scratch is None:
            self._scratch = torch.empty(self.n, self.k, dtype=torch.bfloat16, device=x.device)
            with timed_region("w4a16_dequant"):
                rc = lib.ogb_w4a16_dequant(self.qweight.data_ptr(), self.scales.data_ptr(), self.zp.data_ptr() if self.zp is not None else 0,
                                           self._scratch.data_ptr(), self.n, self.k, int(self.scales_fp32), stream)
            _native.check(rc, "ogb_w4a16_dequant")
            launch_counts["w4a16_dequant"] += 1
        return _gemm(x, self._scratch, bias=self.bias, out=out)

    def device_weight_bytes(self) -> int:
        """Bytes this projection holds in device memory (int4 weights, scales, zero points, bias and, on the dense path, the bf16 copy)."""
        n = self.qweight.numel() + self.scales.numel() * self.scales.element_size()
        n += self.zp.numel() if self.zp is not None else 0
        n += self.bias.numel() * 2 if self.bias is not None else 0
        n += self._scratch.numel() * 2 if self._scratch is not None else 0
        return n
