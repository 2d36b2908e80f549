"""MatMulNBits int4 projections on the GPU: GEMV with in-kernel dequant for decode-sized M, dequant +
tcgen05 GEMM above that.  CPU tensors use the C++ block-wise kernel (ops.cpu), or the fp32 statement in
ops.reference when the runtime library is not built."""
from __future__ import annotations

import torch

from . import _native, launch_counts, reference, status_word, timed_region
from . import gemm as _gemm

GEMV_MAX_M = 8
_native.register("ogb_w4a16_gemv", [_native.P] * 6 + [_native.I] * 6 + [_native.P])
_native.register("ogb_w4a16_dequant", [_native.P] * 4 + [_native.I] * 3 + [_native.P])


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

    def dense(self, dtype=torch.float32):
        return reference.dequant_w4(self.qweight.cpu(), self.scales.float().cpu(), self.zp.cpu() if self.zp is not None else None,
                                    32, self.k).to(dtype)

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
        if m <= GEMV_MAX_M:
            with timed_region("w4a16_gemv"):
                rc = lib.ogb_w4a16_gemv(x.data_ptr(), self.qweight.data_ptr(), self.scales.data_ptr(),
                                        self.zp.data_ptr() if self.zp is not None else 0,
                                        self.bias.data_ptr() if self.bias is not None else 0, out.data_ptr(), m, self.n, self.k,
                                        x.stride(0), out.stride(0), int(self.scales_fp32), stream)
            _native.check(rc, "ogb_w4a16_gemv")
            launch_counts["w4a16_gemv"] += 1
            return out
        if self._scratch is None:
            self._scratch = torch.empty(self.n, self.k, dtype=torch.bfloat16, device=x.device)
        with timed_region("w4a16_dequant"):
            rc = lib.ogb_w4a16_dequant(self.qweight.data_ptr(), self.scales.data_ptr(), self.zp.data_ptr() if self.zp is not None else 0,
                                       self._scratch.data_ptr(), self.n, self.k, int(self.scales_fp32), stream)
        _native.check(rc, "ogb_w4a16_dequant")
        launch_counts["w4a16_dequant"] += 1
        return _gemm(x, self._scratch, bias=self.bias, out=out)
