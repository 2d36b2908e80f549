"""The allocation-free sampler entry point, called through its exported C symbol.

Some embedders may not allocate device memory once they are running (a plugin inside another
runtime's memory plan, a server whose device memory is fully owned by a pool).  For them the
library exports ``ogb_sample_bf16_no_alloc``, whose scratch is a fixed array in the library image.
This test calls that symbol directly with ctypes, twice in a row (the array is shared between
calls and keeps the previous call's contents), and checks the tokens against the regular entry
point that takes a caller-allocated work buffer.  The file sorts last so a run that stops at the
first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.ops import _native

pytestmark = pytest.mark.gpu


def _call(lib, logits, params, rows, vocab, out=None):
    temperature, top_k, top_p, min_p, u = params
    if out is None:
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    fn = lib.ogb_sample_bf16_no_alloc
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    rc = fn(logits.data_ptr(), out.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
            u.data_ptr(), rows, vocab, logits.stride(0), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_no_alloc_sampler_matches_regular_entry_point_twice():
    lib = _native.load()
    torch.manual_seed(123)
    rows = 4
    for call, vocab in enumerate((32000, 151936)):          # second call reuses the array after a different shape
        logits = (torch.randn(rows, vocab, device="cuda") * 3).bfloat16()
        params = (torch.tensor([0.7, 1.0, 0.0, 1.3], device="cuda"), torch.tensor([0, 40, 0, 5], dtype=torch.int32, device="cuda"),
                  torch.tensor([0.9, 1.0, 1.0, 0.8], device="cuda"), torch.tensor([0.0, 0.05, 0.0, 0.0], device="cuda"),
                  torch.rand(rows, device="cuda"))
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        rc, got = _call(lib, logits, params, rows, vocab, out)
        torch.cuda.synchronize()
        assert rc == 0, rc
        want = ops.sample(logits, *params)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want.cpu()), (call, got.tolist(), want.tolist())


def test_no_alloc_sampler_rejects_sizes_beyond_its_array():
    lib = _native.load()
    logits = torch.zeros(5, 64, device="cuda", dtype=torch.bfloat16)
    p = (torch.ones(5, device="cuda"), torch.zeros(5, dtype=torch.int32, device="cuda"), torch.ones(5, device="cuda"),
         torch.zeros(5, device="cuda"), torch.rand(5, device="cuda"))
    rc, out = _call(lib, logits, p, 5, 64)
    assert rc == -3 and int(out[0]) == -1                       # refused: nothing was launched
    rc, _ = _call(lib, logits, p, 1, 262145)
    assert rc == -3
    rc, _ = _call(lib, logits, p, 1, 128)                        # a row stride (64) shorter than the vocabulary
    assert rc == -3
