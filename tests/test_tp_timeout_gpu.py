"""Failure detection on the device without a fault: a wait on another rank's signal that can never be satisfied runs
out after its limit, the kernel returns, the status word says why, and the GPU keeps working.

The group is a loopback (two "ranks" that alias one GPU's region, plain loads, no multicast), so the arrivals a
real peer would send never come.  Nothing here traps, faults or spins without a bound."""
import time

import pytest
import torch

from onnx_genai_b200 import ops
from onnx_genai_b200.ops import _native
from onnx_genai_b200.parallel.fused import FusedComm

pytestmark = pytest.mark.gpu
HID, ROWS = 512, 256


def _group(limit_ns):
    fc = FusedComm.loopback("cuda", HID, ROWS, world=2)
    x = torch.zeros(ROWS, HID, dtype=torch.bfloat16, device="cuda")
    fc.bind_residual(x)
    fc.set_wait_limit(limit_ns)
    return fc, x


def test_exchange_gives_up_when_a_peer_never_signals():
    torch.cuda.synchronize()
    ops.check_status()
    fc, x = _group(2_000_000)                                # 2 ms
    a = (torch.randn(ROWS, 128, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(HID, 128, device="cuda") * 0.1).bfloat16()
    norm_w = torch.ones(HID, dtype=torch.bfloat16, device="cuda")
    t0 = time.perf_counter()
    fc.row_parallel_norm(a, w, ROWS, 0, norm_w, 1e-6)        # this rank's tiles arrive; the other "rank" never produces
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert took < 5.0, took                                   # returned on its own
    with pytest.raises(_native.KernelError, match="peer wait timeout"):
        ops.check_status()
    ops.check_status()                                        # the word was cleared; the context is alive
    # the device keeps working: an ordinary GEMM right after gives the right answer
    out = ops.gemm(a, w)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    assert float((out.float() - ref).norm() / ref.norm()) < 2e-2
    ops.check_status()


def test_gemm_gives_up_when_its_input_rows_never_arrive():
    torch.cuda.synchronize()
    ops.check_status()
    fc, _ = _group(2_000_000)
    a = (torch.randn(ROWS, HID, device="cuda") * 0.1).bfloat16()
    w = (torch.randn(256, HID, device="cuda") * 0.1).bfloat16()
    t0 = time.perf_counter()
    ops.gemm(a, w, a_ready=fc.ready_ptrs(1))                 # nobody bumps the ready counters
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 10.0
    with pytest.raises(_native.KernelError, match="timeout"):
        ops.check_status()
    fc.reset_counters()
    out = ops.gemm(a, w)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    assert float((out.float() - ref).norm() / ref.norm()) < 2e-2
    ops.check_status()


def test_engine_turns_the_status_word_into_a_request_failure():
    """LLMEngine.step reads the status word with the step's tokens and raises before anything is committed."""
    import numpy as np

    from onnx_genai_b200.engine.llm_engine import EngineConfig, LLMEngine
    from onnx_genai_b200.models.config import DecoderConfig

    cfg = DecoderConfig(name="st", num_layers=1, hidden=128, num_heads=2, num_kv_heads=1, head_dim=64, intermediate=256,
                        vocab=512, rope_theta=1e4, tie_embeddings=True, qkv_bias=False, max_position=256)
    eng = LLMEngine(EngineConfig(model=cfg, num_pages=32, max_seqs=4, max_tokens_per_step=64, max_seq_len=128), device="cuda")
    sid = eng.add_request(np.arange(10, dtype=np.int32), 4)
    eng.step()
    ops.status_word("cuda").fill_(ops.STATUS_INDEX_OUT_OF_RANGE)      # what a kernel that met a bad page id would leave
    before = eng.core.seq_len(sid)
    with pytest.raises(_native.KernelError, match="index out of range"):
        eng.step()
    assert eng.core.seq_len(sid) == before and eng.device_faults == 1   # nothing was committed
    ops.check_status()                                                 # the engine cleared the word
