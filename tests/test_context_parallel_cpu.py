"""Context parallelism (parallel/context_parallel.py): the partial-attention merge, the partitions, and ring attention over
gloo ranks against dense causal attention on one process."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from onnx_genai_b200.parallel import context_parallel as cp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _dense(q, k, v, window=0):
    b, hq, t, d = q.shape
    g = hq // k.shape[1]
    kk, vv = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
    s = (q.float() @ kk.float().transpose(-1, -2)) / d ** 0.5
    pos = torch.arange(t)
    ok = pos[None, :] <= pos[:, None]
    if window:
        ok &= pos[None, :] > pos[:, None] - window
    s = s.masked_fill(~ok, float("-inf"))
    return torch.softmax(s, -1) @ vv.float(), torch.logsumexp(s, -1)


def test_merge_of_two_key_halves_is_attention_over_all_keys():
    torch.manual_seed(1)
    q, k, v = torch.randn(1, 4, 9, 16), torch.randn(1, 2, 30, 16), torch.randn(1, 2, 30, 16)
    qpos, kpos = torch.arange(21, 30), torch.arange(30)
    whole, lse = cp.block_attention(q, k, v, qpos, kpos, 0.25)
    a = cp.block_attention(q, k[:, :, :13], v[:, :, :13], qpos, kpos[:13], 0.25)
    b = cp.block_attention(q, k[:, :, 13:], v[:, :, 13:], qpos, kpos[13:], 0.25)
    merged, mlse = cp.merge_partials(*a, *b)
    assert torch.allclose(merged, whole, atol=1e-5) and torch.allclose(mlse, lse, atol=1e-5)
    # a block wholly in the future contributes nothing and does not poison the merge with NaNs
    fut = cp.block_attention(q, k[:, :, :4], v[:, :, :4], qpos, torch.arange(40, 44), 0.25)
    assert torch.isinf(fut[1]).all() and float(fut[0].abs().max()) == 0
    again, alse = cp.merge_partials(whole, lse, *fut)
    assert torch.allclose(again, whole) and torch.allclose(alse, lse) and not torch.isnan(again).any()


def test_zigzag_partition_balances_causal_work():
    total, world = 4096, 8
    zig, run = cp.zigzag_slices(total, world), cp.contiguous_slices(total, world)
    for part in (zig, run):
        assert torch.equal(torch.sort(torch.cat(part)).values, torch.arange(total))
    zp, rp = cp.causal_pairs(zig), cp.causal_pairs(run)
    assert max(zp) / (sum(zp) / world) < 1.01              # even to within a chunk's rounding
    assert max(rp) / (sum(rp) / world) > 1.8               # the last contiguous run does nearly twice the mean
    assert cp.ring_bytes_per_rank(1, 4, 128, 4096, 8) == 2 * 4 * 4096 * 128 * 2 * 7


@pytest.mark.parametrize("world,mode", [(2, "contiguous"), (3, "zigzag"), (4, "zigzag-window"), (3, "contiguous-window")])
def test_ring_attention_over_gloo_ranks_equals_dense(tmp_path, world, mode):
    out = str(tmp_path / "cp.pt")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "cp_worker.py"), out, mode]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-4000:]
    got = torch.load(out)
    want, want_lse = _dense(got["q"], got["k"], got["v"], got["window"])
    assert got["world"] == world
    assert torch.allclose(got["out"], want, atol=2e-5) and torch.allclose(got["lse"], want_lse, atol=2e-5)


def test_whole_decoder_prefill_split_over_three_ranks(tmp_path):
    """Every token-wise operator on a rank's tokens, attention over the ring: hidden rows and roped K / V rows equal the
    one-rank schedule, and the first token equals the engine's."""
    out = str(tmp_path / "cpm.pt")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "cp_worker.py"), out, "model"]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-4000:]
    got = torch.load(out)
    assert torch.allclose(got["hidden"], got["want_hidden"], atol=1e-4)
    for a, b in zip(got["k"] + got["v"], got["want_k"] + got["want_v"]):
        assert torch.allclose(a, b, atol=1e-4)
    assert got["first_cp"] == int(got["first_engine"])
