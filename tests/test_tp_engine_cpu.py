"""Tensor parallelism through the public API on CPU ranks (gloo): rank 0 serves `Engine.generate*`, the other rank
follows the broadcast commands; tokens equal a single-rank engine over the same package."""
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, out, port):
    env = dict(os.environ, PYTHONPATH=ROOT, OGB_TEST_DEVICE="cpu", CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    worker = os.path.join(ROOT, "tests", "tp_engine_worker.py")
    cmd = [sys.executable, worker, out] if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
        "--master-port", str(port), worker, out]
    if nproc == 1:
        env.pop("WORLD_SIZE", None)
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if proc.returncode != 0 and nproc > 1 and "--master-port" in cmd:      # the fixed port may be taken: once more on a free one
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            cmd[cmd.index("--master-port") + 1] = str(s.getsockname()[1])
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    return torch.load(out)


def test_two_rank_engine_serves_like_one_rank(tmp_path):
    one = _run(1, str(tmp_path / "one.pt"), 0)
    two = _run(2, str(tmp_path / "two.pt"), 29671)
    assert two["world"] == 2 and one["world"] == 1
    assert two["greedy"] == one["greedy"] and two["streamed"] == one["streamed"]
    assert len(two["sampled"]) == 8                       # a sampled request runs on the device sampler of every rank alike
    assert "not available under tensor parallelism" in two["refused"]


def test_cli_generate_under_a_launcher_prints_what_one_process_prints(tmp_path):
    """`torchrun -m onnx_genai_b200 generate`: rank 0 answers, rank 1 follows and exits with it; an uneven split of the
    MLP width (688 over 2 ranks in 16-wide units) is part of the case."""
    from onnx_genai_b200.bench.config_bench import _export

    d = str(tmp_path / "m")
    _export("tiny-llama", d, "fp32", layers=1)
    args = ["-m", "onnx_genai_b200", "generate", d, "--prompt", "the quick brown fox", "--max-new-tokens", "6", "--greedy", "--device", "cpu", "--raw"]
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    for k in ("WORLD_SIZE", "RANK", "LOCAL_RANK"):
        env.pop(k, None)
    one = subprocess.run([sys.executable] + args, env=env, capture_output=True, text=True, timeout=600)
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29673"] + args, env=env, capture_output=True, text=True, timeout=600)
    assert one.returncode == 0 and two.returncode == 0, two.stderr[-3000:]
    assert two.stdout == one.stdout and "rank 1: followed" in two.stderr
    spec = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                           "--master-port", "29674"] + args + ["--speculative"], env=env, capture_output=True, text=True, timeout=600)
    assert spec.returncode != 0 and "not available under tensor parallelism" in spec.stderr
