"""Tensor parallelism with CPU ranks (gloo): the host-side logic -- head / column / expert sharding, replicas that
schedule identically, the row-split lm_head + sampler with its token all-gather -- against a single rank."""
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(nproc, mode, out, port, **extra_env):
    env = dict(os.environ, PYTHONPATH=ROOT, OGB_TEST_DEVICE="cpu", CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", **extra_env)
    worker = os.path.join(ROOT, "tests", "tp_worker.py")
    if nproc == 1:
        cmd = [sys.executable, worker, mode, out]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(port), worker, mode, out]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if proc.returncode != 0 and nproc > 1 and "--master-port" in cmd:      # the fixed port may be taken: once more on a free one
        import socket

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            cmd[cmd.index("--master-port") + 1] = str(s.getsockname()[1])
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    return torch.load(out)


def test_two_cpu_ranks_match_one_rank_dense_and_moe(tmp_path):
    for suffix, port in (("", 29651), ("-moe", 29652)):
        single = _run(1, "nccl" + suffix, str(tmp_path / f"s{suffix}.pt"), 0)
        pair = _run(2, "nccl" + suffix, str(tmp_path / f"p{suffix}.pt"), port)
        assert pair["backend"] == "gloo"
        err = float((pair["logits"] - single["logits"]).norm() / single["logits"].norm())
        assert err < 1e-4, (suffix, err)                       # fp32: only the summation order differs
        assert pair["tokens"] == single["tokens"], suffix      # greedy tokens of every request, step by step


def test_four_cpu_ranks_replicate_kv_heads(tmp_path):
    """8 query heads / 2 KV heads over 4 ranks: each KV head is held by two ranks."""
    single = _run(1, "nccl", str(tmp_path / "s.pt"), 0)
    four = _run(4, "nccl", str(tmp_path / "t.pt"), 29653)
    err = float((four["logits"] - single["logits"]).norm() / single["logits"].norm())
    assert err < 1e-4, err
    assert four["tokens"] == single["tokens"]


def test_pipeline_stages_on_cpu_ranks_match_one_rank(tmp_path):
    """Two and three pipeline stages (the three layers split 2 + 1 and 1 + 1 + 1): the residual stream crosses stages by
    send / recv, the last stage samples, every stage commits the same tokens as a single process."""
    single = _run(1, "nccl", str(tmp_path / "s.pt"), 0)
    for stages, port in ((2, 29655), (3, 29656)):
        piped = _run(stages, "pp", str(tmp_path / f"pp{stages}.pt"), port)
        err = float((piped["logits"] - single["logits"]).norm() / single["logits"].norm())
        assert err < 1e-5, (stages, err)
        assert piped["tokens"] == single["tokens"], stages


def test_communicator_exchanges_and_expert_dispatch_over_gloo(tmp_path):
    res = _run(3, "comm-api", str(tmp_path / "c.pt"), 29654)
    assert res["backend"] == "gloo" and res["world"] == 3
    assert res["recv"] == [s + 0 + 1 for s in range(3)]                    # what each source sends to rank 0
    assert res["rows"] == [[s, 0] for s in range(3) for _ in range(s + 1)]
    assert res["ring"] == 2.0 and res["ep_ok"] == 3


def test_token_sharded_expert_dispatch_in_the_engine_matches_one_rank(tmp_path):
    """`OGB_EP_DISPATCH=a2a`: each rank routes its slice of the rows, rows travel to the experts' owners and back
    (exchange_counts + all_to_all_v), an all-gather restores the replicated rows; against one rank holding every expert,
    over 2 and 4 ranks (4: some rows' slices are empty in decode steps with fewer rows than ranks)."""
    one = _run(1, "nccl-moe", str(tmp_path / "o.pt"), 0)
    for world, port in ((2, 29657), (4, 29658)):
        got = _run(world, "nccl-moe", str(tmp_path / f"a{world}.pt"), port, OGB_EP_DISPATCH="a2a")
        err = float((got["logits"] - one["logits"]).norm() / one["logits"].norm())
        assert err < 1e-4, (world, err)
        assert got["tokens"] == one["tokens"]
        assert got["launches"].get("ep_dispatch_a2a", 0) > 0 and one["launches"].get("ep_dispatch_a2a", 0) == 0
