"""Communicator point-to-point and variable-size exchanges on the CPU oracle; token-sharded expert dispatch on top."""
import threading

import pytest
import torch

from onnx_genai_b200.parallel.comm import LocalComm
from onnx_genai_b200.parallel.ep_dispatch import EpDispatcher
from onnx_genai_b200.parallel.oracle import CommAborted, InProcessCommunicator


def run_ranks(world, fn, timeout=5.0):
    comms = InProcessCommunicator.create_group(world, timeout=timeout)
    out, errs = [None] * world, [None] * world

    def body(r):
        try:
            out[r] = fn(comms[r])
        except Exception as e:      # collected, re-raised by the caller's assertions
            errs[r] = e

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return out, errs


def test_all_to_all_v_and_exchange_counts():
    def fn(c):
        # rank r sends (r + dst) rows to dst, each row tagged (r, dst)
        counts = [c.rank + d for d in range(c.world)]
        rows = torch.tensor([[c.rank, d] for d in range(c.world) for _ in range(counts[d])], dtype=torch.int64).reshape(-1, 2)
        recv = c.exchange_counts(counts)
        got = c.all_to_all_v(rows, counts, recv)
        return recv, got

    out, errs = run_ranks(3, fn)
    assert errs == [None] * 3
    for r, (recv, got) in enumerate(out):
        assert recv == [s + r for s in range(3)]
        want = [[s, r] for s in range(3) for _ in range(s + r)]
        assert got.tolist() == want


def test_send_recv_in_order_and_timeout():
    def fn(c):
        if c.rank == 0:
            c.send(torch.tensor([1.0, 2.0]), 1)
            c.send(torch.tensor([3.0, 4.0]), 1)
            return None
        a, b = torch.zeros(2), torch.zeros(2)
        c.recv(a, 0)
        c.recv(b, 0)
        return a.tolist(), b.tolist()

    out, errs = run_ranks(2, fn)
    assert errs == [None, None] and out[1] == ([1.0, 2.0], [3.0, 4.0])

    def lonely(c):
        if c.rank == 1:
            c.recv(torch.zeros(1), 0)

    _, errs = run_ranks(2, lonely, timeout=0.3)
    assert isinstance(errs[1], CommAborted) and "nothing was sent" in str(errs[1])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_token_sharded_dispatch_and_combine_match_the_dense_computation(world):
    torch.manual_seed(0)
    experts, hid, k, t_per = 8, 16, 2, 11
    w_exp = torch.randn(experts, hid, hid) * 0.2
    hidden = torch.randn(world, t_per, hid)
    ids = torch.stack([torch.stack([torch.randperm(experts)[:k] for _ in range(t_per)]) for _ in range(world)])
    wts = torch.rand(world, t_per, k)
    dense = torch.zeros(world, t_per, hid)
    for r in range(world):
        for i in range(t_per):
            for j in range(k):
                dense[r, i] += wts[r, i, j] * torch.tanh(hidden[r, i] @ w_exp[ids[r, i, j]])

    def fn(c):
        d = EpDispatcher(c, experts)
        base = c.rank * d.per_rank
        return d.run(hidden[c.rank], ids[c.rank], wts[c.rank], lambda rows, e: torch.tanh(rows @ w_exp[base + e]))

    if world == 1:
        got = [EpDispatcher(LocalComm(), experts).run(hidden[0], ids[0], wts[0], lambda rows, e: torch.tanh(rows @ w_exp[e]))]
    else:
        got, errs = run_ranks(world, fn)
        assert errs == [None] * world
    for r in range(world):
        assert torch.allclose(got[r], dense[r], atol=1e-5)
    with pytest.raises(ValueError, match="do not split evenly"):
        EpDispatcher(LocalComm(), 7).__class__(type("C", (), {"world": 2, "rank": 0})(), 7)
