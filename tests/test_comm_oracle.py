"""CPU-rank communicator: bit-exact reductions, ordering checks, abort / timeout, buffer leases."""
import threading

import pytest
import torch

from onnx_genai_b200.parallel.oracle import (CollectiveMismatch, CommAborted, InProcessCommunicator, LeaseConflict,
                                             OwnershipRegistry, membership_hash)
from onnx_genai_b200.parallel.sharding import shard_heads, shard_range


def run_ranks(world, fn, timeout=5.0):
    comms = InProcessCommunicator.create_group(world, timeout)
    out, errs = [None] * world, [None] * world

    def target(r):
        try:
            out[r] = fn(comms[r], r)
        except Exception as exc:  # noqa: BLE001
            errs[r] = exc

    ts = [threading.Thread(target=target, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(20) for t in ts]
    return out, errs


def test_all_reduce_matches_single_device_bitwise():
    torch.manual_seed(0)
    parts = [torch.randn(1000).bfloat16() for _ in range(4)]
    want = parts[0].clone()
    for p in parts[1:]:
        want = (want.float() + p.float()).bfloat16()
    out, errs = run_ranks(4, lambda c, r: c.all_reduce(parts[r].clone()))
    assert all(e is None for e in errs)
    assert all(torch.equal(o, want) for o in out)


def test_gather_scatter_alltoall_broadcast():
    def fn(c, r):
        g = torch.empty(4 * 3)
        c.all_gather(g, torch.full((3,), float(r)))
        rs = torch.empty(2)
        c.reduce_scatter(rs, torch.arange(8.0) + r)
        a = torch.empty(4)
        c.all_to_all(a, torch.arange(4.0) + 10 * r)
        b = torch.full((2,), float(r))
        c.broadcast(b, src=2)
        counts = c.exchange_counts([r + d for d in range(4)])
        return g, rs, a, b, counts

    out, errs = run_ranks(4, fn)
    assert all(e is None for e in errs), errs
    for r, (g, rs, a, b, counts) in enumerate(out):
        assert g.tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3]
        assert rs.tolist() == [4 * (2 * r) + 6, 4 * (2 * r + 1) + 6]
        assert a.tolist() == [r + 10 * s for s in range(4)]
        assert b.tolist() == [2.0, 2.0]
        assert counts == [s + r for s in range(4)]


def test_mismatched_collective_order_is_rejected():
    def fn(c, r):
        t = torch.ones(4)
        return c.all_reduce(t) if r != 1 else c.broadcast(t, 0)

    _, errs = run_ranks(2, fn)
    assert any(isinstance(e, CollectiveMismatch) for e in errs)
    assert all(isinstance(e, (CollectiveMismatch, CommAborted)) for e in errs)


def test_rank_that_never_joins_times_out_and_abort_wakes_waiters():
    def fn(c, r):
        if r == 2:
            return "absent"      # this rank leaves between steps and never enters the collective
        return c.all_reduce(torch.ones(2))

    out, errs = run_ranks(3, fn, timeout=0.3)
    assert out[2] == "absent"
    assert all(isinstance(errs[r], CommAborted) and "never joined" in str(errs[r]) for r in (0, 1))

    comms = InProcessCommunicator.create_group(2, timeout=5.0)
    res = {}

    def waiter():
        try:
            comms[0].barrier()
        except CommAborted as exc:
            res["err"] = str(exc)

    t = threading.Thread(target=waiter)
    t.start()
    import time
    time.sleep(0.1)
    comms[1].abort("rank 1 lost its device")
    comms[1].abort("second call is ignored")
    t.join(5)
    assert "rank 1 lost its device" in res["err"]
    with pytest.raises(CommAborted):
        comms[1].barrier()
    for c in comms:
        c.restart()
    out = []
    ts = [threading.Thread(target=lambda c=c: out.append(c.all_reduce(torch.ones(1)).item())) for c in comms]
    [x.start() for x in ts]
    [x.join(5) for x in ts]
    assert out == [2.0, 2.0]


def test_ownership_registry_and_hash():
    reg = OwnershipRegistry()
    reg.acquire(0x1000, "read", "a")
    reg.acquire(0x1000, "read", "b")
    with pytest.raises(LeaseConflict, match="cannot lease it for write"):
        reg.acquire(0x1000, "write", "c")
    reg.release(0x1000, "a")
    reg.release(0x1000, "b")
    reg.acquire(0x1000, "write", "c")
    assert membership_hash([0, 1, 2]) != membership_hash([0, 2, 1])


def test_head_sharding_rules():
    # Qwen2.5-7B at TP=8: 28 query heads over 4 KV heads -> uneven 4 + 3 split, KV head replicated on 2 ranks
    got = [shard_heads(28, 4, 8, r) for r in range(8)]
    assert [len(s.q_heads) for s in got] == [4, 3, 4, 3, 4, 3, 4, 3]
    assert sorted(h for s in got for h in s.q_heads) == list(range(28))
    assert [s.kv_heads for s in got] == [[0], [0], [1], [1], [2], [2], [3], [3]]
    assert all(q // 7 == s.kv_heads[0] for s in got for q in s.q_heads)
    assert shard_heads(32, 8, 4, 1).kv_heads == [2, 3]
    spans = [shard_range(18944, 8, r, 32) for r in range(8)]
    assert spans[0][0] == 0 and spans[-1][1] == 18944 and all(b == spans[i + 1][0] for i, (a, b) in enumerate(spans[:-1]))


def _replay_check(log, world, programs):
    """Independent checker: re-derive what the slot log must be from the ranks' programs alone.  Every rank issues the
    same ops in the same order, so the log has one entry per program step, sequence numbers 1..n in order, and the
    op recorded at each slot is the op every rank's program holds there."""
    assert len({tuple(op for op, _ in p) for p in programs}) == 1, "ranks disagree on the program"
    ops = [op for op, _ in programs[0]]
    assert [inst.sequence for inst, _ in log] == list(range(1, len(ops) + 1))
    assert [op for _, op in log] == ops
    assert len({inst.execution for inst, _ in log}) == 1


@pytest.mark.parametrize("seed", range(6))
def test_seeded_schedule_campaign_is_bitwise_stable_and_replays(seed):
    """Random programs of collectives run under random per-rank delays: results never depend on thread timing, equal a
    single-thread evaluation in fixed rank order bit for bit, and the canonical slot log replays."""
    import random
    import time

    rng = random.Random(seed)
    world = rng.choice([2, 3, 4])
    steps = []
    for _ in range(12):
        op = rng.choice(["all_reduce", "all_gather", "reduce_scatter", "broadcast", "all_to_all"])
        n = world * rng.choice([1, 3, 8])
        dtype = rng.choice([torch.float32, torch.bfloat16, torch.float16])
        steps.append((op, (n, dtype, rng.randrange(world))))
    gen = torch.Generator().manual_seed(seed)
    data = [[(torch.randn(n, generator=gen) * 3).to(dt) for _op, (n, dt, _s) in steps] for _ in range(world)]
    delays = [[rng.random() * 0.004 for _ in steps] for _ in range(world)]

    def expect(i, r):
        op, (n, dt, src) = steps[i]
        bufs = {q: data[q][i] for q in range(world)}
        if op == "all_reduce":
            return InProcessCommunicator._reduce(bufs)
        if op == "reduce_scatter":
            return InProcessCommunicator._reduce(bufs).reshape(world, -1)[r]
        if op == "all_gather":
            return torch.cat([bufs[q] for q in range(world)])
        if op == "broadcast":
            return bufs[src]
        return torch.cat([bufs[q].reshape(world, -1)[r] for q in range(world)])

    def run_once(delay_table):
        comms = InProcessCommunicator.create_group(world, timeout=10.0)
        results, errs = [[None] * len(steps) for _ in range(world)], [None] * world

        def body(r):
            try:
                c = comms[r]
                for i, (op, (n, dt, src)) in enumerate(steps):
                    time.sleep(delay_table[r][i])
                    t = data[r][i].clone()
                    if op == "all_reduce":
                        results[r][i] = c.all_reduce(t).clone()
                    elif op == "reduce_scatter":
                        results[r][i] = c.reduce_scatter(torch.empty(n // world, dtype=dt), t).clone()
                    elif op == "all_gather":
                        results[r][i] = c.all_gather(torch.empty(n * world, dtype=dt), t).clone()
                    elif op == "broadcast":
                        results[r][i] = c.broadcast(t, src).clone()
                    else:
                        results[r][i] = c.all_to_all(torch.empty(n, dtype=dt), t).clone()
            except Exception as e:
                errs[r] = e

        threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
        [t.start() for t in threads]
        [t.join() for t in threads]
        assert errs == [None] * world, errs
        return results, comms[0].g.log

    first, log = run_once(delays)
    second, _ = run_once([list(reversed(d)) for d in reversed(delays)])          # a different interleaving
    for r in range(world):
        for i in range(len(steps)):
            assert torch.equal(first[r][i], second[r][i]), (r, i, steps[i][0])
            assert torch.equal(first[r][i], expect(i, r)), (r, i, steps[i][0])
    _replay_check(log, world, [steps] * world)
