"""Bounded models of the runtime's concurrency protocols (exhaustive search), and an exhaustive small-scope conformance
run of the C++ scheduler core's page accounting."""
import itertools

import numpy as np
import pytest

from onnx_genai_b200.specs import stream_k, tp_exchange
from onnx_genai_b200.utils.model_check import explore


def test_the_checker_reports_a_shortest_trace_for_an_invariant_and_for_a_deadlock():
    step = lambda s: [("inc", s + 1), ("dbl", s * 2)] if s < 20 else []
    r = explore(1, step, {"never 12": lambda s: s != 12}, lambda s: True)
    assert not r.ok and r.kind == "invariant" and r.trace == ("inc", "inc", "dbl", "dbl")        # 1 -> 2 -> 3 -> 6 -> 12
    r = explore(0, lambda s: [("a", s + 1)] if s < 3 else [], {}, lambda s: s == 4)
    assert not r.ok and r.kind == "deadlock" and r.trace == ("a", "a", "a")
    assert explore(0, lambda s: [("a", (s + 1) % 5)], {}, lambda s: False).ok                      # a cycle never deadlocks


@pytest.mark.parametrize("ranks,exchanges", [(2, 4), (3, 2)])
def test_tp_exchange_counters_are_safe_when_cleared_by_their_consumer(ranks, exchanges):
    r = tp_exchange.check(ranks=ranks, exchanges=exchanges)
    assert r.ok and r.states > 100, str(r)


def test_tp_exchange_with_a_late_clear_loses_an_arrival():
    r = tp_exchange.check(ranks=2, exchanges=3, guarded=False)
    assert not r.ok and any("gemm1" in step for step in r.trace), str(r)      # the fast rank's next push races the clear


@pytest.mark.parametrize("kw", [dict(ctas=4, slots=1, tiles=3, k_blocks=4), dict(ctas=8, slots=3, tiles=5, k_blocks=7),
                                dict(ctas=6, slots=2, tiles=2, k_blocks=9)])
def test_stream_k_fixups_that_wait_downwards_never_deadlock(kw):
    assert stream_k.check(**kw).ok


def test_stream_k_fixups_that_wait_upwards_deadlock_under_limited_residency():
    r = stream_k.check(ctas=4, slots=1, tiles=3, k_blocks=4, guarded=False)
    assert not r.ok and r.kind == "deadlock"
    assert stream_k.check(ctas=4, slots=4, tiles=3, k_blocks=4, guarded=False).ok              # enough slots hide the flaw


def test_scheduler_core_conserves_pages_over_every_short_action_sequence():
    """Every sequence of up to five actions (admit a short or a long request, run a step, cancel the oldest live request)
    on a pool too small for two long requests: after each action the free pages plus the pages held by live sequences
    make up the pool, and no page belongs to two sequences."""
    from onnx_genai_b200.engine.core import Core, CoreConfig

    pages = 6
    checked = 0
    for actions in itertools.product("sLxc", repeat=5):
        core = Core(CoreConfig(num_pages=pages, max_seqs=4, max_tokens_per_step=64, max_pages_per_seq=8, prefill_chunk=32,
                               enable_prefix_cache=False, preempt="recompute"))
        plan = np.zeros(core.layout.total_words, dtype=np.int32)
        sampled = np.zeros(core.layout.max_rows, dtype=np.int32)
        live = []
        for a in actions:
            if a in "sL":
                sid = core.add_request(np.arange(20 if a == "s" else 70, dtype=np.int32) % 50, 8, ignore_eos=True)
                live.append(sid)
            elif a == "x":
                if core.build_step(plan.ctypes.data) > 0:
                    for sid, _tok, fin in core.commit_step(sampled.ctypes.data, _rows(core, plan)):
                        if fin is not None and sid in live:
                            live.remove(sid)
                            core.release(sid)
            elif live:
                core.cancel(live[0])
                core.release(live.pop(0))
            held = [set(int(p) for p in core.seq_pages(s)) for s in live]
            union = set().union(*held) if held else set()
            assert sum(len(h) for h in held) == len(union), (actions, held)
            assert all(0 <= p < pages for p in union)
            assert core.num_free_pages + len(union) <= pages and core.num_free_pages >= 0, (actions, core.num_free_pages, union)
            checked += 1
        for sid in live:
            core.release(sid)
        assert core.num_free_pages == pages, (actions, core.num_free_pages)
    assert checked == 5 * 4 ** 5


def _rows(core, plan):
    from onnx_genai_b200.engine.llm_engine import HDR

    return int(plan[HDR["num_logit_rows"]])
