"""Model of the counters that chain a tensor-parallel exchange: scatter GEMM -> exchange kernel -> consumer GEMM.

Every rank owns one row group.  Per exchange ``e`` each rank's scatter GEMM stores its partial product of every group
into the owner's buffer and bumps the owner's arrival counter; the owner's exchange kernel waits until all ranks'
partials are there, clears the counter, reduces, stores the normed rows into every rank's activation buffer and bumps
that rank's ready counter; the rank's next GEMM waits for all owners' rows, reads them and clears its ready counter when
it finishes.  No kernel waits for another at a kernel boundary, so a fast rank may be a whole exchange ahead.  The
kernels (csrc/kernels/tp_comm.cu, gemm_tcgen05.cu) rely on one rule: **a counter is cleared by its consumer before the
consumer releases anything a producer of the next exchange depends on**.  ``guarded=False`` moves the arrival counter's
clear to the end of the exchange kernel instead; the checker then finds the lost arrival as a deadlock.

Checked: partials reduced for exchange e were all produced for exchange e; rows consumed for exchange e were all
written for exchange e; every run completes (no lost arrival).
"""
from __future__ import annotations

from ..utils.model_check import Result, explore


def check(ranks: int = 2, exchanges: int = 3, guarded: bool = True, max_states: int = 2_000_000) -> Result:
    R, E = ranks, exchanges
    full = (1 << R) - 1
    # state: (gemm, xchg, cons, cnt, ready, part, h, bad)
    #   gemm[r] = (exchange being produced, owners already pushed to)        xchg[r] = (exchange, phase, ranks already stored to)
    #   cons[r] = (exchanges consumed, reading?)                             cnt[o], ready[r] counters
    #   part[o][s], h[r][o] = exchange whose data sits in the buffer (-1: none)
    init = (tuple((0, 0) for _ in range(R)), tuple((0, 0, 0) for _ in range(R)), tuple((0, 0) for _ in range(R)),
            (0,) * R, (0,) * R, tuple((-1,) * R for _ in range(R)), tuple((-1,) * R for _ in range(R)), False)

    def put(t, i, v):
        return t[:i] + (v,) + t[i + 1:]

    def step(s):
        gemm, xchg, cons, cnt, ready, part, h, bad = s
        for r in range(R):
            ge, pushed = gemm[r]
            if ge < E and cons[r] == (ge, 0):                       # the GEMM's input is the previous consumer's output
                for o in range(R):
                    if not pushed >> o & 1:
                        np_ = pushed | 1 << o
                        g2 = (ge + 1, 0) if np_ == full else (ge, np_)
                        yield (f"r{r}.gemm{ge}->r{o}",
                               (put(gemm, r, g2), xchg, cons, put(cnt, o, cnt[o] + 1), ready, put(part, o, put(part[o], r, ge)), h, bad))
            xe, phase, stored = xchg[r]
            if xe < E and phase == 0 and cnt[r] == R:               # all ranks' partials of this group have arrived
                stale = any(v != xe for v in part[r])
                yield (f"r{r}.xchg{xe}.reduce",
                       (gemm, put(xchg, r, (xe, 1, 0)), cons, put(cnt, r, 0) if guarded else cnt, ready, part, h, bad or stale))
            if xe < E and phase == 1:
                for p in range(R):
                    if not stored >> p & 1:
                        ns = stored | 1 << p
                        last = ns == full
                        yield (f"r{r}.xchg{xe}->r{p}",
                               (gemm, put(xchg, r, (xe + 1, 0, 0) if last else (xe, 1, ns)), cons,
                                put(cnt, r, 0) if (last and not guarded) else cnt, put(ready, p, ready[p] + 1),
                                part, put(h, p, put(h[p], r, xe)), bad))
            ce, reading = cons[r]
            if ce < E and not reading and ready[r] == R:
                stale = any(v != ce for v in h[r])
                yield (f"r{r}.cons{ce}.read", (gemm, xchg, put(cons, r, (ce, 1)), cnt, ready, part, h, bad or stale))
            if reading:                                              # the last CTA to finish zeroes the ready counter
                yield (f"r{r}.cons{ce}.done", (gemm, xchg, put(cons, r, (ce + 1, 0)), cnt, put(ready, r, 0), part, h, bad))

    def done(s):
        return all(g[0] == E for g in s[0]) and all(x[0] == E for x in s[1]) and all(c == (E, 0) for c in s[2])

    return explore(init, step, {"every buffer read holds the data of the exchange being processed": lambda s: not s[7],
                                "counters never exceed the group size": lambda s: max(s[3]) <= R and max(s[4]) <= R}, done, max_states)
