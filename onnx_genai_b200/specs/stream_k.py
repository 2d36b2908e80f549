"""Model of the stream-K GEMM's fix-up order under limited residency.

The (tile, k-block) iterations are cut into one contiguous range per CTA; a tile whose iterations span several CTAs is
finished by the CTA that holds its last k-block, which waits for the partial accumulators of the others.  The hardware
starts CTAs in index order as residency slots free up and never preempts one, so a resident CTA that waits for a CTA
that has not started can wait forever.  The kernel (csrc/kernels/gemm_tcgen05.cu, GemmWork) therefore makes every wait
point at a *lower-numbered* CTA and walks each range backwards, producing the partial a higher CTA needs first.
``guarded=False`` lets the CTA that holds a tile's *first* k-block finish it instead (waits point upwards); with fewer
slots than CTAs the checker finds the deadlock.
"""
from __future__ import annotations

from ..utils.model_check import Result, explore


def check(ctas: int = 4, slots: int = 2, tiles: int = 3, k_blocks: int = 4, guarded: bool = True) -> Result:
    total = tiles * k_blocks
    bounds = [c * total // ctas for c in range(ctas + 1)]
    # segments of CTA c: (tile, is_finisher, CTAs it waits for), in the order the CTA executes them
    plans = []
    for c in range(ctas):
        segs = []
        for t in range(tiles):
            lo, hi = max(bounds[c], t * k_blocks), min(bounds[c + 1], (t + 1) * k_blocks)
            if lo >= hi:
                continue
            holders = [x for x in range(ctas) if max(bounds[x], t * k_blocks) < min(bounds[x + 1], (t + 1) * k_blocks)]
            finisher = holders[-1] if guarded else holders[0]
            segs.append((t, c == finisher, tuple(x for x in holders if x != c) if c == finisher else ()))
        plans.append(tuple(reversed(segs)) if guarded else tuple(segs))
    # state: (next CTA to start, per-CTA progress: -1 not started, i = segments completed), partial flags as a frozenset of (cta, tile)
    init = (0, (-1,) * ctas, frozenset())

    def step(s):
        nxt, prog, flags = s
        resident = sum(1 for c in range(ctas) if 0 <= prog[c] < len(plans[c]))
        if nxt < ctas and resident < slots:
            yield (f"start cta{nxt}", (nxt + 1, prog[:nxt] + (0,) + prog[nxt + 1:], flags))
        for c in range(ctas):
            i = prog[c]
            if 0 <= i < len(plans[c]):
                t, fin, waits = plans[c][i]
                if fin and not all((x, t) in flags for x in waits):
                    continue                                        # spinning on a partial that is not there yet
                yield (f"cta{c}.tile{t}.{'finish' if fin else 'partial'}",
                       (nxt, prog[:c] + (i + 1,) + prog[c + 1:], flags if fin else flags | {(c, t)}))

    def done(s):
        return all(s[1][c] == len(plans[c]) for c in range(ctas))

    return explore(init, step, {}, done)
