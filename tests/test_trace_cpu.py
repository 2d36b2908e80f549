"""Trace spans: the optional NVTX hand-off to external profilers."""
def test_spans_mirror_into_nvtx_ranges_when_asked():
    """With the NVTX hand-off on, every span pushes and pops one range named category:name, nested in order; a push
    that raises turns the hand-off off instead of breaking the span."""
    from onnx_genai_b200.utils.trace import Tracer

    t = Tracer()
    log = []
    assert t.enable_nvtx(push=lambda name: log.append(("push", name)), pop=lambda: log.append(("pop",)))
    with t.span("loop.step"):
        with t.span("gemm", cat="op"):
            pass
    assert log == [("push", "engine:loop.step"), ("push", "op:gemm"), ("pop",), ("pop",)]

    def bad(name):
        raise RuntimeError("no NVTX here")

    t.enable_nvtx(push=bad, pop=lambda: log.append(("pop",)))
    with t.span("x"):
        pass
    assert t.nvtx is None and log[-1] == ("pop",) and len(log) == 4
