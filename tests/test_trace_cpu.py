"""Tracing aids run (as no-ops) without a GPU."""


def test_nvtx_range_and_alloc_tracer_are_usable_without_cuda():
    import io
    from noeira_b200.core.run import PerfTimer
    from noeira_b200.utils.trace import AllocTracer, nvtx_range
    with nvtx_range("phase"):
        pass

    @nvtx_range("decorated")
    def f(x):
        return x + 1
    assert f(1) == 2
    t = PerfTimer()
    with t.section("a"):
        pass
    assert t.report()["a"]["calls"] == 1
    out = io.StringIO()
    tr = AllocTracer(enabled=True, stream=out)
    with tr.scope("step"):
        pass
    g = tr.traced("fn")(lambda: 3)
    assert g() == 3 and tr.report()["step"]["allocations"] == 0 and tr.report()["fn"]["calls"] == 1
    tr.assert_steady("step")
