"""Tracing aids: NVTX ranges and an allocation tracer.

  nvtx_range(name)   context manager / decorator: an NVTX range around a phase (visible in Nsight timelines); a no-op
                     where NVTX is unavailable or ``NOEIRA_NVTX=0``.  ``PerfTimer.section`` opens one as well.
  AllocTracer        counts device allocations (and bytes) made by the caching allocator inside named scopes, to find
                     allocations in what should be a steady-state step: a captured / warmed-up training iteration must
                     allocate nothing.  Enabled explicitly or with ``NOEIRA_ALLOC_TRACE=1``; with tracing on every scope
                     that allocated is printed with its count, bytes and the Python call site that opened it.
                     (The reference traces ``Tensor.alloc_gpu`` calls the same way under ``NOEIRA_ALLOC_TRACE=1``,
                     noeira/nn/core/tensor.mojo:27-57.)
"""
from __future__ import annotations

import contextlib
import functools
import os
import sys
import traceback
from typing import Dict, List


def _nvtx():
    if os.environ.get("NOEIRA_NVTX", "1") == "0":
        return None
    try:
        import torch
        if torch.cuda.is_available():
            return torch.cuda.nvtx
    except Exception:  # noqa: BLE001
        pass
    return None


class nvtx_range(contextlib.ContextDecorator):
    def __init__(self, name: str):
        self.name = name
        self._nv = None

    def __enter__(self):
        self._nv = _nvtx()
        if self._nv is not None:
            self._nv.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self._nv is not None:
            self._nv.range_pop()
        return False


def _alloc_counters(device=None):
    try:
        import torch
        if not torch.cuda.is_available():
            return 0, 0
        st = torch.cuda.memory_stats(device)
        return int(st.get("allocation.all.allocated", 0)), int(st.get("allocated_bytes.all.allocated", 0))
    except Exception:  # noqa: BLE001
        return 0, 0


class AllocTracer:
    def __init__(self, enabled: bool = None, stream=None):
        self.enabled = (os.environ.get("NOEIRA_ALLOC_TRACE", "0") == "1") if enabled is None else enabled
        self.scopes: Dict[str, Dict[str, int]] = {}
        self.order: List[str] = []
        self.stream = stream or sys.stderr

    @contextlib.contextmanager
    def scope(self, name: str):
        if not self.enabled:
            yield self
            return
        site = traceback.extract_stack(limit=3)[0]
        n0, b0 = _alloc_counters()
        try:
            yield self
        finally:
            n1, b1 = _alloc_counters()
            s = self.scopes.setdefault(name, dict(calls=0, allocations=0, bytes=0))
            if name not in self.order:
                self.order.append(name)
            s["calls"] += 1
            s["allocations"] += n1 - n0
            s["bytes"] += b1 - b0
            if n1 > n0:
                print(f"[alloc-trace] {name}: {n1 - n0} allocation(s), {b1 - b0} bytes  ({site.filename}:{site.lineno})",
                      file=self.stream)

    def traced(self, name: str = None):
        def deco(fn):
            label = name or fn.__qualname__

            @functools.wraps(fn)
            def wrapper(*a, **k):
                with self.scope(label):
                    return fn(*a, **k)
            return wrapper
        return deco

    def report(self) -> Dict[str, Dict[str, int]]:
        return {k: dict(self.scopes[k]) for k in self.order}

    def assert_steady(self, name: str):
        """Raise when the LAST recorded call of scope ``name`` is part of a scope that allocated at all."""
        s = self.scopes.get(name)
        if s and s["allocations"]:
            raise AssertionError(f"scope '{name}' made {s['allocations']} device allocation(s) ({s['bytes']} bytes) in {s['calls']} call(s)")
