"""Concurrent branches on side streams.

Kernels that need scratch memory (split-K partial tiles, column-sum partials, norm statistics) draw it from a
per-device workspace that is safe only while the kernels using it serialise on one stream.  A ``Branch`` runs
part of a step on a side stream *and* switches the workspaces to a private slot, so two chains of GEMMs (the
actor and the critic update of PPO, a weight-gradient chain beside the data-gradient chain) can overlap.
Forks and joins are event waits, so a branch is captured into a CUDA graph as a parallel sub-graph.
"""
from __future__ import annotations

import threading

import torch

_TLS = threading.local()


def slot() -> int:
    """Workspace slot of the calling thread (0 = the default, main-stream slot)."""
    return getattr(_TLS, "slot", 0)


def ws_key(device) -> tuple:
    idx = device.index if getattr(device, "index", None) is not None else torch.cuda.current_device()
    return (idx, slot())


class Branch:
    """``with Branch(stream, slot): …`` forks from the current stream on entry; ``join()`` makes the current
    stream wait for everything the branch launched.  Tensors produced inside must stay alive until the join."""

    def __init__(self, stream: torch.cuda.Stream, slot_id: int):
        assert slot_id > 0
        self.stream, self.slot_id = stream, slot_id
        self._ctx = None
        self._keep = []
        self._forked = False

    def __enter__(self):
        self.stream.wait_stream(torch.cuda.current_stream())
        self._forked = True
        self._old = slot()
        _TLS.slot = self.slot_id
        self._ctx = torch.cuda.stream(self.stream)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        self._ctx.__exit__(*exc)
        _TLS.slot = self._old
        return False

    def keep(self, *tensors):
        """Hold references to tensors the branch reads that were allocated on another stream, until the join
        (the caching allocator would otherwise be free to hand their memory out again while the branch runs)."""
        self._keep.extend(tensors)

    def join(self):
        """A join without a fork since the last join is a no-op: waiting on a stream that took no part in the current
        capture would make the capture depend on uncaptured work."""
        if self._forked:
            torch.cuda.current_stream().wait_stream(self.stream)
            self._forked = False
        self._keep.clear()
