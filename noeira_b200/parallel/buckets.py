"""Gradient marks and bucket planning for overlapping the gradient reduction with the backward pass.

Parameters live in one arena; the backward pass finishes their gradients in reverse registration order.  ``GradMarks``
records, per marked unit (a block of the model), the arena byte range of its parameters; ``plan_buckets`` groups
consecutive units (walking from the END of the arena, the order gradients become ready) into buckets of at least
``bucket_bytes``; ``BucketedReducer`` launches one reduction per bucket on a side stream as soon as the backward has
passed the bucket's first unit, and the optimizer waits for all of them.
Reference: ``GradReady`` wrapper + ``GradMarks`` registry (noeira/nn/distributed/grad_marks.mojo:75-132,245-379),
``plan_buckets`` (nn/distributed/buckets.mojo), DDP overlap of nn/distributed/data_parallel.mojo.
On NVSwitch the bucket size is chosen against launch latency, not link count: the default is 8 MB.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Sequence, Tuple


@dataclass
class Mark:
    name: str
    begin: int      # element offsets into the arena
    end: int


class GradMarks:
    def __init__(self):
        self.marks: List[Mark] = []

    def add(self, name: str, begin: int, end: int):
        if self.marks and begin < self.marks[-1].end:
            raise ValueError("marks must be registered in arena order without overlap")
        self.marks.append(Mark(name, begin, end))

    @classmethod
    def from_arena(cls, arena, unit_of: Callable[[str], str]):
        """One mark per unit; ``unit_of(param name)`` maps a parameter to its unit (e.g. its transformer block)."""
        gm = cls()
        cur, b, e = None, 0, 0
        for name, off, n in arena.layout():
            u = unit_of(name)
            if u != cur:
                if cur is not None:
                    gm.add(cur, b, e)
                cur, b = u, off
            e = off + n
        if cur is not None:
            gm.add(cur, b, e)
        return gm


@dataclass
class Bucket:
    begin: int
    end: int
    units: Tuple[str, ...]
    ready_after: str        # the unit whose backward completes the bucket (the FIRST unit in arena order)


def plan_buckets(marks: Sequence[Mark], bucket_elems: int) -> List[Bucket]:
    """Buckets in the order they become ready (last units of the arena first)."""
    out: List[Bucket] = []
    units: List[Mark] = []
    for m in reversed(marks):
        units.append(m)
        if units[0].end - m.begin >= bucket_elems:
            out.append(Bucket(m.begin, units[0].end, tuple(u.name for u in reversed(units)), m.name))
            units = []
    if units:
        out.append(Bucket(units[-1].begin, units[0].end, tuple(u.name for u in reversed(units)), units[-1].name))
    return out


class BucketedReducer:
    """``on_unit_done(name)`` is called by the model's backward after a unit finished; a bucket is reduced by
    ``reduce_fn(begin, end)`` (which enqueues on its own stream) once EVERY unit of it has reported, and only after all
    buckets before it went — the launch order is the planned order on every rank, whatever order the model's backward
    visits the units of one bucket in (a language model finishes its token table before its position table although the
    arena holds them the other way round).  A unit must report once per backward: a module that is applied twice in
    one forward has to be marked as one unit around both applications.  ``finish()`` reduces what is left and resets for
    the next step."""

    def __init__(self, buckets: Sequence[Bucket], reduce_fn: Callable[[int, int], None]):
        self.buckets, self.reduce_fn = list(buckets), reduce_fn
        self._next = 0
        self._done = set()
        self.order: List[Tuple[int, int]] = []

    def _launch(self):
        b = self.buckets[self._next]
        self.reduce_fn(b.begin, b.end)
        self.order.append((b.begin, b.end))
        self._next += 1

    def on_unit_done(self, name: str):
        self._done.add(name)
        while self._next < len(self.buckets) and self._done.issuperset(self.buckets[self._next].units):
            self._launch()

    def finish(self):
        while self._next < len(self.buckets):
            self._launch()
        self._next = 0
        self._done.clear()
