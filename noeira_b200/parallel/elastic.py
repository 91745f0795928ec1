"""Failure detection on the host and restart under a new world size.

Nothing here touches a GPU: a peer that stopped is noticed through a key-value store (the ``torch.distributed`` store
of the job, or any object with ``set`` / ``get``), BEFORE the next collective is launched, so no rank ever waits inside
a kernel for a peer that is gone.

  Heartbeat      every rank publishes ``hb/<rank> = <step>:<wall time>`` after each step (``beat``); ``check()`` raises
                 ``PeerLost`` naming the ranks whose last beat is older than ``deadline_s`` or that announced their
                 departure (``leave``).  Used between steps: a rank leaves only with none of its kernels or collectives
                 in flight, the others learn of it here.
  StepWatchdog   a daemon thread per rank that turns a missed step deadline of THIS rank (a hang in host code, a
                 collective that never returns) into an error: the callback gets the overdue time; the default records it
                 and lets ``check()`` raise ``StepTimeout`` from the training thread.
  resume_plan    which global-batch rows a rank takes after the world size changed (``shard_batch`` rule of the
                 reference: contiguous equal shards of the same global batch, so a run resumed on fewer ranks follows
                 the same trajectory, noeira/nn/distributed/shard_batch.mojo:17-44).

The reference detects failed ranks inside its in-process simulator only (``RankFibers._fail``,
noeira/nn/distributed/fibers.mojo:131-143); multi-process detection is new here.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional


class PeerLost(RuntimeError):
    def __init__(self, ranks: List[int], why: str):
        super().__init__(f"ranks {ranks} are gone ({why})")
        self.ranks, self.why = ranks, why


class StepTimeout(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world: int, deadline_s: float = 30.0, clock: Callable[[], float] = time.time,
                 prefix: str = "hb"):
        self.store, self.rank, self.world, self.deadline_s, self.clock, self.prefix = store, rank, world, deadline_s, clock, prefix
        self.step = 0
        self.beat()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: Optional[int] = None):
        self.step = self.step + 1 if step is None else int(step)
        self.store.set(self._key(self.rank), f"{self.step}:{self.clock():.3f}")

    def leave(self):
        """Announce a clean departure (called between steps, nothing in flight)."""
        self.store.set(self._key(self.rank), f"{self.step}:left")

    def peers(self) -> Dict[int, tuple]:
        out = {}
        for r in range(self.world):
            try:
                raw = self.store.get(self._key(r))
            except Exception:  # noqa: BLE001 — a key that was never set
                out[r] = (-1, None)
                continue
            raw = raw.decode() if isinstance(raw, (bytes, bytearray)) else str(raw)
            step, _, t = raw.partition(":")
            out[r] = (int(step), None if t == "left" else float(t))
        return out

    def check(self):
        """Raise ``PeerLost`` when a peer left or has not beaten within the deadline.  Call before launching the next
        step's collectives."""
        now = self.clock()
        left, stale = [], []
        for r, (step, t) in self.peers().items():
            if r == self.rank:
                continue
            if t is None and step >= 0:
                left.append(r)
            elif t is None or now - t > self.deadline_s:
                stale.append(r)
        if left:
            raise PeerLost(left, "left between steps")
        if stale:
            raise PeerLost(stale, f"no heartbeat for more than {self.deadline_s} s")

    def alive(self) -> List[int]:
        now = self.clock()
        return [r for r, (step, t) in self.peers().items() if r == self.rank or (t is not None and now - t <= self.deadline_s)]


class StepWatchdog:
    def __init__(self, deadline_s: float, on_timeout: Optional[Callable[[float], None]] = None, poll_s: float = 0.05):
        self.deadline_s, self.poll_s = deadline_s, poll_s
        self._last = time.monotonic()
        self._armed = False
        self._tripped: Optional[float] = None
        self._on_timeout = on_timeout
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(self.poll_s):
            if self._armed and self._tripped is None:
                late = time.monotonic() - self._last
                if late > self.deadline_s:
                    self._tripped = late
                    if self._on_timeout is not None:
                        self._on_timeout(late)

    def begin_step(self):
        self._last = time.monotonic()
        self._armed = True

    def end_step(self):
        self._armed = False
        self.check()

    def check(self):
        if self._tripped is not None:
            late, self._tripped = self._tripped, None
            raise StepTimeout(f"step exceeded its {self.deadline_s} s deadline ({late:.2f} s)")

    @property
    def tripped(self) -> bool:
        return self._tripped is not None

    def close(self):
        self._stop.set()
        self._thread.join(timeout=1.0)


def resume_plan(global_batch: int, world: int, rank: int):
    """Rows ``[lo, hi)`` of the global batch that ``rank`` of ``world`` takes (contiguous equal shards)."""
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} does not split over {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per
