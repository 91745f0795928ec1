"""Action-chunk queries off the control thread.

A robot control loop runs at tens of hertz; one VLA query (vision prefix + ten denoising steps) takes longer than a control
period.  ``VLAQueryWorker`` owns a background thread (and, on CUDA, its own stream): the control thread posts the newest
observation with ``submit`` — a pending, not yet started observation is replaced, never queued — and reads the most recent
finished action chunk with ``latest`` without blocking; ``wait`` blocks until a chunk newer than a given sequence number
exists.  ``ChunkCursor`` turns chunks into per-tick actions: it walks the current chunk and jumps to a newer one as soon
as it arrives, skipping the steps that elapsed while the query ran.
(noeira/deep_agents/smolvla/query_worker.mojo: one observation in, one action chunk out, off the control thread.)
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Optional, Tuple

import torch


class VLAQueryWorker:
    def __init__(self, query: Callable, device=None):
        """``query(*observation) → action chunk [chunk, action_dim]`` (e.g. ``lambda img, ids, st: model.sample_actions(img, ids,
        st)[0]``)."""
        self.query = query
        self.device = torch.device(device) if device is not None else None
        self._lock = threading.Condition()
        self._pending: Optional[Tuple[int, tuple]] = None
        self._result: Optional[Tuple[int, torch.Tensor, float]] = None
        self._submitted = self._finished = 0
        self._stop = False
        self.error: Optional[BaseException] = None
        self.dropped = 0
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def submit(self, *observation) -> int:
        """Posts an observation; returns its sequence number.  An observation that was waiting is dropped."""
        with self._lock:
            if self._pending is not None:
                self.dropped += 1
            self._submitted += 1
            self._pending = (self._submitted, observation)
            self._lock.notify_all()
            return self._submitted

    def latest(self):
        """(sequence number of the observation it answers, action chunk, query seconds) of the newest finished query, or None."""
        with self._lock:
            return self._result

    def wait(self, newer_than: int = 0, timeout: float = 10.0):
        deadline = time.monotonic() + timeout
        with self._lock:
            while (self._result is None or self._result[0] <= newer_than) and self.error is None:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError("no action chunk arrived in time")
                self._lock.wait(left)
            if self.error is not None:
                raise RuntimeError("the query thread failed") from self.error
            return self._result

    def close(self):
        with self._lock:
            self._stop = True
            self._lock.notify_all()
        self._thread.join(timeout=5.0)

    def _run(self):
        stream = torch.cuda.Stream(device=self.device) if self.device is not None and self.device.type == "cuda" else None
        while True:
            with self._lock:
                while self._pending is None and not self._stop:
                    self._lock.wait()
                if self._stop:
                    return
                seq, obs = self._pending
                self._pending = None
            t0 = time.monotonic()
            try:
                if stream is not None:
                    with torch.cuda.stream(stream):
                        out = self.query(*obs)
                    stream.synchronize()
                else:
                    out = self.query(*obs)
            except BaseException as e:            # the control thread learns of it at its next wait
                with self._lock:
                    self.error = e
                    self._lock.notify_all()
                return
            with self._lock:
                self._result = (seq, out, time.monotonic() - t0)
                self._finished = seq
                self._lock.notify_all()


class ChunkCursor:
    """Per-tick actions from asynchronously arriving chunks.  ``tick`` is the control step counter at which the observation
    of a chunk was taken; step k of that chunk belongs to control step ``tick + k``."""

    def __init__(self):
        self.chunk, self.tick0 = None, 0

    def offer(self, chunk: torch.Tensor, observed_at_tick: int):
        if self.chunk is None or observed_at_tick >= self.tick0:
            self.chunk, self.tick0 = chunk, observed_at_tick

    def action(self, tick: int) -> Optional[torch.Tensor]:
        if self.chunk is None:
            return None
        k = tick - self.tick0
        return self.chunk[min(max(k, 0), self.chunk.shape[0] - 1)]

    def remaining(self, tick: int) -> int:
        return 0 if self.chunk is None else max(self.chunk.shape[0] - 1 - (tick - self.tick0), 0)
