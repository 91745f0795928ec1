"""Threaded camera reader: a background thread pulls frames from a capture source (device index, ``/dev/video*`` node,
video file, or any object with ``read() -> (ok, frame)``) into a bounded queue; the control loop takes the newest frame
without ever blocking on the camera.  Counters distinguish frames delivered, dropped (queue full), starved takes (no new
frame since the last take) and read failures.
Reference: ``CameraReader`` noeira/vision/camera_thread.mojo:558-1017 (OpenCV VideoCapture behind a BackgroundThread).
"""
from __future__ import annotations

import collections
import threading
import time
from typing import List, Optional

import numpy as np


def camera_spec_is_path(spec: str) -> bool:
    return not spec.strip().lstrip("-").isdigit()


def parse_camera_specs(csv: str) -> List[str]:
    """``"0, /dev/video2,clip.mp4"`` → ``["0", "/dev/video2", "clip.mp4"]``; duplicates are an error (two readers on
    one device starve each other)."""
    out = [s.strip() for s in csv.split(",") if s.strip()]
    if not out:
        raise ValueError("no camera spec given")
    if len(set(out)) != len(out):
        raise ValueError(f"camera specs repeat a device: {out}")
    return out


def open_camera_spec(spec: str, width: int = 0, height: int = 0, fps: float = 0.0):
    import cv2
    cap = cv2.VideoCapture(spec if camera_spec_is_path(spec) else int(spec))
    if not cap.isOpened():
        raise OSError(f"cannot open camera '{spec}'")
    if width and height:
        cap.set(cv2.CAP_PROP_FRAME_WIDTH, width)
        cap.set(cv2.CAP_PROP_FRAME_HEIGHT, height)
    if fps:
        cap.set(cv2.CAP_PROP_FPS, fps)
    return cap


class CameraReader:
    def __init__(self, source, depth: int = 2, label: str = "", period_s: float = 0.0):
        """``source``: a spec string or a capture object.  ``depth``: queue length (older frames are dropped).
        ``period_s``: minimum time between reads (file sources have no frame clock of their own)."""
        self.source, self.depth, self.label, self.period_s = source, depth, label or str(source), period_s
        self._cap = None
        self._q = collections.deque(maxlen=depth)
        self._lock = threading.Lock()
        self._new = threading.Condition(self._lock)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.frames = self.dropped = self.starved = self.read_failures = self.delivered = 0
        self._seq = self._taken_seq = 0
        self.eof = False

    def start(self, wait_ms: int = 4000):
        self._cap = open_camera_spec(self.source) if isinstance(self.source, str) else self.source
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        deadline = time.monotonic() + wait_ms / 1e3
        with self._new:
            while self.frames == 0 and not self.eof:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(f"camera '{self.label}' delivered no frame within {wait_ms} ms")
                self._new.wait(left)
        return self

    def _run(self):
        misses = 0
        while not self._stop.is_set():
            t0 = time.monotonic()
            ok, frame = self._cap.read()
            if not ok or frame is None:
                self.read_failures += 1
                misses += 1
                if misses >= 5:                      # a file that ended, a camera that went away
                    with self._new:
                        self.eof = True
                        self._new.notify_all()
                    return
                time.sleep(0.005)
                continue
            misses = 0
            with self._new:
                if len(self._q) == self._q.maxlen:
                    self.dropped += 1
                self._seq += 1
                self._q.append((self._seq, np.ascontiguousarray(frame)))
                self.frames += 1
                self._new.notify_all()
            if self.period_s:
                time.sleep(max(0.0, self.period_s - (time.monotonic() - t0)))

    def take_latest(self):
        """Newest frame (older queued ones are discarded) or ``None`` when nothing new arrived since the last take."""
        with self._lock:
            if not self._q or self._q[-1][0] == self._taken_seq:
                self.starved += 1
                return None
            seq, frame = self._q[-1]
            self._q.clear()
            self._taken_seq = seq
            self.delivered += 1
            return frame

    def take_blocking(self, timeout_ms: int = 1000):
        deadline = time.monotonic() + timeout_ms / 1e3
        with self._new:
            while (not self._q or self._q[-1][0] == self._taken_seq) and not self.eof:
                left = deadline - time.monotonic()
                if left <= 0:
                    return None
                self._new.wait(left)
        return self.take_latest()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        if self._cap is not None and hasattr(self._cap, "release"):
            self._cap.release()
