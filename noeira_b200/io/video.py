"""Video files: sequential decode and encode through OpenCV's FFmpeg backend.

``VideoDecoder`` hands out frames in order (RGB uint8 ``[H, W, 3]``) and can seek to a frame index; ``VideoEncoder`` writes
an mp4.  Decoding is sequential by design: datasets pack many episodes into one file and are read in file order, so one
decoder per camera advances in lock step with the episode loop and peak memory is one frame per camera.
Reference: noeira/io/video/ (a pipe from the ffmpeg binary; here the FFmpeg that OpenCV links).
"""
from __future__ import annotations

import numpy as np


def _cv2():
    try:
        import cv2
    except ImportError as e:  # pragma: no cover
        raise RuntimeError("video IO needs OpenCV (cv2) with FFmpeg") from e
    return cv2


class VideoDecoder:
    def __init__(self, path: str):
        cv2 = _cv2()
        self.cap = cv2.VideoCapture(path)
        if not self.cap.isOpened():
            raise IOError(f"cannot open video {path!r}")
        self.path = path
        self.fps = float(self.cap.get(cv2.CAP_PROP_FPS))
        self.width = int(self.cap.get(cv2.CAP_PROP_FRAME_WIDTH))
        self.height = int(self.cap.get(cv2.CAP_PROP_FRAME_HEIGHT))
        self.n_frames = int(self.cap.get(cv2.CAP_PROP_FRAME_COUNT))
        self.pos = 0

    def read(self) -> np.ndarray:
        """Next frame as RGB uint8 [H, W, 3]; raises EOFError at the end."""
        ok, bgr = self.cap.read()
        if not ok:
            raise EOFError(f"{self.path}: no frame {self.pos}")
        self.pos += 1
        return bgr[:, :, ::-1]

    def skip_to(self, frame: int) -> None:
        """Advances to ``frame`` by decoding (frame-accurate, unlike a container seek); never goes backwards."""
        if frame < self.pos:
            raise ValueError(f"{self.path}: cannot go back from frame {self.pos} to {frame} (sequential decoder)")
        while self.pos < frame:
            if not self.cap.grab():
                raise EOFError(f"{self.path}: no frame {self.pos}")
            self.pos += 1

    def close(self):
        self.cap.release()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class VideoEncoder:
    def __init__(self, path: str, width: int, height: int, fps: float = 30.0, fourcc: str = "mp4v"):
        cv2 = _cv2()
        self.w = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*fourcc), fps, (width, height))
        if not self.w.isOpened():
            raise IOError(f"cannot open video writer for {path!r}")
        self.size = (height, width)
        self.n = 0

    def write(self, rgb: np.ndarray) -> None:
        if rgb.shape[:2] != self.size or rgb.dtype != np.uint8:
            raise ValueError(f"frame must be uint8 {self.size + (3,)}, got {rgb.dtype} {rgb.shape}")
        self.w.write(np.ascontiguousarray(rgb[:, :, ::-1]))
        self.n += 1

    def close(self):
        self.w.release()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
