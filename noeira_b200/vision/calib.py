"""Camera calibration: ChArUco intrinsics (pinhole + radial / tangential distortion) and the calibration file a deployment
reads (intrinsics, distortion, image size, optional camera→base transform).
Reference: noeira/vision/calib_file.mojo:75-260 (``CameraCalib``, ``read_calib`` / ``write_calib``), the ChArUco calibration
of noeira/vision/opencv (cv_* shim over OpenCV's aruco module)."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np


@dataclass
class CameraCalib:
    width: int
    height: int
    fx: float
    fy: float
    cx: float
    cy: float
    dist: List[float] = field(default_factory=lambda: [0.0] * 5)      # k1 k2 p1 p2 k3
    rms_px: float = 0.0
    n_views: int = 0
    base_R: Optional[List[float]] = None                               # row-major 3x3, camera → base
    base_t: Optional[List[float]] = None

    def k_matrix(self) -> np.ndarray:
        return np.array([[self.fx, 0, self.cx], [0, self.fy, self.cy], [0, 0, 1.0]])

    def require_size(self, w: int, h: int):
        if (w, h) != (self.width, self.height):
            raise ValueError(f"calibration is for {self.width}x{self.height}, the camera delivers {w}x{h}")

    def base_from_camera(self, p_cam: Sequence[float]) -> np.ndarray:
        if self.base_R is None:
            raise ValueError("this calibration has no camera-to-base transform")
        return np.asarray(self.base_R, float).reshape(3, 3) @ np.asarray(p_cam, float) + np.asarray(self.base_t, float)


def write_calib(path: str, c: CameraCalib):
    tmp = path + ".tmp"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(tmp, "w") as f:
        json.dump({"schema_version": 1, **c.__dict__}, f, indent=1)
    os.replace(tmp, path)


def read_calib(path: str) -> CameraCalib:
    d = json.load(open(path))
    d.pop("schema_version", None)
    return CameraCalib(**d)


def make_charuco_board(squares_x=7, squares_y=5, square_len=0.04, marker_len=0.03, dictionary="DICT_5X5_100"):
    import cv2
    dic = cv2.aruco.getPredefinedDictionary(getattr(cv2.aruco, dictionary))
    return cv2.aruco.CharucoBoard((squares_x, squares_y), square_len, marker_len, dic)


def detect_charuco(gray: np.ndarray, board):
    """→ (corners [n, 2], ids [n]) of the chessboard corners seen in one image (empty arrays when none)."""
    import cv2
    det = cv2.aruco.CharucoDetector(board)
    corners, ids, _, _ = det.detectBoard(gray)
    if ids is None or len(ids) == 0:
        return np.zeros((0, 2), np.float32), np.zeros((0,), np.int32)
    return corners.reshape(-1, 2).astype(np.float32), ids.reshape(-1).astype(np.int32)


def calibrate_charuco(images: Sequence[np.ndarray], board, min_corners: int = 8) -> CameraCalib:
    """Intrinsics from several views of a ChArUco board (views with fewer than ``min_corners`` corners are skipped)."""
    import cv2
    obj_all = board.getChessboardCorners()
    objp, imgp = [], []
    h, w = images[0].shape[:2]
    for im in images:
        gray = im if im.ndim == 2 else cv2.cvtColor(im, cv2.COLOR_BGR2GRAY)
        c, ids = detect_charuco(gray, board)
        if len(ids) >= min_corners:
            objp.append(obj_all[ids].astype(np.float32))
            imgp.append(c)
    if len(objp) < 3:
        raise ValueError(f"only {len(objp)} usable views: a calibration needs at least 3")
    rms, K, dist, _, _ = cv2.calibrateCamera(objp, imgp, (w, h), None, None)
    d = [float(x) for x in dist.reshape(-1)[:5]] + [0.0] * max(0, 5 - dist.size)
    return CameraCalib(w, h, float(K[0, 0]), float(K[1, 1]), float(K[0, 2]), float(K[1, 2]), d, float(rms), len(objp))


def board_pose(gray: np.ndarray, board, calib: CameraCalib):
    """Pose of the board in the camera frame: (R [3,3], t [3]) or None when too few corners are visible."""
    import cv2
    c, ids = detect_charuco(gray, board)
    if len(ids) < 6:
        return None
    ok, rvec, tvec = cv2.solvePnP(board.getChessboardCorners()[ids].astype(np.float32), c, calib.k_matrix(),
                                  np.asarray(calib.dist, float))
    if not ok:
        return None
    return cv2.Rodrigues(rvec)[0], tvec.reshape(3)
