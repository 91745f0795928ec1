"""Camera → robot-base extrinsics from point correspondences: least-squares rigid fit (Kabsch / Umeyama without scale), with
a degeneracy check on the spread of the points, and the variant that also solves for an unknown constant offset of the
touched point in the tool frame.  Reference: noeira/vision/extrinsics.mojo:91-420 (``RigidFit``, ``fit_rigid``,
``fit_rigid_with_offset``)."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class RigidFit:
    R: np.ndarray
    t: np.ndarray
    rms_mm: float
    max_mm: float
    n: int
    spread_mm: float

    def apply(self, p_cam):
        return self.R @ np.asarray(p_cam, float) + self.t


def _spread_mm(p: np.ndarray) -> float:
    """Smallest principal standard deviation (mm): near zero means the points are coplanar / collinear and the rotation
    about that direction is not determined."""
    s = np.linalg.svd(p - p.mean(0), compute_uv=False) / np.sqrt(max(len(p) - 1, 1))
    return float(s[-1] * 1e3)


def fit_rigid(p_cam, p_base, min_spread_mm: float = 5.0) -> RigidFit:
    a, b = np.asarray(p_cam, float), np.asarray(p_base, float)
    if a.shape != b.shape or a.ndim != 2 or a.shape[1] != 3 or len(a) < 4:
        raise ValueError("fit_rigid needs at least 4 matching 3-D points")
    spread = _spread_mm(a)
    if spread < min_spread_mm:
        raise ValueError(f"points are degenerate: smallest spread {spread:.2f} mm < {min_spread_mm} mm")
    ca, cb = a.mean(0), b.mean(0)
    H = (a - ca).T @ (b - cb)
    U, _, Vt = np.linalg.svd(H)
    D = np.diag([1.0, 1.0, np.sign(np.linalg.det(Vt.T @ U.T))])
    R = Vt.T @ D @ U.T
    t = cb - R @ ca
    err = np.linalg.norm((a @ R.T + t) - b, axis=1)
    return RigidFit(R, t, float(np.sqrt((err ** 2).mean()) * 1e3), float(err.max() * 1e3), len(a), spread)


def fit_rigid_with_offset(p_cam, tool_R, tool_t, iters: int = 20, min_spread_mm: float = 5.0):
    """The camera sees a marker rigidly attached to the tool at an UNKNOWN offset ``o`` (tool frame):
    ``p_base_i = tool_R_i o + tool_t_i``.  Alternates a rigid fit with the linear solve for ``o``.
    Returns (RigidFit, offset [3])."""
    a = np.asarray(p_cam, float)
    Rs, ts = np.asarray(tool_R, float).reshape(-1, 3, 3), np.asarray(tool_t, float).reshape(-1, 3)
    o = np.zeros(3)
    fit = None
    for _ in range(iters):
        fit = fit_rigid(a, np.einsum("nij,j->ni", Rs, o) + ts, min_spread_mm)
        # R a_i + t = Rs_i o + ts_i  →  least squares in o
        rhs = (a @ fit.R.T + fit.t - ts).reshape(-1)
        o = np.linalg.lstsq(Rs.reshape(-1, 3), rhs, rcond=None)[0]
    return fit, o
