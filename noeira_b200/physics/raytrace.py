"""Ray-traced cameras over batched worlds (CUDA kernel ``csrc/raytrace.cu``) and the NumPy oracle of the same math.

``BatchedCameraRenderer(model, cameras, height, width)`` builds the static geom table from a ``RigidModel`` (every
capsule / sphere geom of every body plus the ground plane); ``render(xpos, xmat)`` takes the body poses of all
worlds (``PhysicsEngine.body_poses()``) and returns ``uint8 [worlds, cams, H, W, 3]`` and ``float32`` depth on
the device — no graphics API involved (noeira/physics3d/raytrace/batch.mojo BatchedCameraRenderer; CPU path
host_render.mojo).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from .._native import check, cuda_lib, ptr, stream_ptr

GEOM_FLOATS = 24
TYPES = {"plane": 0, "sphere": 1, "capsule": 2, "box": 3}


def _quat_to_mat(q):
    w, x, y, z = [float(v) for v in q]
    n = (w * w + x * x + y * y + z * z) ** 0.5
    w, x, y, z = w / n, x / n, y / n, z / n
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                     [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                     [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]])


@dataclass
class Camera:
    pos: Sequence[float]
    look_at: Sequence[float] = (0.0, 0.0, 0.5)
    fovy_deg: float = 45.0
    track_body: int = -1          # >= 0: ``pos`` is an offset from that body's position (orientation stays fixed)

    def record(self):
        p, t = np.asarray(self.pos, float), np.asarray(self.look_at, float)
        back = p - t if self.track_body < 0 else p.copy()
        back = back / np.linalg.norm(back)
        right = np.cross([0.0, 0.0, 1.0], back)
        right = right / max(np.linalg.norm(right), 1e-9)
        up = np.cross(back, right)
        rot = np.stack([right, up, back], 1)       # columns
        return np.concatenate([p, rot.reshape(-1), [np.deg2rad(self.fovy_deg), float(self.track_body), 0.0, 0.0]]).astype(np.float32)


def geom_table(model, ground_rgba=(0.45, 0.55, 0.45, 1.0)) -> np.ndarray:
    rows = []

    def row(typ, body, pos, rot, size, rgba):
        r = np.zeros(GEOM_FLOATS, np.float32)
        r[0], r[1] = TYPES[typ], body
        r[2:5], r[5:14] = pos, np.asarray(rot).reshape(-1)
        r[14:14 + len(size)] = size
        r[17:21] = rgba
        return r

    rows.append(row("plane", -1, (0, 0, float(model.opt.plane_offset)), np.eye(3), (0, 0, 0), ground_rgba))
    for bi, b in enumerate(model.bodies):
        for g in b.geoms:
            rows.append(row(g.type, bi, g.pos, _quat_to_mat(g.quat), tuple(g.size), g.rgba))
    return np.stack(rows)


class BatchedCameraRenderer:
    def __init__(self, model, cameras: List[Camera], height: int = 64, width: int = 64, device="cuda",
                 light_dir=(0.3, -0.4, 0.85), ambient=0.35, diffuse=0.75, shadows=True):
        self.model, self.H, self.W = model, height, width
        self.device = torch.device(device)
        self.geoms_np = geom_table(model)
        self.cams_np = np.stack([c.record() for c in cameras])
        ld = np.asarray(light_dir, np.float64)
        ld = ld / np.linalg.norm(ld)
        self.light_np = np.array([*ld, ambient, diffuse, 1.0 if shadows else 0.0, 0, 0], np.float32)
        if self.device.type == "cuda":
            self.geoms = torch.from_numpy(self.geoms_np).to(self.device)
            self.cams = torch.from_numpy(self.cams_np).to(self.device)
            self.light = torch.from_numpy(self.light_np).to(self.device)
        self._rgb = self._depth = None

    def render(self, xpos: torch.Tensor, xmat: torch.Tensor):
        n, nb = xpos.shape[0], xpos.shape[1]
        nc = len(self.cams_np)
        if not xpos.is_cuda:
            return render_reference(self.geoms_np, xpos.numpy(), xmat.numpy(), self.cams_np, self.H, self.W, self.light_np)
        if self._rgb is None or self._rgb.shape[0] != n:
            self._rgb = torch.empty(n, nc, self.H, self.W, 3, dtype=torch.uint8, device=self.device)
            self._depth = torch.empty(n, nc, self.H, self.W, dtype=torch.float32, device=self.device)
        check(cuda_lib().nb_raytrace(ptr(self.geoms), ctypes.c_int(len(self.geoms_np)), ptr(xpos.contiguous()),
                                     ptr(xmat.contiguous()), ctypes.c_int(nb), ptr(self.cams), ctypes.c_int(nc),
                                     ctypes.c_int(self.H), ctypes.c_int(self.W), ptr(self.light), ptr(self._rgb),
                                     ptr(self._depth), ctypes.c_int(n), stream_ptr()), "raytrace")
        return self._rgb, self._depth


# ------------------------------------------------------------------------------------------ NumPy oracle
def _hit_local(typ, size, o, d, tmin):
    """Vectorised over rays: o, d [R, 3] → (t [R] (inf = miss), n [R, 3])."""
    R = o.shape[0]
    t = np.full(R, np.inf, np.float32)
    n = np.zeros((R, 3), np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        if typ == 0:
            tt = -o[:, 2] / d[:, 2]
            ok = (np.abs(d[:, 2]) >= 1e-9) & (tt > tmin)
            t[ok] = tt[ok]
            n[ok] = (0, 0, 1)
        elif typ == 1:
            b = (o * d).sum(1)
            c = (o * o).sum(1) - size[0] ** 2
            disc = b * b - c
            s = np.sqrt(np.maximum(disc, 0))
            tt = np.where(-b - s > tmin, -b - s, -b + s)
            ok = (disc >= 0) & (tt > tmin)
            t[ok] = tt[ok]
            n[ok] = (o[ok] + tt[ok, None] * d[ok]) / size[0]
        elif typ == 2:
            r, h = size[0], size[1]
            a = d[:, 0] ** 2 + d[:, 1] ** 2
            b = o[:, 0] * d[:, 0] + o[:, 1] * d[:, 1]
            c = o[:, 0] ** 2 + o[:, 1] ** 2 - r * r
            disc = b * b - a * c
            s = np.sqrt(np.maximum(disc, 0))
            for sgn in (-1, 1):
                tt = (-b + sgn * s) / a
                z = o[:, 2] + tt * d[:, 2]
                ok = (a > 1e-12) & (disc >= 0) & (tt > tmin) & (np.abs(z) <= h) & (tt < t)
                t[ok] = tt[ok]
                n[ok, 0] = (o[ok, 0] + tt[ok] * d[ok, 0]) / r
                n[ok, 1] = (o[ok, 1] + tt[ok] * d[ok, 1]) / r
                n[ok, 2] = 0
            for cap in (-1, 1):
                oc = o.copy()
                oc[:, 2] -= cap * h
                bb = (oc * d).sum(1)
                cc = (oc * oc).sum(1) - r * r
                disc = bb * bb - cc
                s = np.sqrt(np.maximum(disc, 0))
                for sgn in (-1, 1):
                    tt = -bb + sgn * s
                    z = oc[:, 2] + tt * d[:, 2]
                    ok = (disc >= 0) & (tt > tmin) & (z * cap >= 0) & (tt < t)
                    t[ok] = tt[ok]
                    n[ok] = (oc[ok] + tt[ok, None] * d[ok]) / r
        else:
            t0 = np.full(R, -1e30, np.float32)
            t1 = np.full(R, 1e30, np.float32)
            n0 = np.zeros((R, 3), np.float32)
            n1 = np.zeros((R, 3), np.float32)
            miss = np.zeros(R, bool)
            for k in range(3):
                par = np.abs(d[:, k]) < 1e-12
                miss |= par & (np.abs(o[:, k]) > size[k])
                ta, tb = (-size[k] - o[:, k]) / d[:, k], (size[k] - o[:, k]) / d[:, k]
                swap = ta > tb
                lo, hi = np.where(swap, tb, ta), np.where(swap, ta, tb)
                slo, shi = np.where(swap, 1.0, -1.0), np.where(swap, -1.0, 1.0)
                u0 = (~par) & (lo > t0)
                t0[u0] = lo[u0]
                n0[u0] = 0
                n0[u0, k] = slo[u0]
                u1 = (~par) & (hi < t1)
                t1[u1] = hi[u1]
                n1[u1] = 0
                n1[u1, k] = shi[u1]
            ok = ~miss & (t0 <= t1)
            first = ok & (t0 > tmin)
            second = ok & ~first & (t1 > tmin)
            t[first], n[first] = t0[first], n0[first]
            t[second], n[second] = t1[second], n1[second]
    return t, n


def _trace(geoms, xpos, xmat, o, d, tmin):
    R = o.shape[0]
    best_t = np.full(R, np.inf, np.float32)
    best_n = np.tile(np.array([0, 0, 1], np.float32), (R, 1))
    best_g = np.full(R, -1, np.int64)
    for gi, G in enumerate(geoms):
        body = int(G[1])
        rot, pos = G[5:14].reshape(3, 3).astype(np.float32), G[2:5].astype(np.float32)
        if body >= 0:
            bm = xmat[body].reshape(3, 3).astype(np.float32)
            Rw, p = bm @ rot, xpos[body].astype(np.float32) + bm @ pos
        else:
            Rw, p = rot, pos
        ol, dl = (o - p) @ Rw, d @ Rw
        t, nl = _hit_local(int(G[0]), G[14:17], ol.astype(np.float32), dl.astype(np.float32), tmin)
        upd = t < best_t
        best_t[upd], best_g[upd] = t[upd], gi
        best_n[upd] = (nl @ Rw.T)[upd]
    return best_t, best_n, best_g


def render_reference(geoms, xpos, xmat, cams, H, W, light):
    """float32 NumPy restatement of the kernel: → (uint8 [n, cams, H, W, 3], float32 depth)."""
    n = xpos.shape[0]
    rgb = np.zeros((n, len(cams), H, W, 3), np.uint8)
    depth = np.zeros((n, len(cams), H, W), np.float32)
    py, px = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    for w in range(n):
        for ci, C in enumerate(cams):
            o0 = C[0:3].astype(np.float32).copy()
            if int(C[13]) >= 0:
                o0 = o0 + xpos[w, int(C[13])].astype(np.float32)
            rot = C[3:12].reshape(3, 3).astype(np.float32)
            th = np.float32(np.tan(0.5 * C[12]))
            u = ((2 * (px + 0.5) / W - 1) * th * (W / H)).astype(np.float32).reshape(-1)
            v = ((1 - 2 * (py + 0.5) / H) * th).astype(np.float32).reshape(-1)
            d = u[:, None] * rot[:, 0] + v[:, None] * rot[:, 1] - rot[:, 2]
            d = (d / np.linalg.norm(d, axis=1, keepdims=True)).astype(np.float32)
            o = np.tile(o0, (H * W, 1))
            t, nn, g = _trace(geoms, xpos[w], xmat[w], o, d, 1e-4)
            hit = g >= 0
            s = 0.5 * (d[:, 2] + 1)
            col = np.stack([0.55 + 0.25 * (1 - s), 0.70 + 0.15 * (1 - s), np.full_like(s, 0.95)], 1).astype(np.float32)
            if hit.any():
                hp = o[hit] + t[hit, None] * d[hit]
                base = geoms[g[hit], 17:20].astype(np.float32).copy()
                plane = geoms[g[hit], 0] == 0
                check_f = np.where((np.floor(hp[:, 0] * 2).astype(np.int64) + np.floor(hp[:, 1] * 2).astype(np.int64)) & 1, 1.0, 0.6)
                base[plane] *= check_f[plane, None].astype(np.float32)
                nh = nn[hit].copy()
                flip = (nh * d[hit]).sum(1) > 0
                nh[flip] = -nh[flip]
                L = light[0:3].astype(np.float32)
                diff = np.maximum(nh @ L, 0)
                if light[5] != 0:
                    so = hp + 1e-3 * nh
                    _, _, sg = _trace(geoms, xpos[w], xmat[w], so.astype(np.float32), np.tile(L, (len(so), 1)), 1e-4)
                    diff = np.where((sg >= 0) & (diff > 0), 0, diff)
                lum = light[3] + light[4] * diff
                col[hit] = np.minimum(base * lum[:, None], 1.0)
            rgb[w, ci] = (col * 255 + 0.5).astype(np.uint8).reshape(H, W, 3)
            depth[w, ci] = np.where(hit, t, 0).reshape(H, W)
    return rgb, depth
