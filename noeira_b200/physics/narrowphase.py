"""Convex narrow phase and broad phase for the general engine.

* ``gjk_epa``: distance (GJK with Johnson's sub-algorithm on simplices of up to four points) or penetration (expanding
  polytope) of two convex point sets, each optionally inflated by a radius, so that spheres (one point), capsules (two
  points), boxes (eight corners) and convex meshes (their vertices) all go through one routine.  Exact, float64, one pair
  at a time on the host: the batched engine loops over its lanes for these pairs.
* ``contact_manifold``: up to five contacts of a pair from the one GJK gives, by re-running it with the second shape
  turned by a small angle about the two tangent axes (faces that rest on faces get a supporting polygon).
* ``mesh_mass_inertia``: volume integrals of the convex hull of a vertex set.
* ``HeightField``: bilinear terrain, height and normal at batched points.
* ``sap_overlaps``: sweep-and-prune on the axis of largest spread, batched: which of the candidate pairs have overlapping
  bounding boxes in ANY lane of the batch.

Reference: noeira/physics3d/collision/ (GJK / EPA, multicontact, convex hull, hfield, SAP broad phase for ≥ 16 geoms).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


# ---- GJK ----------------------------------------------------------------------------------------------------------------
def _support(va: np.ndarray, vb: np.ndarray, d: np.ndarray):
    ia, ib = int(np.argmax(va @ d)), int(np.argmax(vb @ -d))
    return va[ia] - vb[ib], ia, ib


def _closest_on_simplex(pts: np.ndarray):
    """Point of the convex hull of 1–4 points nearest to the origin → (point, barycentric weights); weights of vertices
    that do not support the point are zero (Johnson's sub-algorithm by enumeration of the faces)."""
    n = len(pts)
    best, best_w = None, None
    # enumerate non-empty subsets, smallest first; a subset is the answer when the projection of the origin on its affine
    # hull has positive weights and no other vertex improves it: equivalently, take the feasible subset of least distance
    for mask in range(1, 1 << n):
        idx = [i for i in range(n) if mask >> i & 1]
        p = pts[idx]
        if len(idx) == 1:
            w = np.array([1.0])
        else:
            e = (p[1:] - p[0]).T                                   # [3, k]
            g = e.T @ e
            try:
                lam = np.linalg.solve(g, -e.T @ p[0])
            except np.linalg.LinAlgError:
                continue
            w = np.concatenate([[1.0 - lam.sum()], lam])
            if (w < -1e-12).any():
                continue
        q = w @ p
        d = float(q @ q)
        if best is None or d < best - 1e-18:
            best = d
            best_w = np.zeros(n)
            best_w[idx] = np.clip(w, 0.0, None)
    return best_w @ pts, best_w


def gjk_epa(va: np.ndarray, vb: np.ndarray, ra: float = 0.0, rb: float = 0.0, tol: float = 1e-10, max_iter: int = 64):
    """→ (signed distance, normal from A to B, point on A, point on B) of the convex hulls of ``va`` and ``vb`` inflated
    by ``ra`` and ``rb``.  Negative distance = penetration depth along the normal."""
    d = va.mean(0) - vb.mean(0)
    if float(d @ d) < 1e-20:
        d = np.array([1.0, 0.0, 0.0])
    w, ia, ib = _support(va, vb, -d)
    simplex, sa, sb = [w], [ia], [ib]
    v = w
    for _ in range(max_iter):
        vv = float(v @ v)
        if vv < 1e-20:
            break                                                   # the origin is in the simplex: the cores overlap
        w, ia, ib = _support(va, vb, -v)
        if vv - float(v @ w) <= tol * max(vv, 1.0) or any((ia == a and ib == b) for a, b in zip(sa, sb)):
            break                                                   # no progress towards the origin: v is the closest point
        simplex.append(w), sa.append(ia), sb.append(ib)
        v, bw = _closest_on_simplex(np.array(simplex))
        keep = [i for i in range(len(simplex)) if bw[i] > 0]
        simplex, sa, sb = [simplex[i] for i in keep], [sa[i] for i in keep], [sb[i] for i in keep]
        if len(simplex) == 4:
            v = np.zeros(3)
            break
    dist = float(np.linalg.norm(v))
    if dist > 1e-9:
        _, bw = _closest_on_simplex(np.array(simplex))
        pa, pb = bw @ va[sa], bw @ vb[sb]
        n = -v / dist                                               # v = a − b points from B to A
        return dist - ra - rb, n, pa + ra * n, pb - rb * n
    depth, n, pa, pb = _epa(va, vb, simplex, sa, sb)
    return -depth - ra - rb, n, pa + ra * n, pb - rb * n


def _epa(va, vb, simplex, sa, sb, max_iter: int = 64, tol: float = 1e-9):
    """Expanding polytope from a simplex that contains the origin → (depth, normal A→B, point on A, point on B)."""
    pts, ia_l, ib_l = list(simplex), list(sa), list(sb)
    # grow a degenerate simplex to a tetrahedron with supports along coordinate directions
    dirs = [np.array(x, float) for x in ((1, 0, 0), (-1, 0, 0), (0, 1, 0), (0, -1, 0), (0, 0, 1), (0, 0, -1))]
    k = 0
    while len(pts) < 4 and k < len(dirs):
        w, ia, ib = _support(va, vb, dirs[k])
        k += 1
        cand = np.array(pts + [w])
        if np.linalg.matrix_rank(cand - cand[0], tol=1e-9) == len(pts):
            pts.append(w), ia_l.append(ia), ib_l.append(ib)
    if len(pts) < 4:                                                # flat Minkowski difference: touching, zero depth
        n = np.array([0.0, 0.0, 1.0])
        return 0.0, n, va[ia_l[0]], vb[ib_l[0]]
    faces = [(0, 1, 2), (0, 3, 1), (0, 2, 3), (1, 3, 2)]

    centre = np.mean(pts, 0)
    oriented = []
    for f in faces:
        a, b, c = (pts[i] for i in f)
        if float(np.cross(b - a, c - a) @ (a - centre)) < 0:
            f = (f[0], f[2], f[1])
        oriented.append(f)
    faces = oriented
    for _ in range(max_iter):
        best, bn, bd = None, None, np.inf
        for f in faces:
            a, b, c = (pts[i] for i in f)
            n = np.cross(b - a, c - a)
            ln = np.linalg.norm(n)
            if ln < 1e-14:
                continue
            n = n / ln
            dd = float(n @ a)
            if dd < bd:
                best, bn, bd = f, n, dd
        w, ia, ib = _support(va, vb, bn)
        if float(bn @ w) - bd < tol:
            break
        pts.append(w), ia_l.append(ia), ib_l.append(ib)
        new = len(pts) - 1
        visible = [f for f in faces if float(np.cross(pts[f[1]] - pts[f[0]], pts[f[2]] - pts[f[0]]) @ (w - pts[f[0]])) > 1e-14]
        edges = {}
        for f in visible:
            for e in ((f[0], f[1]), (f[1], f[2]), (f[2], f[0])):
                if (e[1], e[0]) in edges:
                    del edges[(e[1], e[0])]
                else:
                    edges[e] = True
        faces = [f for f in faces if f not in visible] + [(e[0], e[1], new) for e in edges]
    a, b, c = (pts[i] for i in best)
    proj = bn * bd                                                  # the origin projected on the nearest face
    m = np.array([b - a, c - a]).T
    lam, *_ = np.linalg.lstsq(m, proj - a, rcond=None)
    wts = np.array([1 - lam.sum(), lam[0], lam[1]])
    pa = wts @ va[[ia_l[i] for i in best]]
    pb = wts @ vb[[ib_l[i] for i in best]]
    # A − B reaches the origin's nearest boundary point at bd·n: moving B by that vector shifts the difference by its negative
    # and puts the origin on the boundary, so n is the direction from A to B
    return bd, bn, pa, pb


def contact_manifold(va, vb, ra=0.0, rb=0.0, centre_b: Optional[np.ndarray] = None, angle: float = 0.02, margin: float = 0.0):
    """One to five contacts (point, normal A→B, depth) of a pair: the GJK / EPA contact plus those found with B turned by
    ±``angle`` about the two tangents of the first normal (about ``centre_b``), kept when they touch within ``margin``."""
    dist, n, pa, pb = gjk_epa(va, vb, ra, rb)
    out = [(0.5 * (pa + pb), n, -dist)]
    if dist > margin or len(vb) < 3 or len(va) < 3:
        return out
    c = vb.mean(0) if centre_b is None else centre_b
    ref = np.array([1.0, 0, 0]) if abs(n[0]) < 0.9 else np.array([0, 1.0, 0])
    t1 = np.cross(n, ref)
    t1 /= np.linalg.norm(t1)
    t2 = np.cross(n, t1)
    for ax in (t1, -t1, t2, -t2):
        K = np.array([[0, -ax[2], ax[1]], [ax[2], 0, -ax[0]], [-ax[1], ax[0], 0]])
        R = np.eye(3) + np.sin(angle) * K + (1 - np.cos(angle)) * K @ K
        vb2 = (vb - c) @ R.T + c
        d2, n2, pa2, pb2 = gjk_epa(va, vb2, ra, rb)
        # undo the turn for the point on B, measure its depth along the unperturbed normal
        pb0 = (pb2 - c) @ R + c
        depth = float((pa2 - pb0) @ n)
        p = 0.5 * (pa2 + pb0)
        if depth > -margin - 1e-9 and all(np.linalg.norm(p - q[0]) > 1e-4 for q in out):
            out.append((p, n, depth))
    return out


# ---- mass properties of a convex mesh -------------------------------------------------------------------------------------
def mesh_mass_inertia(vertices: Sequence[Sequence[float]], density: float):
    """(mass, diagonal inertia about the centre of mass in the mesh axes, centre of mass) of the convex hull."""
    from scipy.spatial import ConvexHull
    v = np.asarray(vertices, float)
    hull = ConvexHull(v)
    inside = v[hull.vertices].mean(0)
    vol, first, second = 0.0, np.zeros(3), np.zeros((3, 3))
    canon = (np.ones((3, 3)) + np.eye(3)) / 120.0                 # ∫ x xᵀ over the unit tetrahedron, per unit determinant
    for tri in hull.simplices:
        a, b, c = v[tri] - inside
        det = float(np.dot(a, np.cross(b, c)))
        if det < 0:
            b, c, det = c, b, -det
        vol += det / 6.0
        first += det / 24.0 * (a + b + c)
        m = np.array([a, b, c]).T
        second += det * m @ canon @ m.T
    com_rel = first / vol
    cov = second - vol * np.outer(com_rel, com_rel)               # ∫ (x − c)(x − c)ᵀ
    inertia = np.array([cov[1, 1] + cov[2, 2], cov[0, 0] + cov[2, 2], cov[0, 0] + cov[1, 1]])
    return density * vol, (density * inertia).tolist(), (inside + com_rel).tolist()


# ---- terrain ---------------------------------------------------------------------------------------------------------------
class HeightField:
    """Heights ``data [ny, nx]`` over the rectangle [−half_x, half_x] × [−half_y, half_y] about ``pos``, bilinear between
    the samples, clamped at the border."""

    def __init__(self, data, half_x: float, half_y: float, pos=(0.0, 0.0, 0.0), friction: float = 1.0):
        self.data = torch.as_tensor(np.asarray(data), dtype=torch.float64)
        self.half_x, self.half_y, self.pos, self.friction = float(half_x), float(half_y), tuple(float(p) for p in pos), friction

    def sample(self, x: torch.Tensor, y: torch.Tensor):
        """→ (height, unit normal [..., 3]) at world (x, y)."""
        d = self.data.to(x.device, x.dtype)
        ny, nx = d.shape
        dx, dy = 2 * self.half_x / (nx - 1), 2 * self.half_y / (ny - 1)
        u = ((x - self.pos[0] + self.half_x) / dx).clamp(0, nx - 1 - 1e-9)
        v = ((y - self.pos[1] + self.half_y) / dy).clamp(0, ny - 1 - 1e-9)
        i, j = v.floor().long(), u.floor().long()
        fv, fu = v - i, u - j
        h00, h01, h10, h11 = d[i, j], d[i, j + 1], d[i + 1, j], d[i + 1, j + 1]
        h = (1 - fv) * ((1 - fu) * h00 + fu * h01) + fv * ((1 - fu) * h10 + fu * h11)
        hx = ((1 - fv) * (h01 - h00) + fv * (h11 - h10)) / dx
        hy = ((1 - fu) * (h10 - h00) + fu * (h11 - h01)) / dy
        n = torch.stack([-hx, -hy, torch.ones_like(hx)], -1)
        return h + self.pos[2], n / n.norm(dim=-1, keepdim=True)

    def contact(self, p: torch.Tensor, radius: float):
        """Sphere of ``radius`` at p [B, 3] → (contact point, normal, depth): distance measured along the surface normal
        under the centre (exact on planar patches)."""
        h, n = self.sample(p[:, 0], p[:, 1])
        gap = (p[:, 2] - h) * n[:, 2]
        depth = radius - gap
        return p - n * (radius - 0.5 * depth)[:, None], n, depth


# ---- broad phase -----------------------------------------------------------------------------------------------------------
def sap_overlaps(lo: torch.Tensor, hi: torch.Tensor, pairs: Sequence[Tuple[int, int]]) -> List[bool]:
    """Sweep and prune: ``lo, hi [B, G, 3]`` bounding boxes of the geoms → for each candidate pair, whether the boxes overlap
    in any lane.  Sorting the interval starts along the axis of largest spread bounds the sweep: a geom is tested only
    against those whose start lies before its end."""
    B, G, _ = lo.shape
    axis = int((hi - lo).sum(1).add(lo.amax(1) - lo.amin(1)).mean(0).argmax()) if G > 1 else 0
    order = lo[:, :, axis].argsort(1)                                           # [B, G]
    rank = torch.empty_like(order)
    rank.scatter_(1, order, torch.arange(G, device=lo.device)[None].expand(B, G))
    start = lo[:, :, axis]
    end = hi[:, :, axis]
    # number of starts that lie at or before each geom's end = how far the sweep from that geom reaches
    sorted_start = torch.gather(start, 1, order)
    reach = torch.searchsorted(sorted_start.contiguous(), end.contiguous(), right=True)        # [B, G]
    out = []
    for i, j in pairs:
        first_is_i = rank[:, i] < rank[:, j]
        a = torch.where(first_is_i, i, j)
        b_rank = torch.where(first_is_i, rank[:, j], rank[:, i])
        swept = b_rank < torch.gather(reach, 1, a[:, None])[:, 0]                              # on the sweep axis
        other = ((lo[:, i] <= hi[:, j]) & (lo[:, j] <= hi[:, i])).all(-1)                      # and on all axes
        out.append(bool((swept & other).any()))
    return out
