"""Sheaf world model with holonomy as an observable.

Local representations are stalks (vectors in R^d) on a graph of places; the transports between neighbouring places are
ORTHOGONAL matrices attached to the edges of the graph (never to coordinates of the latents).  Each transport is fitted
on its own edge from observation pairs (orthogonal Procrustes); the holonomy around a cycle, the ordered product of its
transports, is then READ and never optimised: ``det H = −1`` says that the cycle reverses orientation (a corridor whose seam
mirrors the frame is a Möbius strip: consistent on every edge, inconsistent around the loop), which no per-edge noise can
produce.  A cocycle loss ``‖H − I‖²`` cannot learn this: for any reflection it equals ``4 − 2 tr H``, constant on the
``det = −1`` component.

Pieces: O(d) algebra (``skew_from_vector``, ``cayley``, ``expm_skew``, ``householder``), ``procrustes`` by Newton's
iteration for the polar factor (matrix products and inverses only, keeps ``sign det``), ``PlaceGraph`` (spanning-tree
gauge, fundamental cycles, holonomy and its classification), the dense sheaf Laplacian ``δᵀδ`` and Dirichlet-energy
inference (descent and the exact solve), graduated-non-convexity edge confidences, the ``MobiusRing`` world (a transported
landmark mixed with non-transported texture), per-edge fitting from its samples, and a breadth-first planner on the
double cover (place, orientation bit).

Reference: noeira/experimental/swm/ (so_d.mojo, procrustes.mojo, place_graph.mojo, sheaf_laplacian.mojo,
sheaf_inference.mojo, observables.mojo, envs/mobius_ring.mojo, graph_planner.mojo).
"""
from __future__ import annotations

import math
from collections import deque
from typing import Dict, List, Optional, Sequence, Tuple

import torch

DT = torch.float64


# ---- O(d) ---------------------------------------------------------------------------------------------------------------
def skew_from_vector(v: torch.Tensor, d: int) -> torch.Tensor:
    """The d(d−1)/2 entries of ``v`` as the strict upper triangle of a skew-symmetric matrix."""
    a = torch.zeros(d, d, dtype=v.dtype)
    iu = torch.triu_indices(d, d, 1)
    a[iu[0], iu[1]] = v
    return a - a.T


def cayley(a: torch.Tensor) -> torch.Tensor:
    """(I − A)⁻¹ (I + A) ∈ SO(d) for skew A."""
    eye = torch.eye(a.shape[-1], dtype=a.dtype)
    return torch.linalg.solve(eye - a, eye + a)


def expm_skew(a: torch.Tensor) -> torch.Tensor:
    return torch.linalg.matrix_exp(a)


def householder(u: torch.Tensor) -> torch.Tensor:
    """The reflection through the hyperplane normal to u (det = −1)."""
    u = u / u.norm()
    return torch.eye(u.numel(), dtype=u.dtype) - 2.0 * torch.outer(u, u)


def polar_orthogonal(m: torch.Tensor, iters: int = 60, tol: float = 1e-14) -> torch.Tensor:
    """Orthogonal polar factor of a non-singular matrix by Newton's iteration Q ← ½ (Q + Q⁻ᵀ)."""
    q = m.clone()
    for _ in range(iters):
        nxt = 0.5 * (q + torch.linalg.inv(q).T)
        if (nxt - q).abs().max() < tol:
            return nxt
        q = nxt
    return q


def procrustes(x: torch.Tensor, y: torch.Tensor) -> Tuple[torch.Tensor, float]:
    """argmin over R ∈ O(d) of Σ ‖R x_k − y_k‖² for samples in the ROWS of x, y [n, d] → (R, rms residual).  R is the polar
    factor of Yᵀ X, so a reflection in the data comes out as a reflection."""
    r = polar_orthogonal(y.T @ x)
    res = (x @ r.T - y).pow(2).sum(1).mean().sqrt()
    return r, float(res)


# ---- the graph of places -----------------------------------------------------------------------------------------------
class PlaceGraph:
    """Undirected graph whose edge (i, j) carries R_ij with x_j ≈ R_ij x_i (and R_ji = R_ijᵀ), a residual and a confidence."""

    def __init__(self, n: int, d: int):
        self.n, self.d = n, d
        self.edges: Dict[Tuple[int, int], torch.Tensor] = {}
        self.residual: Dict[Tuple[int, int], float] = {}
        self.weight: Dict[Tuple[int, int], float] = {}

    def add_edge(self, i: int, j: int, r: torch.Tensor, residual: float = 0.0, weight: float = 1.0):
        self.edges[(i, j)] = r.to(DT)
        self.residual[(i, j)], self.weight[(i, j)] = float(residual), float(weight)

    def transport(self, i: int, j: int) -> torch.Tensor:
        return self.edges[(i, j)] if (i, j) in self.edges else self.edges[(j, i)].T

    def neighbours(self, i: int) -> List[int]:
        return sorted({b for a, b in self.edges if a == i} | {a for a, b in self.edges if b == i})

    def spanning_tree(self, root: int = 0):
        """→ (parent per node, frames G_i with x_i = G_i x_root along the tree, the non-tree edges)."""
        parent = {root: None}
        frame = {root: torch.eye(self.d, dtype=DT)}
        queue = deque([root])
        while queue:
            i = queue.popleft()
            for j in self.neighbours(i):
                if j not in parent:
                    parent[j] = i
                    frame[j] = self.transport(i, j) @ frame[i]
                    queue.append(j)
        chords = [e for e in self.edges if parent.get(e[1]) != e[0] and parent.get(e[0]) != e[1]]
        return parent, frame, chords

    def fundamental_cycles(self, root: int = 0) -> List[List[int]]:
        """One cycle per non-tree edge: root-ward tree path of one end, the chord, tree path back (as a closed node list)."""
        parent, _, chords = self.spanning_tree(root)

        def up(i):
            path = [i]
            while parent[path[-1]] is not None:
                path.append(parent[path[-1]])
            return path
        cycles = []
        for a, b in chords:
            pa, pb = up(a), up(b)
            in_b = set(pb)
            common = next(x for x in pa if x in in_b)
            # the closed walk: common → … → a, the chord a → b, b → … → common
            cycles.append(pa[: pa.index(common) + 1][::-1] + pb[: pb.index(common) + 1])
        return cycles

    def holonomy(self, cycle: Sequence[int]) -> torch.Tensor:
        """Product of the transports along a closed node list (first node == last node)."""
        h = torch.eye(self.d, dtype=DT)
        for i, j in zip(cycle[:-1], cycle[1:]):
            h = self.transport(i, j) @ h
        return h

    def classify_cycle(self, cycle: Sequence[int], tol: float = 1e-6) -> Dict[str, float]:
        """det H (±1), the number of invariant directions dim ker(H − I), and the summed edge residual of the cycle."""
        h = self.holonomy(cycle)
        sv = torch.linalg.svdvals(h - torch.eye(self.d, dtype=DT))
        res = sum(self.residual.get((i, j), self.residual.get((j, i), 0.0)) for i, j in zip(cycle[:-1], cycle[1:]))
        return {"det": float(torch.sign(torch.linalg.det(h))), "invariant_dims": int((sv < tol).sum()), "residual": res}


def sheaf_laplacian(g: PlaceGraph) -> torch.Tensor:
    """Dense L = δᵀ W δ [n d, n d] with (δ x)_e = R_ij x_i − x_j."""
    n, d = g.n, g.d
    lap = torch.zeros(n * d, n * d, dtype=DT)
    eye = torch.eye(d, dtype=DT)
    for (i, j), r in g.edges.items():
        w = g.weight[(i, j)]
        si, sj = slice(i * d, (i + 1) * d), slice(j * d, (j + 1) * d)
        lap[si, si] += w * eye              # RᵀR = I
        lap[sj, sj] += w * eye
        lap[si, sj] -= w * r.T
        lap[sj, si] -= w * r
    return lap


def dirichlet_energy(g: PlaceGraph, x: torch.Tensor) -> torch.Tensor:
    return sum(g.weight[e] * (r @ x[e[0]] - x[e[1]]).pow(2).sum() for e, r in g.edges.items())


def sheaf_inference(g: PlaceGraph, observed: Dict[int, torch.Tensor], iters: int = 0, lr: float = None) -> torch.Tensor:
    """The section [n, d] of least Dirichlet energy that agrees with ``observed`` on its nodes: ``iters = 0`` solves the
    linear system of the free block, otherwise that many steps of gradient descent (step 1 / max degree by default)."""
    n, d = g.n, g.d
    lap = sheaf_laplacian(g)
    x = torch.zeros(n, d, dtype=DT)
    for i, v in observed.items():
        x[i] = v.to(DT)
    free = [i for i in range(n) if i not in observed]
    if not free:
        return x
    fidx = torch.tensor([i * d + k for i in free for k in range(d)])
    bidx = torch.tensor([i * d + k for i in observed for k in range(d)])
    lff, lfb = lap[fidx][:, fidx], lap[fidx][:, bidx]
    xb = torch.cat([x[i] for i in observed])
    if iters == 0:
        xf = torch.linalg.solve(lff, -lfb @ xb)
    else:
        step = lr if lr is not None else 1.0 / float(lff.diagonal().max())
        xf = torch.zeros(len(fidx), dtype=DT)
        for _ in range(iters):
            xf = xf - step * (lff @ xf + lfb @ xb)
    x.view(-1)[fidx] = xf
    return x


def gnc_confidence(residuals: Sequence[float], c: float, mu: float = 1.0) -> List[float]:
    """Geman–McClure weights of graduated non-convexity: w = (μ c² / (r² + μ c²))²; a residual far above the scale c gets a
    weight near zero, one at the scale gets ¼ for μ = 1."""
    return [(mu * c * c / (r * r + mu * c * c)) ** 2 for r in residuals]


# ---- a world: the ring with a seam --------------------------------------------------------------------------------------
class MobiusRing:
    """A ring of ``n`` cells.  A landmark vector in R^d is carried from cell to cell by a fixed rotation per step; the step
    from cell n − 1 to cell 0 returns to the first frame, through a reflection when ``twist`` (the holonomy of the ring is
    then that reflection, otherwise the identity).  An observation at a cell is that landmark in
    the cell's frame plus noise, concatenated with ``texture`` values that belong to the cell and are NOT transported."""

    def __init__(self, n: int = 12, d: int = 2, twist: bool = True, noise: float = 0.01, texture: int = 2, seed: int = 0):
        self.n, self.d, self.twist, self.noise, self.texture = n, d, twist, noise, texture
        g = torch.Generator().manual_seed(seed)
        self.gen = g
        self.step_rot = [expm_skew(skew_from_vector(0.4 * torch.randn(d * (d - 1) // 2, generator=g, dtype=DT), d)) for _ in range(n)]
        self.tex = torch.randn(n, texture, generator=g, dtype=DT)
        self.frames = [torch.eye(d, dtype=DT)]
        for i in range(n - 1):
            self.frames.append(self.step_rot[i] @ self.frames[-1])
        # the last step closes the ring: back to the frame of cell 0, through a mirror when twisted
        seam = householder(torch.randn(d, generator=g, dtype=DT)) if twist else torch.eye(d, dtype=DT)
        self.step_rot[n - 1] = seam @ self.frames[n - 1].T

    def true_transport(self, i: int) -> torch.Tensor:
        """From cell i to cell (i + 1) mod n."""
        return self.step_rot[i]

    def observe(self, cell: int, landmark: torch.Tensor) -> torch.Tensor:
        """``landmark`` is given in the frame of cell 0 on the current sheet."""
        z = self.frames[cell] @ landmark + self.noise * torch.randn(self.d, generator=self.gen, dtype=DT)
        return torch.cat([z, self.tex[cell] + self.noise * torch.randn(self.texture, generator=self.gen, dtype=DT)])

    def sample_edge(self, i: int, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """k observation pairs (at cell i, after one step forward) of random landmarks → ([k, d + texture], same)."""
        a, b = [], []
        for _ in range(k):
            lm = torch.randn(self.d, generator=self.gen, dtype=DT)
            here = self.frames[i] @ lm
            there = self.step_rot[i] @ here
            nz = lambda m: self.noise * torch.randn(m, generator=self.gen, dtype=DT)
            a.append(torch.cat([here + nz(self.d), self.tex[i] + nz(self.texture)]))
            b.append(torch.cat([there + nz(self.d), self.tex[(i + 1) % self.n] + nz(self.texture)]))
        return torch.stack(a), torch.stack(b)


def fit_ring(world: MobiusRing, samples: int = 40, frame_dims: Optional[Sequence[int]] = None) -> PlaceGraph:
    """One Procrustes fit per edge on the frame channel of the observation pairs (the first d values unless given)."""
    dims = list(range(world.d)) if frame_dims is None else list(frame_dims)
    g = PlaceGraph(world.n, len(dims))
    for i in range(world.n):
        a, b = world.sample_edge(i, samples)
        r, res = procrustes(a[:, dims], b[:, dims])
        g.add_edge(i, (i + 1) % world.n, r, res)
    return g


def transported_fraction(a: torch.Tensor, b: torch.Tensor, dims: Sequence[int]) -> float:
    """R² of the best orthogonal map between the chosen channels of an observation pair set: near 1 for a channel that is
    transported, near 0 for texture that merely belongs to the cells."""
    x, y = a[:, list(dims)], b[:, list(dims)]
    x, y = x - x.mean(0), y - y.mean(0)
    if float(torch.linalg.matrix_rank(y.T @ x)) < len(dims):
        return 0.0
    r, _ = procrustes(x, y)
    return float(1.0 - (x @ r.T - y).pow(2).sum() / y.pow(2).sum().clamp_min(1e-30))


# ---- planning on the double cover --------------------------------------------------------------------------------------
def plan_double_cover(g: PlaceGraph, start: int, goal: int, goal_parity: int, start_parity: int = 0) -> Optional[List[int]]:
    """Shortest node path from ``start`` to ``goal`` that arrives with the requested orientation bit: states are (place, u)
    and an edge flips u when its transport has determinant −1 (breadth-first search)."""
    flips = {}
    for (i, j), r in g.edges.items():
        f = int(torch.linalg.det(r) < 0)
        flips[(i, j)] = flips[(j, i)] = f
    first = (start, start_parity)
    prev = {first: None}
    queue = deque([first])
    while queue:
        s = queue.popleft()
        if s == (goal, goal_parity):
            path = []
            while s is not None:
                path.append(s[0])
                s = prev[s]
            return path[::-1]
        for j in g.neighbours(s[0]):
            t = (j, s[1] ^ flips[(s[0], j)])
            if t not in prev:
                prev[t] = s
                queue.append(t)
    return None
