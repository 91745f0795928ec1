"""2-D navigation on occupancy grids: batched value iteration as a tensor program (many goals / maps at once), A* for a single
query, and path shortcutting.

``distance_field(occ, goals)``   cost-to-go from every free cell to its map's goal over the 8-connected grid (diagonal moves cost
                                 √2, no corner cutting), computed by min-plus sweeps until nothing changes: one tensor op per
                                 sweep for the whole batch of maps (CPU or GPU)
``descend(field, start)``        the path that follows the steepest descent of a distance field
``astar(occ, start, goal)``      heap-based A* with the octile heuristic (optimal on the same move set)
``shortcut(occ, path)``          removes way-points whose neighbours see each other (line-of-sight test on the grid)
(noeira/planners/nav2d/.)
"""
from __future__ import annotations

import heapq
import math
from typing import List, Optional, Tuple

import torch

_MOVES = [(-1, 0, 1.0), (1, 0, 1.0), (0, -1, 1.0), (0, 1, 1.0), (-1, -1, math.sqrt(2)), (-1, 1, math.sqrt(2)), (1, -1, math.sqrt(2)),
          (1, 1, math.sqrt(2))]


def distance_field(occ: torch.Tensor, goals: torch.Tensor, max_sweeps: int = 0) -> torch.Tensor:
    """occ ``[B, H, W]`` bool (True = blocked), goals ``[B, 2]`` (row, col) → ``[B, H, W]`` cost-to-go (inf where unreachable)."""
    B, H, W = occ.shape
    inf = float("inf")
    d = torch.full((B, H, W), inf, device=occ.device)
    d[torch.arange(B, device=occ.device), goals[:, 0], goals[:, 1]] = 0.0
    free = ~occ
    pad_occ = torch.nn.functional.pad(occ, (1, 1, 1, 1), value=True)
    for _ in range(max_sweeps or 4 * (H + W)):
        p = torch.nn.functional.pad(d, (1, 1, 1, 1), value=inf)
        best = d
        for dr, dc, cost in _MOVES:
            nb = p[:, 1 + dr: 1 + dr + H, 1 + dc: 1 + dc + W] + cost
            if dr and dc:          # a diagonal move needs both orthogonal neighbours free
                clear = ~pad_occ[:, 1 + dr: 1 + dr + H, 1: 1 + W] & ~pad_occ[:, 1: 1 + H, 1 + dc: 1 + dc + W]
                nb = torch.where(clear, nb, torch.full_like(nb, inf))
            best = torch.minimum(best, nb)
        best = torch.where(free, best, torch.full_like(best, inf))
        if torch.equal(best, d):
            break
        d = best
    return d


def descend(field: torch.Tensor, start: Tuple[int, int], occ: Optional[torch.Tensor] = None) -> List[Tuple[int, int]]:
    """Steepest-descent path on ONE map's field ``[H, W]`` from ``start`` to the goal (empty if unreachable)."""
    H, W = field.shape
    r, c = start
    if not math.isfinite(float(field[r, c])):
        return []
    path = [(r, c)]
    while float(field[r, c]) > 0:
        nxt = None
        for dr, dc, cost in _MOVES:
            rr, cc = r + dr, c + dc
            if not (0 <= rr < H and 0 <= cc < W) or not math.isfinite(float(field[rr, cc])):
                continue
            if dr and dc and occ is not None and (bool(occ[rr, c]) or bool(occ[r, cc])):
                continue
            v = float(field[rr, cc]) + cost              # Bellman: the best neighbour reproduces this cell's value
            if nxt is None or v < nxt[0]:
                nxt = (v, rr, cc)
        if nxt is None or nxt[0] > float(field[r, c]) + 1e-4 or len(path) > H * W:
            return []
        r, c = nxt[1], nxt[2]
        path.append((r, c))
    return path


def astar(occ, start: Tuple[int, int], goal: Tuple[int, int]):
    """→ (path, cost) on one map ``[H, W]`` (bool tensor or nested lists); ``([], inf)`` if there is no path."""
    grid = occ.tolist() if hasattr(occ, "tolist") else occ
    H, W = len(grid), len(grid[0])

    def h(r, c):
        dr, dc = abs(r - goal[0]), abs(c - goal[1])
        return max(dr, dc) + (math.sqrt(2) - 1) * min(dr, dc)

    openq = [(h(*start), 0.0, start)]
    g, parent = {start: 0.0}, {}
    while openq:
        _, gc, cur = heapq.heappop(openq)
        if cur == goal:
            path = [cur]
            while cur in parent:
                cur = parent[cur]
                path.append(cur)
            return path[::-1], gc
        if gc > g.get(cur, math.inf):
            continue
        r, c = cur
        for dr, dc, cost in _MOVES:
            rr, cc = r + dr, c + dc
            if not (0 <= rr < H and 0 <= cc < W) or grid[rr][cc]:
                continue
            if dr and dc and (grid[rr][c] or grid[r][cc]):
                continue
            ng = gc + cost
            if ng < g.get((rr, cc), math.inf) - 1e-12:
                g[(rr, cc)], parent[(rr, cc)] = ng, cur
                heapq.heappush(openq, (ng + h(rr, cc), ng, (rr, cc)))
    return [], math.inf


def _visible(grid, a, b) -> bool:
    (r0, c0), (r1, c1) = a, b
    n = int(max(abs(r1 - r0), abs(c1 - c0)) * 2) + 1
    for i in range(n + 1):
        t = i / n
        r, c = r0 + (r1 - r0) * t, c0 + (c1 - c0) * t
        for rr in {math.floor(r + 1e-9), math.ceil(r - 1e-9)}:
            for cc in {math.floor(c + 1e-9), math.ceil(c - 1e-9)}:
                if grid[rr][cc]:
                    return False
    return True


def shortcut(occ, path: List[Tuple[int, int]]) -> List[Tuple[int, int]]:
    grid = occ.tolist() if hasattr(occ, "tolist") else occ
    if len(path) < 3:
        return list(path)
    out, i = [path[0]], 0
    while i < len(path) - 1:
        j = len(path) - 1
        while j > i + 1 and not _visible(grid, path[i], path[j]):
            j -= 1
        out.append(path[j])
        i = j
    return out
