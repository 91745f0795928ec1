"""Placement sampling: every ``init=`` of a task is a DISTRIBUTION, drawn again at each reset.

``sample_placements`` draws, for N environments at once, a pose for every initialised slot:
  * a region target: uniform inside the region's rectangle about its site, rejected (and redrawn, per environment)
    while the circle of the new object overlaps an already placed one — distance below
    ``max(r_i + r_j, sep_i, sep_j)``; height = site z + TABLE_Z_OFFSET − bottom_z (an ``:in`` init omits the fixture's
    own top offset, an ``On`` init onto a fixture region adds it);
  * a slot target (a stack): directly on top of that slot, at its x / y, no draw;
  * ``:yaw`` draws a yaw uniformly on (−π, π].
``build_init_table`` precomputes K such placements on the device so that a reset is an index draw and a gather — no
rejection loop inside the step (reference: noeira/tasks/sampler.mojo:1-561, noeira/tasks/init_table.mojo).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .spec import (INIT_TARGET_REGION, SLOT_FREE, STACK_Z_OFFSET, TABLE_Z_OFFSET, FamilySpec, TaskSpec, order_inits,
                   validate_task_against_family)

DEFAULT_RADIUS = 0.02
MAX_REJECTION_ROUNDS = 64


@dataclass
class Placements:
    pos: torch.Tensor     # [N, S, 3]  (inactive free slots sit at the family's park pose)
    quat: torch.Tensor    # [N, S, 4]  (w, x, y, z)
    ok: torch.Tensor      # [N] bool: every rejection test was satisfied within the round limit


def sample_placements(task: TaskSpec, family: FamilySpec, site_pos: Dict[str, torch.Tensor], n: int,
                      generator: Optional[torch.Generator] = None, device="cpu") -> Placements:
    """``site_pos``: region name → site position ``[3]`` (world) or ``[n, 3]`` (per environment)."""
    validate_task_against_family(task, family)
    S = len(family.slots)
    pos = torch.empty(n, S, 3, device=device)
    quat = torch.zeros(n, S, 4, device=device)
    quat[..., 0] = 1.0
    for i, s in enumerate(family.slots):
        if s.kind == SLOT_FREE:
            pos[:, i] = torch.tensor(family.park, device=device) + torch.tensor([0.0, 0.3 * i, 0.0], device=device)
        else:
            pos[:, i] = torch.tensor(s.pose, device=device)
            quat[:, i] = torch.tensor([math.cos(0.5 * s.yaw), 0.0, 0.0, math.sin(0.5 * s.yaw)], device=device)
    ok = torch.ones(n, dtype=torch.bool, device=device)
    placed = []  # (slot index, radius, sep)

    def rand(*shape):
        return torch.rand(*shape, generator=generator, device=device)

    for init in order_inits(task, family):
        si = family.slot_index(init.slot)
        slot = family.slots[si]
        radius = slot.h_radius if slot.has_geom else DEFAULT_RADIUS
        sep = init.sep_mm / 1000.0
        if family.init_target_kind(init.region) == INIT_TARGET_REGION:
            r = family.regions[family.region_index(init.region)]
            site = site_pos[r.name].to(device)
            site = site.expand(n, 3) if site.dim() == 1 else site
            rect = r.rect if r.rect is not None else (-0.01, -0.01, 0.01, 0.01)
            lo = torch.tensor(rect[:2], device=device)
            span = torch.tensor([rect[2] - rect[0], rect[3] - rect[1]], device=device)
            xy = site[:, :2] + lo + span * rand(n, 2)
            todo = torch.ones(n, dtype=torch.bool, device=device)
            for _ in range(MAX_REJECTION_ROUNDS):
                clash = torch.zeros(n, dtype=torch.bool, device=device)
                for pj, rj, sj in placed:
                    dmin = max(radius + rj, sep, sj)
                    clash |= torch.linalg.vector_norm(xy - pos[:, pj, :2], dim=-1) < dmin
                todo = clash
                if not bool(todo.any()):
                    break
                fresh = site[:, :2] + lo + span * rand(n, 2)
                xy = torch.where(todo[:, None], fresh, xy)
            ok &= ~todo
            z = site[:, 2] + TABLE_Z_OFFSET - (slot.bottom_z if slot.has_geom else -radius)
            pos[:, si, :2] = xy
            pos[:, si, 2] = z
        else:
            bi = family.slot_index(init.region)
            below = family.slots[bi]
            top = below.top_z if below.has_geom else DEFAULT_RADIUS
            pos[:, si, :2] = pos[:, bi, :2]
            pos[:, si, 2] = pos[:, bi, 2] + top + STACK_Z_OFFSET - (slot.bottom_z if slot.has_geom else -radius)
        if init.yaw:
            yaw = (rand(n) * 2.0 - 1.0) * math.pi
            quat[:, si, 0] = torch.cos(0.5 * yaw)
            quat[:, si, 3] = torch.sin(0.5 * yaw)
        placed.append((si, radius, sep))
    return Placements(pos, quat, ok)


class InitTable:
    """K precomputed placements of one task, resident on the device; ``draw(env_ids)`` gathers fresh ones."""

    def __init__(self, task: TaskSpec, family: FamilySpec, site_pos, k: int = 4096, seed: int = 0, device="cpu"):
        g = torch.Generator(device=device).manual_seed(seed)
        pl = sample_placements(task, family, site_pos, k, g, device)
        keep = pl.ok.nonzero().squeeze(-1)
        if keep.numel() == 0:
            raise RuntimeError(f"tasks: task {task.name!r}: no placement satisfied the separation tests; the regions "
                               f"are too small for the objects")
        self.pos, self.quat = pl.pos[keep].contiguous(), pl.quat[keep].contiguous()
        self.gen = g
        self.rejected = k - int(keep.numel())

    def __len__(self):
        return self.pos.shape[0]

    def draw(self, n: int):
        idx = torch.randint(0, len(self), (n,), generator=self.gen, device=self.pos.device)
        return self.pos[idx], self.quat[idx]
