"""ParamArena: all parameters of one optimizer packed into contiguous fp32 buffers.

``val | grd | m | v`` have identical layout; every parameter starts on a 128-byte boundary
(``PARAM_ALIGN`` = 32 floats, noeira/nn/optimizer/param_arena.mojo:52), so
  * the optimizer is ONE kernel over the arena (noeira/nn/optimizer/adam.mojo:91-128),
  * zero_grad is one fill, the gradient all-reduce needs no per-module hooks — buckets are byte
    ranges of ``grd`` (noeira/nn/distributed/data_parallel.mojo:190-202),
  * a bf16 shadow of ``val`` with the same layout feeds the tensor cores and is rewritten by the
    same kernel that applies the update.
Per-parameter attributes (decay / frozen) are per 32-float row in ``row_flags``.
"""
from __future__ import annotations

from typing import Iterable, List, Tuple

import torch

from .param import Param

PARAM_ALIGN = 32


def _align(n: int, a: int = PARAM_ALIGN) -> int:
    return (n + a - 1) // a * a


class ParamArena:
    def __init__(self, named_params: Iterable[Tuple[str, Param]], device=None, with_moments: bool = True,
                 with_shadow: bool = None, tensor_factory=None):
        """``tensor_factory(numel, dtype)`` lets a caller place the arena in special memory
        (the symmetric heap of ``noeira_b200.parallel`` maps the gradient arena into every peer)."""
        self.entries: List[Tuple[str, Param, int, int]] = []  # name, param, offset, storage numel
        seen = {}
        off = 0
        for name, p in named_params:
            if id(p) in seen:  # tied parameter: one slot
                continue
            seen[id(p)] = name
            n = p.storage_numel
            self.entries.append((name, p, off, n))
            off += _align(n)
        self.numel = off
        first = self.entries[0][1] if self.entries else None
        self.device = torch.device(device) if device is not None else (first.storage.device if first else torch.device("cpu"))
        if with_shadow is None:
            with_shadow = self.device.type == "cuda"
        mk = tensor_factory or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.val = mk(self.numel, torch.float32)
        self.grd = mk(self.numel, torch.float32)
        self.m = mk(self.numel, torch.float32) if with_moments else None
        self.v = mk(self.numel, torch.float32) if with_moments else None
        self.shadow = mk(self.numel, torch.bfloat16) if with_shadow else None
        self.row_flags = torch.zeros(max(self.numel // PARAM_ALIGN, 1), dtype=torch.uint8, device=self.device)
        flags_cpu = torch.zeros(max(self.numel // PARAM_ALIGN, 1), dtype=torch.uint8)
        with torch.no_grad():
            for name, p, o, n in self.entries:
                self.val[o:o + n].copy_(p.storage.reshape(-1))
                if p._grd is not None:
                    self.grd[o:o + n].copy_(p._grd.reshape(-1))
                if p.m is not None and with_moments:
                    self.m[o:o + n].copy_(p.m.reshape(-1))
                    self.v[o:o + n].copy_(p.v.reshape(-1))
                p._val = self.val[o:o + n].view(p.storage_shape)
                p._grd = self.grd[o:o + n].view(p.storage_shape)
                if with_moments:
                    p.m = self.m[o:o + n].view(p.storage_shape)
                    p.v = self.v[o:o + n].view(p.storage_shape)
                if self.shadow is not None:
                    p._shadow = self.shadow[o:o + n].view(p.storage_shape)
                    p._shadow_version = -1
                p.arena = self
                p.arena_offset = o
                fl = (1 if p.decay else 0) | (2 if p.frozen else 0)
                flags_cpu[o // PARAM_ALIGN:(o + _align(n)) // PARAM_ALIGN] = fl
        self.row_flags.copy_(flags_cpu)
        if self.shadow is not None:
            self.refresh_shadow()

    def repad(self, total: int):
        """Re-allocate ``val`` / ``grd`` (and the shadow) with ``total >= numel`` elements and re-point every parameter's
        views: sharding strategies need the arena to be a whole number of equal shards so that reduce-scatter and
        all-gather run in place.  The tail is zero and belongs to no parameter."""
        if total < self.numel:
            raise ValueError("an arena cannot shrink")
        if total == self.val.numel():
            return
        with torch.no_grad():
            for attr in ("val", "grd", "shadow"):
                old = getattr(self, attr)
                if old is None:
                    continue
                new = torch.zeros(total, dtype=old.dtype, device=old.device)
                new[: old.numel()].copy_(old)
                setattr(self, attr, new)
            for _, p, o, n in self.entries:
                p._val = self.val[o:o + n].view(p.storage_shape)
                p._grd = self.grd[o:o + n].view(p.storage_shape)
                if self.shadow is not None:
                    p._shadow = self.shadow[o:o + n].view(p.storage_shape)

    def release_moments(self):
        """Drop the full-size Adam moments (a sharding strategy keeps its own shard-size copies)."""
        self.m = self.v = None
        for _, p, _, _ in self.entries:
            p.m = p.v = None

    def refresh_shadow(self):
        self.shadow.copy_(self.val[: self.shadow.numel()])
        for _, p, _, _ in self.entries:
            p.mark_shadow_fresh()

    def refresh_flags(self):
        flags_cpu = torch.zeros(self.row_flags.numel(), dtype=torch.uint8)
        for name, p, o, n in self.entries:
            fl = (1 if p.decay else 0) | (2 if p.frozen else 0)
            flags_cpu[o // PARAM_ALIGN:(o + _align(n)) // PARAM_ALIGN] = fl
        self.row_flags.copy_(flags_cpu)

    def zero_grad(self):
        self.grd.zero_()

    def layout(self):
        """(name, element offset, element count) of every parameter, in arena order."""
        return [(name, o, n) for name, _, o, n in self.entries]

    def bump_versions(self, shadow_fresh: bool):
        for _, p, _, _ in self.entries:
            p.version += 1
            if shadow_fresh:
                p.mark_shadow_fresh()

    def byte_range(self, name: str) -> Tuple[int, int]:
        for n, p, o, k in self.entries:
            if n == name:
                return 4 * o, 4 * (o + _align(k))
        raise KeyError(name)

    def state_bytes(self) -> int:
        per = 4 * (2 + (2 if self.m is not None else 0)) + (2 if self.shadow is not None else 0)
        return per * self.numel
