"""Parameters and non-trainable states.

A ``Param`` owns (or, after ``ParamArena.adopt``, views) four fp32 buffers — value, gradient and the
two Adam moments — plus an optional bf16 *shadow* of the value that the tensor-core kernels read.
Reference: ``Param[NAME, APPLY_DECAY, SIZE]`` noeira/nn/core/param.mojo:254 (val, grd, lazy m, v;
frozen = no gradient, :296-318) and ``State`` noeira/nn/core/state.mojo:52.

Storage may be wider than the logical shape: a 2-D parameter ``[R, C]`` is stored with its row pitch
rounded up to 8 elements so that a bf16 row is a multiple of 16 bytes (TMA requirement); the pad
columns are zero and receive zero gradients.  Checkpoints always hold the logical shape.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class Param:
    def __init__(self, name: str, shape: Sequence[int], decay: bool = True, device="cpu", pad_rows: bool = True):
        self.name = name
        self.shape = tuple(int(s) for s in shape)
        self.decay = bool(decay)
        self.frozen = False
        self.version = 0
        if len(self.shape) == 2 and pad_rows:
            self.storage_shape = (self.shape[0], _pad8(self.shape[1]))
        elif len(self.shape) == 1 and pad_rows:
            self.storage_shape = (_pad8(self.shape[0]),)
        else:
            self.storage_shape = self.shape
        self._val = torch.zeros(self.storage_shape, dtype=torch.float32, device=device)
        self._grd: Optional[torch.Tensor] = None
        self._shadow: Optional[torch.Tensor] = None
        self.m: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        # optional layout hooks: files hold `to_file(data)`; `from_file(tensor)` maps back (e.g. conv weights)
        self.to_file = None
        self.from_file = None

    # ---- storage (padded) views
    @property
    def storage(self) -> torch.Tensor:
        return self._val

    @property
    def grad_storage(self) -> torch.Tensor:
        if self._grd is None:
            self._grd = torch.zeros_like(self._val)
        return self._grd

    @property
    def shadow(self) -> torch.Tensor:
        """bf16 copy of the padded storage; refreshed by the optimizer (or lazily when stale)."""
        if self._shadow is None:
            self._shadow = self._val.to(torch.bfloat16)
            self._shadow_version = self.version
        elif getattr(self, "_shadow_version", -1) != self.version:
            self._shadow.copy_(self._val)
            self._shadow_version = self.version
        return self._shadow

    def mark_shadow_fresh(self):
        self._shadow_version = self.version

    # ---- logical views
    def _logical(self, t: torch.Tensor) -> torch.Tensor:
        if self.storage_shape == self.shape:
            return t
        if len(self.shape) == 2:
            return t[:, : self.shape[1]]
        return t[: self.shape[0]]

    @property
    def data(self) -> torch.Tensor:
        return self._logical(self._val)

    @property
    def grad(self) -> torch.Tensor:
        return self._logical(self.grad_storage)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def storage_numel(self) -> int:
        return self._val.numel()

    @property
    def file_numel(self) -> int:
        """Element count of the parameter as files hold it (``to_file`` may strip kernel-side padding, e.g. the
        zero input channels of a 3-channel convolution stem)."""
        if self.to_file is None:
            return self.numel
        if getattr(self, "_file_numel", None) is None:
            self._file_numel = int(self.file_view().numel())
        return self._file_numel

    def file_view(self, t: Optional[torch.Tensor] = None) -> torch.Tensor:
        t = self.data if t is None else t
        return self.to_file(t) if self.to_file is not None else t

    def load_file_(self, flat: torch.Tensor):
        self.set_(self.from_file(flat) if self.from_file is not None else flat)

    def set_(self, value: torch.Tensor):
        with torch.no_grad():
            self.data.copy_(value.reshape(self.shape).to(self._val.device, torch.float32))
        self.version += 1

    def zero_grad(self):
        if self._grd is not None:
            self._grd.zero_()

    def to(self, device):
        self._val = self._val.to(device)
        if self._grd is not None:
            self._grd = self._grd.to(device)
        if self.m is not None:
            self.m, self.v = self.m.to(device), self.v.to(device)
        self._shadow = None
        return self


class State:
    """Persisted, never optimized (e.g. BatchNorm running statistics)."""

    def __init__(self, name: str, shape: Sequence[int], device="cpu", fill: float = 0.0):
        self.name = name
        self.shape = tuple(shape)
        self.data = torch.full(self.shape, fill, dtype=torch.float32, device=device)

    def to(self, device):
        self.data = self.data.to(device)
        return self
