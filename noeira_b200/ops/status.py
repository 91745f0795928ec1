"""Device status words written by bounded waits inside kernels (see csrc/common.cuh).

Each device has one ``int32[4]`` tensor: [code, where, block, extra].  Kernels record the first
failure with an atomic compare-and-swap and then unwind normally, so the CUDA context stays usable;
``check_status`` is the host side read (it synchronises — call it at logging cadence, not per launch).
"""
from __future__ import annotations

import torch

_STATUS = {}
_CODES = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bounds check failed",
          4: "non-finite value"}


class DeviceStatusError(RuntimeError):
    def __init__(self, code, where, block, extra):
        super().__init__(f"kernel reported '{_CODES.get(code, code)}' at site {where}, block {block}, extra {extra}")
        self.code, self.where, self.block, self.extra = code, where, block, extra


def device_status(device=None) -> torch.Tensor:
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[key] = t
        from .._native import register_bounds_status
        register_bounds_status(t)          # bounds-checked build: failed index tests are reported through this word
    return t


def check_status(device=None, clear: bool = True) -> None:
    t = device_status(device)
    code, where, block, extra = (int(x) for x in t.cpu())
    if code != 0:
        if clear:
            t.zero_()
        raise DeviceStatusError(code, where, block, extra)
