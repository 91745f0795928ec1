"""Name / layout maps between this framework's parameters and PyTorch-named safetensors files.

``TorchNameMap`` is one architecture's table of (our dotted name, their name, layout kind, THEIR shape):
  TN_PLAIN      same numbers, same order — a rename only
  TN_TRANSPOSE  their ``[R, C]`` is our ``[C, R]`` (``torch.nn.Linear.weight`` is ``[out, in]``, ours is ``[in, out]``)
  TN_ZEROS      ours exists, theirs does not: zero on load, skipped on save
``load_torch_named`` fills the parameters (and states) of a subtree from a file and keeps five lists, because the ways
this goes wrong differ: ``loaded``, ``zeroed``, ``missing`` (the map names a tensor the file lacks), ``unmapped`` (the
model has a parameter under the prefix that the map does not mention) and ``unclaimed`` (file tensors no map entry
names: coverage of the model is not coverage of the file).  Shapes are checked, not only element counts: a ``[512,
256]`` and a ``[256, 512]`` hold the same number of floats.
Reference: noeira/nn/core/torch_names.mojo:50-330 (TorchNameMap, LoadTorchNamed, SaveTorchNamed).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import numpy as np
import torch

from ..io.safetensors import SafeTensors, SafeTensorsWriter

TN_PLAIN, TN_TRANSPOSE, TN_ZEROS = 0, 1, 2


class TorchNameError(RuntimeError):
    pass


class TorchNameMap:
    def __init__(self):
        self.ours: List[str] = []
        self.theirs: List[str] = []
        self.kind: List[int] = []
        self.shapes: List[Tuple[int, ...]] = []
        self._index: Dict[str, int] = {}

    def __len__(self):
        return len(self.ours)

    def add(self, ours: str, theirs: str, shape: Sequence[int], kind: int = TN_PLAIN):
        """``shape`` is THEIR shape — the one that goes in the file."""
        if ours in self._index:
            raise TorchNameError(f"TorchNameMap: '{ours}' mapped twice (to '{self.theirs[self._index[ours]]}' and '{theirs}')")
        if kind == TN_TRANSPOSE and len(shape) != 2:
            raise TorchNameError(f"TorchNameMap: '{ours}' is marked TN_TRANSPOSE but its shape has rank {len(shape)}")
        self._index[ours] = len(self.ours)
        self.ours.append(ours)
        self.theirs.append(theirs)
        self.kind.append(kind)
        self.shapes.append(tuple(int(s) for s in shape))
        return self

    def add_linear(self, ours: str, theirs: str, out_features: int, in_features: int):
        """A ``torch.nn.Linear`` weight: theirs ``[out, in]``, ours ``[in, out]``."""
        return self.add(ours, theirs, (out_features, in_features), TN_TRANSPOSE)

    def add_zeros(self, ours: str, shape: Sequence[int] = ()):
        return self.add(ours, "", shape, TN_ZEROS)

    def index_of_ours(self, name: str) -> int:
        return self._index.get(name, -1)

    def numel(self, i: int) -> int:
        return int(np.prod(self.shapes[i])) if self.shapes[i] else 1


class TorchLoadReport:
    def __init__(self, prefix: str):
        self.prefix = prefix
        self.loaded: List[str] = []
        self.zeroed: List[str] = []
        self.missing: List[str] = []
        self.unmapped: List[str] = []
        self.unclaimed: List[str] = []
        self.skipped = 0

    def check(self, what: str = "load_torch_named", allow_unclaimed: bool = True):
        """Raise unless every mapped tensor under the prefix was filled."""
        if self.unmapped:
            raise TorchNameError(f"{what}: {len(self.unmapped)} parameter(s) under '{self.prefix}' are not in the name map, first "
                                 f"'{self.unmapped[0]}' - the model's topology and the map have drifted apart")
        if self.missing:
            raise TorchNameError(f"{what}: {len(self.missing)} tensor(s) named by the map are absent from the file, first "
                                 f"'{self.missing[0]}' - the file is a different variant of this architecture")
        if not self.loaded:
            raise TorchNameError(f"{what}: matched NOTHING under '{self.prefix}' - the prefix and the walk have drifted apart")
        if self.unclaimed and not allow_unclaimed:
            raise TorchNameError(f"{what}: {len(self.unclaimed)} file tensor(s) are named by no map entry, first '{self.unclaimed[0]}'")


def load_torch_named(file, name_map: TorchNameMap, named_params: Iterable[Tuple[str, object]], named_states=(), prefix: str = "",
                     their_prefix: str = "") -> TorchLoadReport:
    """Fill every parameter / state whose dotted name starts with ``prefix`` from ``file`` (a path or an open
    ``SafeTensors``) through ``name_map`` (keys are names RELATIVE to the prefix; ``their_prefix`` is prepended to the
    file names)."""
    st = file if isinstance(file, SafeTensors) else SafeTensors(file)
    rep = TorchLoadReport(prefix)
    have = set(st.names())
    claimed = set()
    for name, obj in list(named_params) + list(named_states):
        if not name.startswith(prefix):
            rep.skipped += 1
            continue
        local = name[len(prefix):]
        i = name_map.index_of_ours(local)
        if i < 0:
            rep.unmapped.append(local)
            continue
        is_param = hasattr(obj, "load_file_")
        shape = tuple(obj.shape)
        n = int(np.prod(shape)) if shape else 1
        if name_map.kind[i] == TN_ZEROS:
            z = torch.zeros(n)
            obj.set_(z.reshape(shape)) if is_param else obj.data.zero_()
            rep.zeroed.append(local)
            continue
        key = their_prefix + name_map.theirs[i]
        if key not in have:
            rep.missing.append(key)
            continue
        claimed.add(key)
        got, want = tuple(st.shape(key)), name_map.shapes[i]
        if got != want:
            raise TorchNameError(f"load_torch_named: '{key}' has shape {list(got)} but the map declares {list(want)}")
        vals = torch.from_numpy(np.asarray(st.get(key), dtype=np.float32).copy()).reshape(want)
        if name_map.kind[i] == TN_TRANSPOSE:
            vals = vals.t().contiguous()
        if vals.numel() != n:
            raise TorchNameError(f"load_torch_named: '{key}' holds {vals.numel()} values, '{local}' needs {n}")
        if is_param:
            obj.set_(vals.reshape(shape))
        else:
            with torch.no_grad():
                obj.data.copy_(vals.reshape(obj.data.shape))
        rep.loaded.append(local)
    rep.unclaimed = sorted(k for k in have if k.startswith(their_prefix) and k not in claimed)
    return rep


def save_torch_named(path: str, name_map: TorchNameMap, named_params, named_states=(), prefix: str = "", their_prefix: str = "",
                     dtype: str = "f32") -> int:
    """Write the subtree under ``prefix`` with THEIR names and layouts (the inverse of ``load_torch_named``)."""
    w = SafeTensorsWriter()
    w.add_metadata("producer", "noeira_b200")
    n_written = 0
    for name, obj in list(named_params) + list(named_states):
        if not name.startswith(prefix):
            continue
        i = name_map.index_of_ours(name[len(prefix):])
        if i < 0:
            raise TorchNameError(f"save_torch_named: '{name}' is not in the name map")
        if name_map.kind[i] == TN_ZEROS:
            continue
        t = obj.data.detach().float().cpu()
        if name_map.kind[i] == TN_TRANSPOSE:
            t = t.t()
        arr = np.ascontiguousarray(t.numpy()).reshape(name_map.shapes[i])
        (w.add_bf16 if dtype == "bf16" else w.add_f32)(their_prefix + name_map.theirs[i], arr, list(name_map.shapes[i]))
        n_written += 1
    w.write(path)
    return n_written


def mlp_name_map(dims: Sequence[int], ours_fmt: str = "{i}.", theirs_fmt: str = "{j}.", stride: int = 2) -> TorchNameMap:
    """Map of a ``Sequential`` of Linear(+activation) layers onto a ``torch.nn.Sequential`` whose Linear modules sit at
    indices 0, ``stride``, 2·``stride``, … (activation modules in between)."""
    m = TorchNameMap()
    for i in range(len(dims) - 1):
        m.add_linear(ours_fmt.format(i=i) + "weight", theirs_fmt.format(j=i * stride) + "weight", dims[i + 1], dims[i])
        m.add(ours_fmt.format(i=i) + "bias", theirs_fmt.format(j=i * stride) + "bias", (dims[i + 1],))
    return m
