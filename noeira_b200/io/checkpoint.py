"""v3 binary checkpoints — same on-disk layout as the reference (noeira/nn/core/checkpoint.mojo:1-40):

    storage-ckpt v3\\n
    P <dotted-name> <size> <has_moments:0|1>\\n  <size·4 bytes fp32 LE>[<m bytes><v bytes>]
    S <dotted-name> <size>\\n                    <size·4 bytes fp32 LE>
    K <name>\\n                                  <8 bytes float64 LE>      (after every P/S section)

Rules kept from the reference: sections follow the module walk order and the loader VALIDATES every
name and size against the in-memory walk (topology drift raises); files are written to ``path.tmp``
in ≤1 GiB chunks and renamed atomically; device tensors are staged to the host in ≤64 MB pieces;
``K`` values are raw float64 (a counter stored as fp32 stops at 2^24).  Parameters are written in
their LOGICAL shape (row padding used by the kernels is stripped), so files are interchangeable with
the reference's.  ``Linear.weight`` is ``[IN, OUT]`` row-major.
"""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

HEADER = b"storage-ckpt v3\n"
_WRITE_CHUNK = 1 << 30
_STAGE_ELEMS = 1 << 24


class CheckpointError(RuntimeError):
    pass


def _to_host_f32(t: torch.Tensor) -> np.ndarray:
    t = t.detach()
    if t.device.type == "cpu":
        return t.contiguous().to(torch.float32).numpy().reshape(-1)
    flat = t.contiguous().reshape(-1).to(torch.float32)
    out = np.empty(flat.numel(), np.float32)
    for o in range(0, flat.numel(), _STAGE_ELEMS):
        out[o:o + _STAGE_ELEMS] = flat[o:o + _STAGE_ELEMS].cpu().numpy()
    return out


def _write_chunked(f, b: bytes):
    mv = memoryview(b)
    for o in range(0, len(mv), _WRITE_CHUNK):
        f.write(mv[o:o + _WRITE_CHUNK])


def _check_name(name: str):
    if not name or " " in name or "\n" in name:
        raise CheckpointError(f"invalid section name {name!r}")


def _write_groups(path: str, groups, scalars: Dict[str, float], with_moments: bool) -> None:
    """``groups`` = [(named_params, named_states), ...]: for every group its P sections, then its S sections (the
    reference walks one model at a time, noeira/nn/core/checkpoint.mojo:804-827); the K scalars come once, last."""
    tmp = path + ".tmp"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(tmp, "wb") as f:
        f.write(HEADER)
        for named_params, named_states in groups:
            for name, p in named_params:
                _check_name(name)
                has_m = 1 if (with_moments and p.m is not None) else 0
                f.write(f"P {name} {p.file_numel} {has_m}\n".encode())
                _write_chunked(f, _to_host_f32(p.file_view()).tobytes())
                if has_m:
                    _write_chunked(f, _to_host_f32(p.file_view(p._logical(p.m))).tobytes())
                    _write_chunked(f, _to_host_f32(p.file_view(p._logical(p.v))).tobytes())
            for name, s in named_states:
                _check_name(name)
                f.write(f"S {name} {s.data.numel()}\n".encode())
                _write_chunked(f, _to_host_f32(s.data).tobytes())
        for k, v in (scalars or {}).items():
            _check_name(k)
            f.write(f"K {k}\n".encode())
            f.write(struct.pack("<d", float(v)))
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def save_checkpoint(path: str, named_params: Iterable[Tuple[str, "Param"]], named_states: Iterable[Tuple[str, "State"]],
                    scalars: Dict[str, float] = None, with_moments: bool = True) -> None:
    _write_groups(path, [(list(named_params), list(named_states))], scalars, with_moments)


class _Reader:
    def __init__(self, path):
        self.f = open(path, "rb")
        self.size = os.path.getsize(path)
        head = self.f.read(len(HEADER))
        if head != HEADER:
            raise CheckpointError(f"{path}: not a storage-ckpt v3 file")

    def line(self):
        b = bytearray()
        while True:
            c = self.f.read(1)
            if not c:
                return None if not b else b.decode()
            if c == b"\n":
                return b.decode()
            b += c

    def payload(self, n_elems: int) -> np.ndarray:
        need = 4 * n_elems
        out = bytearray()
        while len(out) < need:
            chunk = self.f.read(min(_WRITE_CHUNK, need - len(out)))
            if not chunk:
                raise CheckpointError("truncated checkpoint payload")
            out += chunk
        return np.frombuffer(bytes(out), dtype="<f4")


def _read_groups(path: str, groups, load_moments: bool) -> Dict[str, float]:
    r = _Reader(path)
    for named_params, named_states in groups:
        for name, p in named_params:
            ln = r.line()
            if ln is None:
                raise CheckpointError(f"checkpoint ends before parameter {name}")
            parts = ln.split(" ")
            if len(parts) != 4 or parts[0] != "P":
                raise CheckpointError(f"expected 'P {name} ...', found {ln!r}")
            if parts[1] != name or int(parts[2]) != p.file_numel:
                raise CheckpointError(f"section mismatch: file has {parts[1]}[{parts[2]}], model walk expects {name}[{p.file_numel}]")
            vals = r.payload(p.file_numel)
            p.load_file_(torch.from_numpy(vals.copy()))
            if int(parts[3]):
                m, v = r.payload(p.file_numel), r.payload(p.file_numel)
                if load_moments and p.m is not None:
                    with torch.no_grad():
                        fm = (lambda t: p.from_file(t)) if p.from_file is not None else (lambda t: t)
                        p._logical(p.m).copy_(fm(torch.from_numpy(m.copy())).reshape(p.shape))
                        p._logical(p.v).copy_(fm(torch.from_numpy(v.copy())).reshape(p.shape))
        for name, s in named_states:
            ln = r.line()
            parts = (ln or "").split(" ")
            if len(parts) != 3 or parts[0] != "S" or parts[1] != name or int(parts[2]) != s.data.numel():
                raise CheckpointError(f"state section mismatch at {name}: {ln!r}")
            with torch.no_grad():
                s.data.copy_(torch.from_numpy(r.payload(s.data.numel()).copy()).reshape(s.data.shape))
    scalars: Dict[str, float] = {}
    while True:
        ln = r.line()
        if ln is None:
            break
        parts = ln.split(" ")
        if len(parts) != 2 or parts[0] != "K":
            raise CheckpointError(f"unexpected trailing section {ln!r}")
        b = r.f.read(8)
        if len(b) != 8:
            raise CheckpointError("truncated scalar section")
        scalars[parts[1]] = struct.unpack("<d", b)[0]
    return scalars


def load_checkpoint(path: str, named_params: Iterable[Tuple[str, "Param"]], named_states: Iterable[Tuple[str, "State"]],
                    load_moments: bool = True) -> Dict[str, float]:
    return _read_groups(path, [(list(named_params), list(named_states))], load_moments)


def save_params_multi(path: str, modules: List, scalars=None, with_moments=True):
    """Several networks in pack order in one file WITHOUT prefixes (the SAC layout: actor, critic 1, critic 2):
    module by module, the P sections of a module followed by its S sections
    (noeira/nn/core/checkpoint.mojo:804-827)."""
    _write_groups(path, [(list(m.named_params()), list(m.named_states())) for m in modules], scalars, with_moments)


def load_params_multi(path: str, modules: List, load_moments=True):
    return _read_groups(path, [(list(m.named_params()), list(m.named_states())) for m in modules], load_moments)
