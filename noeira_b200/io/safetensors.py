"""safetensors reader / writer written from the format definition (8-byte LE header length, JSON
header with dtype / shape / data_offsets, raw little-endian payload).

Validation follows the reference's reader (noeira/io/safetensors.mojo:348): header length within the
file, offsets monotone, non-overlapping, tiling the payload exactly, byte size = prod(shape)·sizeof.
Module-level save/load (noeira/nn/core/safetensors_io.mojo:198,230): names are the dotted walk paths,
tensors are written rank-1 ``[N]`` F32 — parameters then states — with ``__metadata__.producer``;
loading is BY NAME with a ``strict`` switch.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_DT = {"F32": ("<f4", 4), "F64": ("<f8", 8), "F16": ("<f2", 2), "BF16": (None, 2), "U8": ("u1", 1),
       "I32": ("<i4", 4), "I64": ("<i8", 8)}


class SafeTensorsError(RuntimeError):
    pass


class SafeTensorsWriter:
    def __init__(self):
        self.tensors = []  # name, dtype, shape, bytes
        self.metadata: Dict[str, str] = {}

    def add_metadata(self, k: str, v: str):
        self.metadata[k] = str(v)

    def add_f32(self, name, arr, shape=None):
        a = np.ascontiguousarray(arr, dtype="<f4")
        self.tensors.append((name, "F32", list(shape if shape is not None else a.shape), a.tobytes()))

    def add_bf16(self, name, arr_f32, shape=None):
        t = torch.from_numpy(np.ascontiguousarray(arr_f32, dtype=np.float32)).to(torch.bfloat16)
        b = t.view(torch.int16).numpy().astype("<i2").tobytes()
        self.tensors.append((name, "BF16", list(shape if shape is not None else t.shape), b))

    def add_u8(self, name, arr, shape=None):
        a = np.ascontiguousarray(arr, dtype=np.uint8)
        self.tensors.append((name, "U8", list(shape if shape is not None else a.shape), a.tobytes()))

    def write(self, path: str):
        header = {}
        if self.metadata:
            header["__metadata__"] = self.metadata
        off = 0
        for name, dt, shape, b in self.tensors:
            if name in header:
                raise SafeTensorsError(f"duplicate tensor name {name}")
            header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(b)]}
            off += len(b)
        hj = json.dumps(header, separators=(",", ":")).encode()
        hj += b" " * ((8 - len(hj) % 8) % 8)
        tmp = path + ".tmp"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(tmp, "wb") as f:
            f.write(struct.pack("<Q", len(hj)))
            f.write(hj)
            for _, _, _, b in self.tensors:
                mv = memoryview(b)
                for o in range(0, len(mv), 1 << 30):
                    f.write(mv[o:o + (1 << 30)])
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)


class SafeTensors:
    """Reader: every tensor is returned as float32 (F32/F64/F16/BF16) or its integer type."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            hb = f.read(8)
            if len(hb) != 8:
                raise SafeTensorsError("file shorter than the 8-byte header length")
            (hlen,) = struct.unpack("<Q", hb)
            if hlen > size - 8 or hlen > (100 << 20):
                raise SafeTensorsError("header length exceeds file size")
            try:
                self.header = json.loads(f.read(hlen).decode())
            except Exception as e:  # noqa: BLE001
                raise SafeTensorsError(f"header is not valid JSON: {e}")
        self.data_start = 8 + hlen
        self.metadata = self.header.pop("__metadata__", {}) if isinstance(self.header, dict) else {}
        payload = size - self.data_start
        spans = []
        for name, e in self.header.items():
            if e.get("dtype") not in _DT:
                raise SafeTensorsError(f"{name}: unsupported dtype {e.get('dtype')}")
            b, en = e["data_offsets"]
            n = 1
            for s in e["shape"]:
                n *= int(s)
            if b < 0 or en < b or en > payload:
                raise SafeTensorsError(f"{name}: offsets outside the payload")
            if en - b != n * _DT[e["dtype"]][1]:
                raise SafeTensorsError(f"{name}: byte size does not match shape × dtype")
            spans.append((b, en, name))
        spans.sort()
        cur = 0
        for b, en, name in spans:
            if b != cur:
                raise SafeTensorsError(f"{name}: tensors must tile the payload without gaps or overlap")
            cur = en
        if cur != payload:
            raise SafeTensorsError("payload has trailing bytes not covered by any tensor")

    def names(self):
        return list(self.header.keys())

    def shape(self, name):
        return tuple(self.header[name]["shape"])

    def get(self, name: str) -> np.ndarray:
        e = self.header[name]
        b, en = e["data_offsets"]
        with open(self.path, "rb") as f:
            f.seek(self.data_start + b)
            raw = f.read(en - b)
        dt = e["dtype"]
        if dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_DT[dt][0])
            if dt in ("F64", "F16"):
                arr = arr.astype(np.float32)
        return arr.reshape(e["shape"])


def save_safetensors(path: str, named_params: Iterable[Tuple[str, "Param"]], named_states=(), producer="noeira_b200") -> int:
    w = SafeTensorsWriter()
    w.add_metadata("producer", producer)
    n = 0
    for name, p in named_params:
        w.add_f32(name, p.file_view().detach().float().cpu().contiguous().numpy().reshape(-1))
        n += 1
    for name, s in named_states:
        w.add_f32(name, s.data.detach().float().cpu().numpy().reshape(-1))
        n += 1
    w.write(path)
    return n


def load_safetensors(path: str, named_params, named_states=(), strict: bool = True) -> int:
    st = SafeTensors(path)
    have = set(st.names())
    used = 0
    for name, p in named_params:
        if name not in have:
            if strict:
                raise SafeTensorsError(f"missing tensor {name}")
            continue
        a = st.get(name)
        if a.size != p.file_numel:
            raise SafeTensorsError(f"{name}: file has {a.size} values, parameter has {p.file_numel}")
        p.load_file_(torch.from_numpy(np.array(a, dtype=np.float32)).reshape(-1))
        used += 1
    for name, s in named_states:
        if name not in have:
            if strict:
                raise SafeTensorsError(f"missing state {name}")
            continue
        a = st.get(name)
        with torch.no_grad():
            s.data.copy_(torch.from_numpy(np.array(a, dtype=np.float32)).reshape(s.data.shape))
        used += 1
    if strict and used != len(have):
        extra = have - {n for n, _ in named_params} - {n for n, _ in named_states}
        if extra:
            raise SafeTensorsError(f"unexpected tensors in file: {sorted(extra)[:5]}")
    return used
