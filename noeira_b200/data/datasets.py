"""Dataset readers and the episodic trajectory store.

``load_mnist_idx`` (IDX files, optionally gzip'ed — inflated by the native zlib binding), ``load_cifar10_bin`` (the binary
batches: 1 label byte + 3072 pixel bytes per record), ``CharCorpus`` (character-level tokenizer + resident token stream
for ``AutoregressiveTrainer``).  ``TrajectoryStore`` / ``TrajectoryWriter``: episodes of fixed-width float32 steps in one
binary file with a JSON index, read back whole, by episode, or streamed as shuffled step batches by the native
prefetching loader.  (Reference: noeira/nn/datasets/{mnist,cifar10,tiny_shakespeare}.mojo; noeira/data/store.mojo:99,387
``TrajectoryStore(Writer)`` over HDF5 — no HDF5 library in this image, the container format here is the store's own.)
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional

import numpy as np

from ..runtime import RecordLoader, gzip_inflate, write_file_atomic


def _read_maybe_gz(path: str) -> bytes:
    raw = open(path, "rb").read()
    return gzip_inflate(raw) if raw[:2] == b"\x1f\x8b" else raw


def load_mnist_idx(images_path: str, labels_path: str):
    """→ (uint8 [N, 28, 28], uint8 [N])"""
    im, lb = _read_maybe_gz(images_path), _read_maybe_gz(labels_path)
    magic, n, h, w = struct.unpack(">IIII", im[:16])
    if magic != 2051:
        raise ValueError("bad IDX image magic")
    magic2, n2 = struct.unpack(">II", lb[:8])
    if magic2 != 2049 or n2 != n:
        raise ValueError("bad IDX label file")
    return np.frombuffer(im, np.uint8, offset=16).reshape(n, h, w).copy(), np.frombuffer(lb, np.uint8, offset=8).copy()


def load_cifar10_bin(paths: List[str]):
    """→ (uint8 [N, 3, 32, 32], uint8 [N])"""
    xs, ys = [], []
    for p in paths:
        rec = np.frombuffer(open(p, "rb").read(), np.uint8).reshape(-1, 3073)
        ys.append(rec[:, 0].copy())
        xs.append(rec[:, 1:].reshape(-1, 3, 32, 32).copy())
    return np.concatenate(xs), np.concatenate(ys)


class CharCorpus:
    def __init__(self, text: str):
        self.chars = sorted(set(text))
        self.stoi = {c: i for i, c in enumerate(self.chars)}
        self.tokens = np.array([self.stoi[c] for c in text], np.int64)

    @property
    def vocab(self) -> int:
        return len(self.chars)

    def encode(self, s: str) -> np.ndarray:
        return np.array([self.stoi[c] for c in s], np.int64)

    def decode(self, ids) -> str:
        return "".join(self.chars[int(i)] for i in ids)

    @classmethod
    def from_file(cls, path: str):
        return cls(open(path, encoding="utf-8").read())


# ------------------------------------------------------------------------------------------ trajectory store
MAGIC = b"NBTRAJ01"


class TrajectoryWriter:
    """Appends episodes; ``close`` writes data and index atomically.  A step is the concatenation of its fields."""

    def __init__(self, path: str, fields: Dict[str, int], meta: Optional[dict] = None):
        self.path, self.fields, self.meta = path, dict(fields), dict(meta or {})
        self.width = sum(fields.values())
        self.episodes: List[np.ndarray] = []

    def add_episode(self, **arrays):
        T = len(next(iter(arrays.values())))
        cols = []
        for name, w in self.fields.items():
            a = np.asarray(arrays[name], np.float32).reshape(T, w)
            cols.append(a)
        self.episodes.append(np.concatenate(cols, 1))

    def close(self):
        lengths = [len(e) for e in self.episodes]
        index = json.dumps({"fields": self.fields, "lengths": lengths, "meta": self.meta}).encode()
        header = MAGIC + struct.pack("<QQ", len(index), self.width) + index
        pad = (-len(header)) % 64
        write_file_atomic(self.path, [header + b"\0" * pad] + [e.reshape(-1) for e in self.episodes])


class TrajectoryStore:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(24)
            if head[:8] != MAGIC:
                raise ValueError("not a trajectory store")
            n_index, self.width = struct.unpack("<QQ", head[8:24])
            idx = json.loads(f.read(n_index))
        self.fields: Dict[str, int] = idx["fields"]
        self.lengths: List[int] = idx["lengths"]
        self.meta = idx["meta"]
        self.header_bytes = (24 + n_index + 63) // 64 * 64
        self.offsets = np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int64)
        self.n_steps = int(self.offsets[-1])

    def _split(self, block: np.ndarray) -> Dict[str, np.ndarray]:
        out, c = {}, 0
        for name, w in self.fields.items():
            out[name] = block[:, c: c + w]
            c += w
        return out

    def episode(self, i: int) -> Dict[str, np.ndarray]:
        a = np.fromfile(self.path, np.float32, count=self.lengths[i] * self.width,
                        offset=self.header_bytes + int(self.offsets[i]) * self.width * 4)
        return self._split(a.reshape(-1, self.width))

    def all_steps(self) -> Dict[str, np.ndarray]:
        a = np.fromfile(self.path, np.float32, count=self.n_steps * self.width, offset=self.header_bytes)
        return self._split(a.reshape(-1, self.width))

    def loader(self, batch: int, seed: int = 0, shuffle: bool = True, threads: int = 2) -> "StepBatches":
        return StepBatches(self, batch, seed, shuffle, threads)


class StepBatches:
    """Shuffled step batches through the native prefetching loader; iterate one epoch at a time."""

    def __init__(self, store: TrajectoryStore, batch: int, seed: int, shuffle: bool, threads: int):
        self.store, self.batch = store, batch
        self.loader = RecordLoader(store.path, store.width * 4, store.n_steps, batch, header_bytes=store.header_bytes,
                                   threads=threads, seed=seed, shuffle=shuffle, drop_last=True)
        self.buf = np.zeros((batch, store.width), np.float32)
        self.epoch = 0

    def __iter__(self):
        self.loader.reset(self.epoch)
        self.epoch += 1
        while True:
            n, idx = self.loader.next_into(self.buf)
            if n == 0:
                return
            yield self.store._split(self.buf[:n].copy()), idx

    def close(self):
        self.loader.close()
