"""ctypes bindings of ``libnoeira_b200_host.so`` (C ABI in ``csrc/host/host_api.h``)."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import numpy as np

from .._native import host_lib

_c = ctypes
_configured = False


def _lib():
    global _configured
    L = host_lib()
    if not _configured:
        L.nbh_ring_create.restype = _c.c_void_p
        L.nbh_ring_create.argtypes = [_c.c_size_t]
        L.nbh_ring_destroy.argtypes = [_c.c_void_p]
        L.nbh_ring_push.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_uint32]
        L.nbh_ring_pop.restype = _c.c_int64
        L.nbh_ring_pop.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_uint32]
        L.nbh_ring_used.restype = _c.c_size_t
        L.nbh_ring_used.argtypes = [_c.c_void_p]
        L.nbh_filesink_start.restype = _c.c_void_p
        L.nbh_filesink_start.argtypes = [_c.c_void_p, _c.c_char_p]
        L.nbh_filesink_stop.argtypes = [_c.c_void_p]
        L.nbh_serial_open.argtypes = [_c.c_char_p, _c.c_int]
        L.nbh_serial_write.restype = _c.c_int64
        L.nbh_serial_write.argtypes = [_c.c_int, _c.c_void_p, _c.c_size_t]
        L.nbh_serial_read.restype = _c.c_int64
        L.nbh_serial_read.argtypes = [_c.c_int, _c.c_void_p, _c.c_size_t, _c.c_int]
        L.nbh_http_request.argtypes = [_c.c_char_p, _c.c_char_p, _c.c_char_p, _c.c_void_p, _c.c_size_t, _c.c_int,
                                       _c.POINTER(_c.c_void_p), _c.POINTER(_c.c_size_t)]
        L.nbh_gzip_inflate.restype = _c.c_int64
        L.nbh_gzip_inflate.argtypes = [_c.c_void_p, _c.c_size_t, _c.POINTER(_c.c_void_p), _c.POINTER(_c.c_size_t)]
        L.nbh_free.argtypes = [_c.c_void_p]
        L.nbh_convex_hull.argtypes = [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int]
        L.nbh_write_file_atomic.argtypes = [_c.c_char_p, _c.c_void_p, _c.c_void_p, _c.c_int]
        L.nbh_read_file_range.restype = _c.c_int64
        L.nbh_read_file_range.argtypes = [_c.c_char_p, _c.c_uint64, _c.c_void_p, _c.c_size_t]
        L.nbh_sha256.argtypes = [_c.c_void_p, _c.c_size_t, _c.c_void_p]
        L.nbh_loader_create.restype = _c.c_void_p
        L.nbh_loader_create.argtypes = [_c.c_char_p, _c.c_uint64, _c.c_uint64, _c.c_uint64, _c.c_uint32, _c.c_uint32,
                                        _c.c_uint32, _c.c_uint64, _c.c_int, _c.c_int]
        L.nbh_loader_next.restype = _c.c_int64
        L.nbh_loader_next.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_void_p]
        L.nbh_loader_reset.argtypes = [_c.c_void_p, _c.c_uint64]
        L.nbh_loader_destroy.argtypes = [_c.c_void_p]
        _configured = True
    return L


def _err(rc, what):
    if rc < 0:
        raise OSError(-rc, f"{what}: {os.strerror(-rc)}")
    return rc


class SpscRing:
    """Single-producer / single-consumer ring of byte messages (one thread pushes, one pops)."""

    def __init__(self, capacity_bytes: int = 1 << 20):
        self._h = _lib().nbh_ring_create(capacity_bytes)
        if not self._h:
            raise MemoryError("ring")
        self._buf = ctypes.create_string_buffer(1 << 16)

    def push(self, data: bytes) -> bool:
        rc = _lib().nbh_ring_push(self._h, data, len(data))
        if rc == -11:  # EAGAIN
            return False
        _err(rc, "ring_push")
        return True

    def pop(self) -> Optional[bytes]:
        n = _lib().nbh_ring_pop(self._h, self._buf, len(self._buf))
        if n == -11:
            return None
        if n == -90:  # EMSGSIZE
            self._buf = ctypes.create_string_buffer(len(self._buf) * 4)
            return self.pop()
        _err(n, "ring_pop")
        return self._buf.raw[:n]

    def used(self) -> int:
        return _lib().nbh_ring_used(self._h)

    def close(self):
        if self._h:
            _lib().nbh_ring_destroy(self._h)
            self._h = None


class FileSink:
    """Background thread that appends every message pushed into ``ring`` to ``path`` (loggers write through this
    so that the training loop never blocks on the file system)."""

    def __init__(self, path: str, capacity_bytes: int = 1 << 20):
        self.ring = SpscRing(capacity_bytes)
        self._h = _lib().nbh_filesink_start(self.ring._h, os.fsencode(path))
        if not self._h:
            raise OSError(f"cannot open {path}")

    def write(self, data: bytes):
        import time
        while not self.ring.push(data):
            time.sleep(0.0005)

    def close(self) -> int:
        n = _lib().nbh_filesink_stop(self._h)
        self._h = None
        self.ring.close()
        return n


class SerialPort:
    def __init__(self, path: str = None, baud: int = 1000000, fd: int = None):
        if fd is not None:
            _err(_lib().nbh_serial_configure(fd, baud), "serial_configure")
            self.fd = fd
        else:
            self.fd = _err(_lib().nbh_serial_open(os.fsencode(path), baud), f"serial_open {path}")

    def write(self, data: bytes) -> int:
        return _err(_lib().nbh_serial_write(self.fd, data, len(data)), "serial_write")

    def read(self, n: int, timeout_ms: int = 100) -> bytes:
        buf = ctypes.create_string_buffer(n)
        got = _err(_lib().nbh_serial_read(self.fd, buf, n, timeout_ms), "serial_read")
        return buf.raw[:got]

    def flush(self):
        _err(_lib().nbh_serial_flush(self.fd), "serial_flush")

    def close(self):
        _lib().nbh_serial_close(self.fd)


def http_request(method: str, url: str, headers: dict = None, body: bytes = b"", timeout_ms: int = 10000):
    """→ (status, body bytes); chunked transfer and gzip content encoding are decoded natively."""
    hs = "".join(f"{k}: {v}\r\n" for k, v in (headers or {}).items()).encode() or None
    out, n = _c.c_void_p(), _c.c_size_t()
    st = _err(_lib().nbh_http_request(method.encode(), url.encode(), hs, body, len(body), timeout_ms, _c.byref(out),
                                      _c.byref(n)), f"http {method} {url}")
    data = ctypes.string_at(out, n.value)
    _lib().nbh_free(out)
    return st, data


def gzip_inflate(data: bytes) -> bytes:
    out, n = _c.c_void_p(), _c.c_size_t()
    _err(_lib().nbh_gzip_inflate(data, len(data), _c.byref(out), _c.byref(n)), "gzip_inflate")
    res = ctypes.string_at(out, n.value)
    _lib().nbh_free(out)
    return res


def convex_hull(points) -> np.ndarray:
    """points [n, 3] → int32 [t, 3] outward-facing triangles."""
    p = np.ascontiguousarray(points, dtype=np.float64)
    cap = max(4 * len(p), 16)
    tri = np.zeros((cap, 3), dtype=np.int32)
    n = _err(_lib().nbh_convex_hull(p.ctypes.data, len(p), tri.ctypes.data, cap), "convex_hull")
    return tri[:n].copy()


def write_file_atomic(path: str, chunks: Sequence) -> None:
    bufs = [np.frombuffer(c, dtype=np.uint8) if not isinstance(c, np.ndarray) else c.view(np.uint8).reshape(-1) for c in chunks]
    ptrs = (_c.c_void_p * len(bufs))(*[b.ctypes.data for b in bufs])
    sizes = (_c.c_size_t * len(bufs))(*[b.nbytes for b in bufs])
    _err(_lib().nbh_write_file_atomic(os.fsencode(path), ptrs, sizes, len(bufs)), f"write {path}")


def read_file_range(path: str, offset: int, n: int) -> bytes:
    buf = ctypes.create_string_buffer(n)
    got = _err(_lib().nbh_read_file_range(os.fsencode(path), offset, buf, n), f"read {path}")
    return buf.raw[:got]


def sha256(data: bytes) -> str:
    out = ctypes.create_string_buffer(32)
    _lib().nbh_sha256(data, len(data), out)
    return out.raw.hex()


class RecordLoader:
    """Batches of fixed-size records read ahead by native threads.  ``next_into(tensor)`` fills a (pinned) uint8 /
    typed tensor of at least ``batch * record_bytes`` bytes and returns (count, indices)."""

    def __init__(self, path: str, record_bytes: int, n_records: int, batch: int, header_bytes: int = 0, slots: int = 4,
                 threads: int = 2, seed: int = 0, shuffle: bool = True, drop_last: bool = True):
        self.record_bytes, self.batch = record_bytes, batch
        self._h = _lib().nbh_loader_create(os.fsencode(path), header_bytes, record_bytes, n_records, batch, slots, threads,
                                           seed, int(shuffle), int(drop_last))
        if not self._h:
            raise OSError(f"cannot open {path}")
        self._idx = np.zeros(batch, dtype=np.uint64)

    def next_into(self, dst):
        ptr = dst.data_ptr() if hasattr(dst, "data_ptr") else dst.ctypes.data
        n = _err(_lib().nbh_loader_next(self._h, ptr, self._idx.ctypes.data), "loader_next")
        return n, self._idx[:n].copy()

    def reset(self, epoch: int):
        _lib().nbh_loader_reset(self._h, epoch)

    def close(self):
        if self._h:
            _lib().nbh_loader_destroy(self._h)
            self._h = None
