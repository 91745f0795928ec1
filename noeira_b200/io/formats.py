"""Small file formats used around training: NPY arrays, 8-bit PNG images (written from device frame buffers of the ray
tracer), 16-bit PCM WAV, base64 and JSON lines.  Pure Python over ``zlib`` / ``struct``; large payloads go through the
native atomic writer.  (Reference: noeira/io/ npy.mojo, png.mojo, wav.mojo, base64.mojo, json.mojo.)"""
from __future__ import annotations

import base64 as _b64
import json
import struct
import zlib

import numpy as np

from ..runtime import write_file_atomic


# ------------------------------------------------------------------------------------------ NPY (format 1.0)
def save_npy(path: str, arr: np.ndarray):
    arr = np.ascontiguousarray(arr)
    header = "{'descr': '%s', 'fortran_order': False, 'shape': %s, }" % (arr.dtype.str, str(arr.shape) if arr.ndim != 1 else f"({arr.shape[0]},)")
    pad = 64 - (10 + len(header) + 1) % 64
    h = (header + " " * pad + "\n").encode("latin1")
    write_file_atomic(path, [b"\x93NUMPY\x01\x00" + struct.pack("<H", len(h)) + h, arr.view(np.uint8).reshape(-1)])


def load_npy(path: str) -> np.ndarray:
    raw = open(path, "rb").read()
    if raw[:6] != b"\x93NUMPY":
        raise ValueError("not an NPY file")
    major = raw[6]
    hl, off = (struct.unpack("<H", raw[8:10])[0], 10) if major == 1 else (struct.unpack("<I", raw[8:12])[0], 12)
    meta = eval(raw[off: off + hl].decode("latin1"), {"__builtins__": {}})       # a literal dict written by NumPy
    a = np.frombuffer(raw, dtype=np.dtype(meta["descr"]), offset=off + hl)
    return a.reshape(meta["shape"], order="F" if meta["fortran_order"] else "C").copy()


# ------------------------------------------------------------------------------------------ PNG
def _chunk(tag: bytes, data: bytes) -> bytes:
    return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)


def save_png(path: str, img: np.ndarray, level: int = 6):
    """uint8 ``[H, W]`` (grey), ``[H, W, 3]`` (RGB) or ``[H, W, 4]`` (RGBA)."""
    img = np.ascontiguousarray(img, dtype=np.uint8)
    if img.ndim == 2:
        img = img[:, :, None]
    H, W, C = img.shape
    ctype = {1: 0, 3: 2, 4: 6}[C]
    rows = np.concatenate([np.zeros((H, 1), np.uint8), img.reshape(H, W * C)], 1)       # filter type 0 per scanline
    data = b"\x89PNG\r\n\x1a\n" + _chunk(b"IHDR", struct.pack(">IIBBBBB", W, H, 8, ctype, 0, 0, 0)) + \
        _chunk(b"IDAT", zlib.compress(rows.tobytes(), level)) + _chunk(b"IEND", b"")
    write_file_atomic(path, [data])


def load_png(path: str) -> np.ndarray:
    raw = open(path, "rb").read()
    if raw[:8] != b"\x89PNG\r\n\x1a\n":
        raise ValueError("not a PNG file")
    pos, idat, W = 8, b"", None
    while pos < len(raw):
        n, tag = struct.unpack(">I", raw[pos: pos + 4])[0], raw[pos + 4: pos + 8]
        body = raw[pos + 8: pos + 8 + n]
        if tag == b"IHDR":
            W, H, depth, ctype, _, _, interlace = struct.unpack(">IIBBBBB", body)
            if depth != 8 or interlace or ctype not in (0, 2, 6):
                raise ValueError("only 8-bit non-interlaced grey / RGB / RGBA PNGs are supported")
        elif tag == b"IDAT":
            idat += body
        pos += 12 + n
    C = {0: 1, 2: 3, 6: 4}[ctype]
    rows = np.frombuffer(zlib.decompress(idat), np.uint8).reshape(H, 1 + W * C)
    out = np.zeros((H, W * C), np.uint8)
    prev = np.zeros(W * C, np.int32)
    for y in range(H):
        f, line = rows[y, 0], rows[y, 1:].astype(np.int32)
        if f == 0:
            cur = line
        elif f == 2:
            cur = (line + prev) & 255
        else:                                  # Sub / Average / Paeth need the left neighbour: sequential per pixel
            cur = np.zeros(W * C, np.int32)
            for i in range(W * C):
                a = cur[i - C] if i >= C else 0
                b, c = prev[i], (prev[i - C] if i >= C else 0)
                if f == 1:
                    pred = a
                elif f == 3:
                    pred = (a + b) // 2
                else:
                    p = a + b - c
                    pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
                    pred = a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)
                cur[i] = (line[i] + pred) & 255
        out[y] = cur
        prev = cur
    out = out.reshape(H, W, C)
    return out[:, :, 0] if C == 1 else out


# ------------------------------------------------------------------------------------------ WAV / base64 / JSON lines
def save_wav(path: str, samples: np.ndarray, rate: int = 16000):
    s = np.asarray(samples)
    if s.dtype != np.int16:
        s = (np.clip(s, -1, 1) * 32767).astype(np.int16)
    ch = 1 if s.ndim == 1 else s.shape[1]
    data = s.tobytes()
    hdr = b"RIFF" + struct.pack("<I", 36 + len(data)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, ch, rate, rate * ch * 2, ch * 2, 16) + \
        b"data" + struct.pack("<I", len(data))
    write_file_atomic(path, [hdr + data])


def load_wav(path: str):
    raw = open(path, "rb").read()
    if raw[:4] != b"RIFF" or raw[8:12] != b"WAVE":
        raise ValueError("not a WAV file")
    pos, fmt, data = 12, None, None
    while pos + 8 <= len(raw):
        tag, n = raw[pos: pos + 4], struct.unpack("<I", raw[pos + 4: pos + 8])[0]
        if tag == b"fmt ":
            fmt = struct.unpack("<HHIIHH", raw[pos + 8: pos + 24])
        elif tag == b"data":
            data = raw[pos + 8: pos + 8 + n]
        pos += 8 + n + (n & 1)
    s = np.frombuffer(data, np.int16)
    return (s.reshape(-1, fmt[1]) if fmt[1] > 1 else s), fmt[2]


def b64encode(b: bytes) -> str:
    return _b64.b64encode(b).decode()


def b64decode(s: str) -> bytes:
    return _b64.b64decode(s)


def write_jsonl(path: str, rows):
    write_file_atomic(path, ["".join(json.dumps(r) + "\n" for r in rows).encode()])


def read_jsonl(path: str):
    return [json.loads(l) for l in open(path, encoding="utf-8") if l.strip()]


# ------------------------------------------------------------------------------------------ zstd (system libzstd through ctypes)
_ZSTD = None


def _zstd():
    global _ZSTD
    if _ZSTD is None:
        import ctypes
        import ctypes.util
        name = ctypes.util.find_library("zstd") or "libzstd.so.1"
        lib = ctypes.CDLL(name)
        lib.ZSTD_compressBound.restype = ctypes.c_size_t
        lib.ZSTD_compressBound.argtypes = [ctypes.c_size_t]
        lib.ZSTD_compress.restype = ctypes.c_size_t
        lib.ZSTD_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t, ctypes.c_int]
        lib.ZSTD_isError.restype = ctypes.c_uint
        lib.ZSTD_isError.argtypes = [ctypes.c_size_t]
        lib.ZSTD_getErrorName.restype = ctypes.c_char_p
        lib.ZSTD_getErrorName.argtypes = [ctypes.c_size_t]
        lib.ZSTD_createDStream.restype = ctypes.c_void_p
        lib.ZSTD_freeDStream.argtypes = [ctypes.c_void_p]
        lib.ZSTD_initDStream.restype = ctypes.c_size_t
        lib.ZSTD_initDStream.argtypes = [ctypes.c_void_p]
        lib.ZSTD_decompressStream.restype = ctypes.c_size_t
        lib.ZSTD_decompressStream.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        _ZSTD = lib
    return _ZSTD


def zstd_compress(data: bytes, level: int = 3) -> bytes:
    import ctypes
    lib = _zstd()
    cap = lib.ZSTD_compressBound(len(data))
    buf = ctypes.create_string_buffer(cap)
    n = lib.ZSTD_compress(buf, cap, data, len(data), level)
    if lib.ZSTD_isError(n):
        raise ValueError(f"zstd: {lib.ZSTD_getErrorName(n).decode()}")
    return buf.raw[:n]


def zstd_decompress(data: bytes, chunk: int = 1 << 17) -> bytes:
    """Streaming decode: works for frames without a stored content size and for several concatenated frames (what a
    chunked HTTP body of a ``.zst`` shard delivers)."""
    import ctypes

    class _Buf(ctypes.Structure):
        _fields_ = [("ptr", ctypes.c_void_p), ("size", ctypes.c_size_t), ("pos", ctypes.c_size_t)]

    lib = _zstd()
    ds = lib.ZSTD_createDStream()
    try:
        lib.ZSTD_initDStream(ds)
        src = ctypes.create_string_buffer(data, len(data))
        inb = _Buf(ctypes.cast(src, ctypes.c_void_p), len(data), 0)
        dst = ctypes.create_string_buffer(chunk)
        out = bytearray()
        while True:
            outb = _Buf(ctypes.cast(dst, ctypes.c_void_p), chunk, 0)
            rc = lib.ZSTD_decompressStream(ds, ctypes.byref(outb), ctypes.byref(inb))
            if lib.ZSTD_isError(rc):
                raise ValueError(f"zstd: {lib.ZSTD_getErrorName(rc).decode()}")
            out += dst.raw[: outb.pos]
            if inb.pos >= inb.size and outb.pos < chunk:
                if rc != 0:
                    raise ValueError("zstd: truncated frame")
                return bytes(out)
    finally:
        lib.ZSTD_freeDStream(ds)


# ------------------------------------------------------------------------------------------ tar archives
def write_tar(path: str, members: dict, compression: str = ""):
    """``members``: ``{name: bytes}``; ``compression``: "", "gz", "bz2" or "xz"."""
    import io
    import tarfile
    with tarfile.open(path, f"w:{compression}" if compression else "w") as tf:
        for name, data in members.items():
            info = tarfile.TarInfo(name)
            info.size = len(data)
            tf.addfile(info, io.BytesIO(data))


def read_tar(path: str, prefix: str = "") -> dict:
    """Regular files of an archive (any compression tarfile recognises) as ``{name: bytes}``.  Members whose names would
    leave the archive root (absolute paths, ``..``) are refused."""
    import tarfile
    out = {}
    with tarfile.open(path, "r:*") as tf:
        for m in tf:
            if not m.isfile() or not m.name.startswith(prefix):
                continue
            if m.name.startswith("/") or ".." in m.name.split("/"):
                raise ValueError(f"unsafe member name {m.name!r}")
            out[m.name] = tf.extractfile(m).read()
    return out
