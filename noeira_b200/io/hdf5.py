"""HDF5 files without libhdf5: a reader for the classic on-disk layout and a writer that produces it.

Robot-learning datasets (ALOHA / ACT episodes, robomimic) are HDF5 files written with the library defaults: version-0
superblock, version-1 object headers, groups as symbol tables (B-tree of symbol nodes + local heap of names), datasets stored
contiguously or chunked with the deflate / shuffle filters.  This module implements exactly that subset in pure Python
(struct + zlib + numpy): there is no libhdf5 / h5py in the image, and the reference binds libhdf5 through FFI
(noeira/io/hdf5/, 13 files; noeira/data/store.mojo builds its trajectory store on it).

Reader   ``H5File(path)``: ``keys()``, ``f["a/b"]`` → ``H5Group`` or ``H5Dataset`` (``shape``, ``dtype``, ``read()``, ``[...]``
         with leading-axis slicing that only touches the chunks it needs), ``attrs`` (numeric and fixed-length string
         attributes).  Follows object-header continuation blocks, multi-level B-trees of both kinds, edge chunks, the
         shuffle + deflate + fletcher32 pipeline.  Files written with ``libver="latest"`` (version-2 headers, fractal heaps)
         are reported as unsupported.
Writer   ``write_hdf5(path, tree, compression=None, chunk_rows=None, attrs=None)``: ``tree`` is a nested dict of numpy arrays;
         datasets are contiguous, or chunked along the first axis with deflate (+ shuffle) when ``compression="gzip"``.
"""
from __future__ import annotations

import struct
import zlib
from typing import Dict, Iterator, List, Optional, Tuple

import numpy as np

SIGNATURE = b"\x89HDF\r\n\x1a\n"
UNDEF = 0xFFFFFFFFFFFFFFFF
MSG_DATASPACE, MSG_DATATYPE, MSG_FILL, MSG_LAYOUT, MSG_FILTERS, MSG_ATTR, MSG_CONT, MSG_SYMTAB = 0x1, 0x3, 0x5, 0x8, 0xB, 0xC, 0x10, 0x11


class H5Error(ValueError):
    pass


def _pad8(n: int) -> int:
    return (n + 7) & ~7


# ------------------------------------------------------------------------------------------ datatypes
VLEN_STR = np.dtype([("len", "<u4"), ("addr", "<u8"), ("idx", "<u4")])      # the 16-byte element of a variable-length string


def _vlen_type_message(utf8: bool = True) -> bytes:
    """Class 9 (variable length), type string, null-terminated, UTF-8 or ASCII; base type: one-byte string."""
    base = struct.pack("<BBBBI", 0x10 | 3, 0x10 if utf8 else 0, 0, 0, 1)
    return struct.pack("<BBBBI", 0x10 | 9, 0x01, 0x01 if utf8 else 0, 0, 16) + base


def _decode_dtype(b: bytes) -> Tuple[np.dtype, int]:
    cls, ver = b[0] & 0x0F, b[0] >> 4
    bits0 = b[1]
    size = struct.unpack_from("<I", b, 4)[0]
    order = ">" if bits0 & 1 else "<"
    if cls == 0:
        return np.dtype(f"{order}{'i' if bits0 & 0x08 else 'u'}{size}"), size
    if cls == 1:
        return np.dtype(f"{order}f{size}"), size
    if cls == 3:
        return np.dtype(f"S{size}"), size
    if cls == 9 and (bits0 & 0x0F) == 1:                       # variable-length string: (length, global-heap address, index)
        return VLEN_STR, 16
    raise H5Error(f"datatype class {cls} (version {ver}) is not supported")


def _encode_dtype(dt: np.dtype) -> bytes:
    dt = np.dtype(dt)
    size = dt.itemsize
    if dt.kind in "iu" or dt.kind == "b":
        bits0 = 0x08 if dt.kind == "i" else 0
        return struct.pack("<BBBBIHH", 0x10 | 0, bits0, 0, 0, size, 0, size * 8)
    if dt.kind == "f":
        exp, mant, bias = {2: (5, 10, 15), 4: (8, 23, 127), 8: (11, 52, 1023)}[size]
        return struct.pack("<BBBBIHHBBBBI", 0x10 | 1, 0x20, size * 8 - 1, 0, size, 0, size * 8, mant, exp, 0, mant, bias)
    if dt.kind == "S":
        return struct.pack("<BBBBI", 0x10 | 3, 0, 0, 0, size)
    raise H5Error(f"cannot store dtype {dt}")


# ------------------------------------------------------------------------------------------ reader
class _Reader:
    def __init__(self, data):
        self.d = data

    def at(self, off: int, fmt: str):
        return struct.unpack_from("<" + fmt, self.d, off)

    def messages(self, addr: int) -> List[Tuple[int, bytes]]:
        """All messages of a version-1 object header, continuation blocks included."""
        d = self.d
        if d[addr: addr + 4] == b"OHDR":
            raise H5Error("version-2 object headers (libver='latest') are not supported")
        ver, _, nmsg, _refs, hsize = self.at(addr, "BBHII")
        if ver != 1:
            raise H5Error(f"object header version {ver}")
        out, blocks = [], [(addr + 16, hsize)]
        while blocks and len(out) < nmsg:
            off, left = blocks.pop(0)
            end = off + left
            while off + 8 <= end and len(out) < nmsg:
                mtype, msize, _flags = self.at(off, "HHB")
                body = bytes(d[off + 8: off + 8 + msize])
                off += 8 + msize
                if mtype == MSG_CONT:
                    blocks.append(struct.unpack("<QQ", body[:16]))
                out.append((mtype, body))
        return out

    # ---- groups
    def global_heap_object(self, addr: int, idx: int) -> bytes:
        """Object ``idx`` of the global heap collection at ``addr`` ("GCOL")."""
        if bytes(self.d[addr: addr + 4]) != b"GCOL":
            raise H5Error("bad global heap signature")
        size = struct.unpack_from("<Q", self.d, addr + 8)[0]
        p, end = addr + 16, addr + size
        while p + 16 <= end:
            oid, _ref, _res, osize = struct.unpack_from("<HHIQ", self.d, p)
            if oid == idx:
                return bytes(self.d[p + 16: p + 16 + osize])
            if oid == 0:
                break
            p += 16 + _pad8(osize)
        raise H5Error(f"global heap object {idx} not found")

    def vlen_strings(self, a: np.ndarray) -> np.ndarray:
        out = np.empty(a.shape, dtype=object)
        for i, e in enumerate(a.reshape(-1)):
            out.reshape(-1)[i] = self.global_heap_object(int(e["addr"]), int(e["idx"]))[: int(e["len"])].decode("utf-8", "replace") \
                if int(e["addr"]) not in (0, UNDEF) else ""
        return out

    def heap_name(self, heap_addr: int, off: int) -> str:
        if self.d[heap_addr: heap_addr + 4] != b"HEAP":
            raise H5Error("bad local heap")
        seg = self.at(heap_addr + 24, "Q")[0]
        n = 64
        while True:
            raw = bytes(self.d[seg + off: seg + off + n])
            if b"\0" in raw or len(raw) < n:
                return raw.split(b"\0")[0].decode("utf-8")
            n *= 4

    def group_entries(self, btree: int, heap: int) -> Iterator[Tuple[str, int]]:
        d = self.d
        if d[btree: btree + 4] == b"SNOD":
            n = self.at(btree + 6, "H")[0]
            for i in range(n):
                name_off, obj = self.at(btree + 8 + 40 * i, "QQ")
                yield self.heap_name(heap, name_off), obj
            return
        if d[btree: btree + 4] != b"TREE":
            raise H5Error("bad group B-tree node")
        _type, _level, used = self.at(btree + 4, "BBH")
        p = btree + 24
        for i in range(used):
            child = self.at(p + 8, "Q")[0]          # key i (8), child i (8)
            yield from self.group_entries(child, heap)
            p += 16

    # ---- chunks
    def chunk_entries(self, node: int, rank: int) -> Iterator[Tuple[Tuple[int, ...], int, int, int]]:
        """(chunk offset, stored size, filter mask, address) of every chunk below a chunk B-tree node."""
        d = self.d
        if d[node: node + 4] != b"TREE":
            raise H5Error("bad chunk B-tree node")
        _type, level, used = self.at(node + 4, "BBH")
        key = 8 + 8 * (rank + 1)
        p = node + 24
        for _ in range(used):
            size, mask = self.at(p, "II")
            offs = self.at(p + 8, f"{rank + 1}Q")[:rank]
            child = self.at(p + key, "Q")[0]
            if level == 0:
                yield offs, size, mask, child
            else:
                yield from self.chunk_entries(child, rank)
            p += key + 8


class H5Dataset:
    def __init__(self, rd: _Reader, name: str, msgs):
        self._rd, self.name = rd, name
        self.attrs = _attrs(msgs, rd)
        self.filters: List[Tuple[int, Tuple[int, ...]]] = []
        self.shape: Tuple[int, ...] = ()
        self.dtype = None
        self._layout = None
        for t, b in msgs:
            if t == MSG_DATASPACE:
                self.shape = _decode_space(b)
            elif t == MSG_DATATYPE:
                self.dtype, self._esize = _decode_dtype(b)
            elif t == MSG_LAYOUT:
                self._layout = b
            elif t == MSG_FILTERS:
                self.filters = _decode_filters(b)
        if self.dtype is None or self._layout is None:
            raise H5Error(f"{name}: not a dataset")

    def __len__(self):
        return self.shape[0]

    def read(self, start: int = 0, stop: Optional[int] = None) -> np.ndarray:
        """The whole array, or rows ``[start, stop)`` of the first axis.  Variable-length strings come back as an object
        array of ``str``."""
        a = self._read_raw(start, stop)
        return self._rd.vlen_strings(np.asarray(a)) if self.dtype == VLEN_STR else a

    def _read_raw(self, start: int = 0, stop: Optional[int] = None) -> np.ndarray:
        rd, b = self._rd, self._layout
        ver, cls = b[0], b[1]
        if ver != 3:
            raise H5Error(f"data layout version {ver}")
        shape = self.shape
        n0 = shape[0] if shape else 1
        stop = n0 if stop is None else min(stop, n0)
        row = int(np.prod(shape[1:], dtype=np.int64)) if len(shape) > 1 else 1
        if cls == 1:                                           # contiguous
            addr, _size = struct.unpack_from("<QQ", b, 2)
            if not shape:
                return np.frombuffer(rd.d, self.dtype, 1, addr)[0].copy() if addr != UNDEF else np.zeros((), self.dtype)
            if addr == UNDEF:
                return np.zeros((stop - start,) + shape[1:], self.dtype)
            a = np.frombuffer(rd.d, self.dtype, (stop - start) * row, addr + start * row * self._esize)
            return a.reshape((stop - start,) + shape[1:]).copy()
        if cls == 0:                                           # compact
            size = struct.unpack_from("<H", b, 2)[0]
            a = np.frombuffer(b, self.dtype, size // self._esize, 4).reshape(shape)
            return a[start:stop].copy() if shape else a.copy()
        if cls != 2:
            raise H5Error(f"layout class {cls}")
        rank = b[2] - 1
        btree = struct.unpack_from("<Q", b, 3)[0]
        cdims = struct.unpack_from(f"<{rank}I", b, 11)
        out = np.zeros((stop - start,) + tuple(shape[1:]), self.dtype)
        if btree == UNDEF:
            return out
        for offs, size, mask, addr in rd.chunk_entries(btree, rank):
            if offs[0] >= stop or offs[0] + cdims[0] <= start:
                continue
            raw = bytes(rd.d[addr: addr + size])
            for i, (fid, cd) in enumerate(reversed(self.filters)):
                if mask >> (len(self.filters) - 1 - i) & 1:
                    continue
                if fid == 1:
                    raw = zlib.decompress(raw)
                elif fid == 2:
                    es = cd[0] if cd else self._esize
                    raw = np.frombuffer(raw, np.uint8).reshape(es, -1).T.tobytes()
                elif fid == 3:
                    raw = raw[:-4]
                else:
                    raise H5Error(f"filter {fid} is not supported")
            chunk = np.frombuffer(raw, self.dtype, int(np.prod(cdims))).reshape(cdims)
            src, dst = [], []
            for ax in range(rank):
                lo = offs[ax]
                hi = min(lo + cdims[ax], shape[ax])
                if ax == 0:
                    a0, a1 = max(lo, start), min(hi, stop)
                    src.append(slice(a0 - lo, a1 - lo)), dst.append(slice(a0 - start, a1 - start))
                else:
                    src.append(slice(0, hi - lo)), dst.append(slice(lo, hi))
            out[tuple(dst)] = chunk[tuple(src)]
        return out

    def __getitem__(self, key):
        if key is Ellipsis or key == ():
            return self.read()
        if isinstance(key, slice) and key.step in (None, 1):
            s, e, _ = key.indices(self.shape[0])
            return self.read(s, e)
        if isinstance(key, int):
            k = key % self.shape[0]
            return self.read(k, k + 1)[0]
        return self.read()[key]


def _decode_space(b: bytes) -> Tuple[int, ...]:
    ver, rank = b[0], b[1]
    if ver == 1:
        return tuple(struct.unpack_from(f"<{rank}Q", b, 8))
    if ver == 2:
        return tuple(struct.unpack_from(f"<{rank}Q", b, 4)) if b[3] != 2 else ()
    raise H5Error(f"dataspace version {ver}")


def _decode_filters(b: bytes):
    ver, n = b[0], b[1]
    out = []
    p = 8 if ver == 1 else 2
    for _ in range(n):
        fid = struct.unpack_from("<H", b, p)[0]
        if ver == 1 or fid >= 256:
            nlen, _flags, ncd = struct.unpack_from("<HHH", b, p + 2)
            p += 8
        else:                                        # version 2 drops the name length of the library's own filters
            nlen = 0
            _flags, ncd = struct.unpack_from("<HH", b, p + 2)
            p += 6
        p += _pad8(nlen) if ver == 1 else nlen
        cd = struct.unpack_from(f"<{ncd}I", b, p)
        p += 4 * ncd + (4 if ver == 1 and ncd % 2 else 0)
        out.append((fid, cd))
    return out


def _attrs(msgs, rd: "_Reader" = None) -> Dict[str, object]:
    out = {}
    for t, b in msgs:
        if t != MSG_ATTR or b[0] != 1:
            continue
        nlen, tlen, slen = struct.unpack_from("<HHH", b, 2)
        name = b[8: 8 + nlen].split(b"\0")[0].decode()
        p = 8 + _pad8(nlen)
        try:
            dt, es = _decode_dtype(b[p: p + tlen])
        except H5Error:
            continue
        p += _pad8(tlen)
        shape = _decode_space(b[p: p + slen])
        p += _pad8(slen)
        n = int(np.prod(shape)) if shape else 1
        v = np.frombuffer(b, dt, n, p).reshape(shape)
        if dt == VLEN_STR:
            if rd is not None:
                sv = rd.vlen_strings(v)
                out[name] = sv.item() if not shape else sv
            continue
        out[name] = (v.item() if not shape else v.copy()) if dt.kind != "S" else (v.item().rstrip(b"\0").decode() if not shape else v.copy())
    return out


class H5Group:
    def __init__(self, rd: _Reader, name: str, addr: int):
        self._rd, self.name, self._addr = rd, name, addr
        msgs = rd.messages(addr)
        self.attrs = _attrs(msgs, rd)
        self._links: Dict[str, int] = {}
        for t, b in msgs:
            if t == MSG_SYMTAB:
                btree, heap = struct.unpack_from("<QQ", b, 0)
                self._links = dict(rd.group_entries(btree, heap))
                break
        else:
            if not any(t in (MSG_LAYOUT,) for t, _ in msgs):
                raise H5Error(f"{name or '/'}: group without a symbol table (link messages / fractal heaps are not supported)")

    def keys(self):
        return sorted(self._links)

    def __contains__(self, k):
        return k.split("/")[0] in self._links

    def __getitem__(self, path: str):
        node = self
        for part in [p for p in path.split("/") if p]:
            if not isinstance(node, H5Group) or part not in node._links:
                raise KeyError(path)
            addr = node._links[part]
            msgs = node._rd.messages(addr)
            name = f"{node.name}/{part}"
            node = H5Dataset(node._rd, name, msgs) if any(t == MSG_LAYOUT for t, _ in msgs) else H5Group(node._rd, name, addr)
        return node

    def visit(self, prefix: str = "") -> Iterator[Tuple[str, "H5Dataset"]]:
        """Every dataset below this group as (path, dataset)."""
        for k in self.keys():
            v = self[k]
            p = f"{prefix}{k}"
            if isinstance(v, H5Group):
                yield from v.visit(p + "/")
            else:
                yield p, v


class H5File(H5Group):
    def __init__(self, path: str):
        self._buf = np.memmap(path, dtype=np.uint8, mode="r")
        d = memoryview(self._buf)
        base = 0
        while bytes(d[base: base + 8]) != SIGNATURE:             # the superblock may sit at 0, 512, 1024, ...
            base = 512 if base == 0 else base * 2
            if base + 8 > len(d):
                raise H5Error("not an HDF5 file")
        ver = d[base + 8]
        if ver not in (0, 1):
            raise H5Error(f"superblock version {ver} (libver='latest' files) is not supported")
        if d[base + 13] != 8 or d[base + 14] != 8:
            raise H5Error("only 8-byte offsets and lengths are supported")
        root = base + (24 if ver == 0 else 28) + 32                # root group symbol-table entry
        obj = struct.unpack_from("<Q", d, root + 8)[0]
        super().__init__(_Reader(d), "", obj)

    def close(self):
        self._rd = None
        self._buf = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def read_hdf5(path: str) -> Dict[str, np.ndarray]:
    """Every dataset of a file as ``{path: array}``."""
    with H5File(path) as f:
        return {p: ds.read() for p, ds in f.visit()}


# ------------------------------------------------------------------------------------------ writer
class _Writer:
    def __init__(self):
        self.buf = bytearray(96)                                   # room for the superblock

    def alloc(self, data: bytes) -> int:
        pad = _pad8(len(self.buf)) - len(self.buf)
        self.buf += b"\0" * pad
        addr = len(self.buf)
        self.buf += data
        return addr

    @staticmethod
    def msg(mtype: int, body: bytes, flags: int = 0) -> bytes:
        body = body + b"\0" * (_pad8(len(body)) - len(body))
        return struct.pack("<HHBBBB", mtype, len(body), flags, 0, 0, 0) + body

    def header(self, msgs: List[bytes]) -> int:
        body = b"".join(msgs)
        return self.alloc(struct.pack("<BBHII", 1, 0, len(msgs), 1, len(body)) + b"\0" * 4 + body)

    def attr_msgs(self, attrs) -> List[bytes]:
        out = []
        for k, v in (attrs or {}).items():
            a = np.asarray(v.encode() if isinstance(v, str) else v)
            vlen = a.dtype.kind == "O"                          # an object array of text: variable-length strings
            if vlen:
                a = self.vlen_elements(a)
            if a.dtype.kind == "U":
                a = a.astype("S")
            if a.dtype == np.bool_:
                a = a.astype(np.uint8)
            name = k.encode() + b"\0"
            dt = _vlen_type_message() if vlen else _encode_dtype(a.dtype)
            sp = _encode_space(a.shape)
            body = struct.pack("<BBHHH", 1, 0, len(name), len(dt), len(sp)) + name + b"\0" * (_pad8(len(name)) - len(name)) + \
                dt + b"\0" * (_pad8(len(dt)) - len(dt)) + sp + b"\0" * (_pad8(len(sp)) - len(sp)) + a.tobytes()
            out.append(self.msg(MSG_ATTR, body))
        return out

    def global_heap(self, items: List[bytes]) -> List[Tuple[int, int, int]]:
        """One global heap collection holding ``items`` → (length, collection address, object index) per item.  The
        collection is at least 4096 bytes; the rest is the free-space object 0."""
        body = bytearray()
        for i, it in enumerate(items):
            body += struct.pack("<HHIQ", i + 1, 1, 0, len(it)) + it + b"\0" * (_pad8(len(it)) - len(it))
        total = max(4096, _pad8(16 + len(body) + 16))
        free = total - 16 - len(body)
        blob = b"GCOL" + struct.pack("<B3xQ", 1, total) + bytes(body) + struct.pack("<HHIQ", 0, 0, 0, free) + b"\0" * (free - 16)
        addr = self.alloc(blob)
        return [(len(it), addr, i + 1) for i, it in enumerate(items)]

    def vlen_elements(self, a: np.ndarray) -> np.ndarray:
        items = [(x if isinstance(x, bytes) else str(x).encode("utf-8")) for x in a.reshape(-1)]
        el = np.zeros(len(items), VLEN_STR)
        if items:
            for i, (ln, addr, idx) in enumerate(self.global_heap(items)):
                el[i] = (ln, addr, idx)
        return el.reshape(a.shape)

    def dataset(self, a: np.ndarray, compression, chunk_rows, attrs) -> int:
        a = np.asarray(a)
        if a.dtype.kind in "UO":                                # text of any length: variable-length strings
            el = self.vlen_elements(a)
            msgs = [self.msg(MSG_DATASPACE, _encode_space(a.shape)), self.msg(MSG_DATATYPE, _vlen_type_message(), flags=1),
                    self.msg(MSG_FILL, struct.pack("<BBBB", 2, 2, 0, 0)),
                    self.msg(MSG_LAYOUT, struct.pack("<BBQQ", 3, 1, self.alloc(el.tobytes()) if el.size else UNDEF, el.nbytes))]
            return self.header(msgs + self.attr_msgs(attrs))
        a = np.ascontiguousarray(a)
        if a.dtype == np.bool_:
            a = a.astype(np.uint8)
        if a.dtype.byteorder == ">":
            a = a.astype(a.dtype.newbyteorder("<"))
        msgs = [self.msg(MSG_DATASPACE, _encode_space(a.shape)), self.msg(MSG_DATATYPE, _encode_dtype(a.dtype), flags=1),
                self.msg(MSG_FILL, struct.pack("<BBBB", 2, 2, 0, 0))]
        es = a.dtype.itemsize
        if compression is None or a.ndim == 0 or a.size == 0:
            addr = self.alloc(a.tobytes()) if a.size else UNDEF
            msgs.append(self.msg(MSG_LAYOUT, struct.pack("<BBQQ", 3, 1, addr, a.nbytes)))
        else:
            if compression != "gzip":
                raise H5Error("compression must be None or 'gzip'")
            rank = a.ndim
            rows = chunk_rows or max(1, min(a.shape[0], (1 << 20) // max(a[0].nbytes, 1)))
            cdims = (rows,) + a.shape[1:]
            nchunks = -(-a.shape[0] // rows)
            if nchunks > 64:
                raise H5Error("more than 64 chunks along the first axis: raise chunk_rows")
            entries = []
            for c in range(nchunks):
                blk = np.zeros(cdims, a.dtype)
                part = a[c * rows: (c + 1) * rows]
                blk[: part.shape[0]] = part
                raw = np.frombuffer(blk.tobytes(), np.uint8).reshape(-1, es).T.tobytes()          # shuffle
                comp = zlib.compress(raw, 4)
                entries.append(((c * rows,) + (0,) * (rank - 1), len(comp), self.alloc(comp)))
            node = bytearray(b"TREE" + struct.pack("<BBHQQ", 1, 0, len(entries), UNDEF, UNDEF))
            for offs, size, addr in entries:
                node += struct.pack(f"<II{rank + 1}Q", size, 0, *offs, 0) + struct.pack("<Q", addr)
            node += struct.pack(f"<II{rank + 1}Q", 0, 0, *((nchunks * rows,) + (0,) * (rank - 1)), 0)  # closing key
            node += b"\0" * (24 + 65 * (8 + 8 * (rank + 1)) + 64 * 8 - len(node))       # allocated at full capacity (K = 32)
            btree = self.alloc(bytes(node))
            filt = struct.pack("<BB6x", 1, 2) + struct.pack("<HHHHI4x", 2, 0, 1, 1, es) + struct.pack("<HHHHI4x", 1, 0, 1, 1, 4)
            msgs.append(self.msg(MSG_FILTERS, filt))
            msgs.append(self.msg(MSG_LAYOUT, struct.pack(f"<BBBQ{rank + 1}I", 3, 2, rank + 1, btree, *cdims, es)))
        return self.header(msgs + self.attr_msgs(attrs))

    def group(self, tree: dict, compression, chunk_rows, attrs) -> Tuple[int, int, int]:
        """Writes the children, then heap, symbol nodes, B-tree and header.  Returns (header, btree, heap) addresses."""
        node_attrs = (attrs or {}).get("", {}) if isinstance(attrs, dict) else {}
        children = {}
        for name in tree:
            sub_attrs = {k[len(name) + 1:] if k != name else "": v for k, v in (attrs or {}).items() if k == name or k.startswith(name + "/")}
            v = tree[name]
            if isinstance(v, dict):
                children[name] = self.group(v, compression, chunk_rows, sub_attrs)[0]
            else:
                children[name] = self.dataset(np.asarray(v), compression, chunk_rows, sub_attrs.get("", {}))
        names = sorted(children, key=lambda s: s.encode())
        if len(names) > 256:
            raise H5Error("more than 256 links in one group")
        heap_data, offs = bytearray(b"\0" * 8), {}
        for n in names:
            offs[n] = len(heap_data)
            e = n.encode() + b"\0"
            heap_data += e + b"\0" * (_pad8(len(e)) - len(e))
        seg = self.alloc(bytes(heap_data))
        heap = self.alloc(b"HEAP" + struct.pack("<B3xQQQ", 0, len(heap_data), UNDEF, seg))
        snods = []
        for i in range(0, max(len(names), 1), 8):
            part = names[i: i + 8]
            body = bytearray(b"SNOD" + struct.pack("<BBH", 1, 0, len(part)))
            for n in part:
                body += struct.pack("<QQII16x", offs[n], children[n], 0, 0)
            body += b"\0" * (40 * (8 - len(part)))
            snods.append((self.alloc(bytes(body)), offs[part[-1]] if part else 0))
        node = bytearray(b"TREE" + struct.pack("<BBHQQ", 0, 0, len(snods), UNDEF, UNDEF) + struct.pack("<Q", 0))
        for addr, last in snods:
            node += struct.pack("<QQ", addr, last)
        node += b"\0" * (16 * (32 - len(snods)))                    # a group node is allocated at its full capacity (K = 16)
        btree = self.alloc(bytes(node))
        hdr = self.header([self.msg(MSG_SYMTAB, struct.pack("<QQ", btree, heap))] + self.attr_msgs(node_attrs))
        return hdr, btree, heap


def _encode_space(shape) -> bytes:
    return struct.pack("<BBBB4x", 1, len(shape), 0, 0) + b"".join(struct.pack("<Q", int(s)) for s in shape)


def write_hdf5(path: str, tree: dict, compression: Optional[str] = None, chunk_rows: Optional[int] = None, attrs: Optional[dict] = None):
    """``tree``: nested dict of arrays.  ``attrs``: ``{"": {...root...}, "group/dataset": {...}}`` numeric / string values."""
    w = _Writer()
    hdr, btree, heap = w.group(tree, compression, chunk_rows, attrs or {})
    eof = _pad8(len(w.buf))
    w.buf += b"\0" * (eof - len(w.buf))
    sb = SIGNATURE + struct.pack("<BBBBBBBBHHI", 0, 0, 0, 0, 0, 8, 8, 0, 4, 16, 0) + struct.pack("<QQQQ", 0, UNDEF, eof, UNDEF) + \
        struct.pack("<QQII", 0, hdr, 1, 0) + struct.pack("<QQ", btree, heap)
    assert len(sb) == 96
    w.buf[:96] = sb
    with open(path, "wb") as f:
        f.write(w.buf)
