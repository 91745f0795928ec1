"""Fetch, verify, extract and materialise an asset pack; ``pull_pack(pack, into_dir)`` is idempotent.

Three separate stages:
  1. FETCH    ``<cache>/assets/<sha256>.archive``   verified against the declared SHA-256 (and size)
  2. EXTRACT  ``<cache>/assets/<sha256>/``          once, marked by a ``.ok`` file
  3. LINK     ``<into_dir>/<dest>/``                hard links, falling back to copies; never symlinks (a link into a
                                                     cache dies with the cache and breaks under rsync)
The cache is keyed by the archive's hash, not the pack name: two environments declaring the same bytes share one
download, and a re-cut archive can never be served from a stale entry.
The credential is chosen by the pack's provider, never inferred from the URL (reference: noeira/assets/resolve.mojo:45-255).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import tarfile
import zipfile
from dataclasses import dataclass, field
from typing import Dict

from .pack import PROVIDER_HF, PROVIDER_HTTPS, PROVIDER_NOEIRA, Pack


def cache_root() -> str:
    root = os.environ.get("NOEIRA_CACHE") or os.path.join(os.path.expanduser("~"), ".cache", "noeira")
    return os.path.join(root, "assets")


@dataclass
class Resolved:
    url: str
    headers: Dict[str, str] = field(default_factory=dict)


def _http(method, url, headers=None, body=b""):
    from ..runtime.host import http_request
    return http_request(method, url, headers=headers or {}, body=body, timeout_ms=60000)


def resolve_url(pack: Pack) -> Resolved:
    """Where the bytes are and which header (if any) goes with the request."""
    if pack.provider == PROVIDER_HTTPS:
        hdr = {}
        if pack.token_env:
            tok = os.environ.get(pack.token_env, "")
            if not tok:
                raise RuntimeError(f"pack {pack.ref()}: token_env={pack.token_env} is not set")
            hdr["Authorization"] = f"Bearer {tok}"
        return Resolved(pack.url, hdr)
    if pack.provider == PROVIDER_HF:
        tok = os.environ.get("HF_TOKEN", "")
        return Resolved(pack.url, {"Authorization": f"Bearer {tok}"} if tok else {})
    if pack.provider == PROVIDER_NOEIRA:
        key = os.environ.get("NOEIRA_CLOUD_API_KEY", "")
        base = os.environ.get("NOEIRA_CLOUD_URL", "")
        if not key or not base:
            raise RuntimeError(f"pack {pack.ref()}: provider=noeira needs NOEIRA_CLOUD_API_KEY and NOEIRA_CLOUD_URL")
        st, body = _http("GET", f"{base.rstrip('/')}/v1/assets/{pack.id}", {"Authorization": f"Bearer {key}"})
        if st != 200:
            raise RuntimeError(f"pack {pack.ref()}: catalog answered {st}")
        url = json.loads(body.decode())["url"]
        return Resolved(url, {})  # presigned: the transfer itself carries no credential
    raise ValueError(f"unknown provider {pack.provider!r}")


def archive_path(pack: Pack) -> str:
    return os.path.join(cache_root(), f"{pack.sha256}.archive")


def extract_dir(pack: Pack) -> str:
    return os.path.join(cache_root(), pack.sha256)


def _sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def pack_status(pack: Pack, into_dir: str) -> str:
    """'linked' (dest is populated), 'extracted', 'fetched' or 'absent'."""
    if os.path.isfile(os.path.join(into_dir, pack.dest, ".pack_ok")):
        return "linked"
    if os.path.isfile(os.path.join(extract_dir(pack), ".ok")):
        return "extracted"
    if os.path.isfile(archive_path(pack)):
        return "fetched"
    return "absent"


def _safe_members(tf: tarfile.TarFile, root: str):
    for m in tf.getmembers():
        target = os.path.realpath(os.path.join(root, m.name))
        if not target.startswith(os.path.realpath(root) + os.sep) and target != os.path.realpath(root):
            raise RuntimeError(f"archive member {m.name!r} escapes the extraction directory")
        if m.issym() or m.islnk():
            raise RuntimeError(f"archive member {m.name!r} is a link; packs hold plain files only")
        yield m


def _extract(archive: str, out: str) -> None:
    tmp = out + ".partial"
    shutil.rmtree(tmp, ignore_errors=True)
    os.makedirs(tmp)
    with open(archive, "rb") as f:
        magic = f.read(6)
    if magic[:4] == b"\x28\xb5\x2f\xfd":
        raise RuntimeError("zstd-compressed archives need a zstd decoder, which this build does not have; "
                           "re-cut the pack as .tar.gz")
    if magic[:2] == b"PK":
        with zipfile.ZipFile(archive) as z:
            for n in z.namelist():
                if os.path.isabs(n) or ".." in n.split("/"):
                    raise RuntimeError(f"archive member {n!r} escapes the extraction directory")
            z.extractall(tmp)
    else:
        with tarfile.open(archive, "r:*") as tf:
            tf.extractall(tmp, members=_safe_members(tf, tmp), filter="data")
    with open(os.path.join(tmp, ".ok"), "w") as f:
        f.write("ok\n")
    shutil.rmtree(out, ignore_errors=True)
    os.replace(tmp, out)


def materialise(src_dir: str, dest: str) -> None:
    """Mirror ``src_dir`` into ``dest`` with hard links, copying where a link is refused (another file system)."""
    for root, _dirs, files in os.walk(src_dir):
        rel = os.path.relpath(root, src_dir)
        tgt = os.path.join(dest, rel) if rel != "." else dest
        os.makedirs(tgt, exist_ok=True)
        for fn in files:
            if rel == "." and fn == ".ok":
                continue
            s, d = os.path.join(root, fn), os.path.join(tgt, fn)
            if os.path.exists(d):
                os.remove(d)
            try:
                os.link(s, d)
            except OSError:
                shutil.copy2(s, d)


def pull_pack(pack: Pack, into_dir: str, force: bool = False) -> str:
    """Makes ``<into_dir>/<dest>`` hold the pack's files; returns that path.  No bytes move when it already does."""
    pack.validate()
    dest = os.path.join(into_dir, pack.dest)
    if not force and pack_status(pack, into_dir) == "linked":
        return dest
    os.makedirs(cache_root(), exist_ok=True)
    arch = archive_path(pack)
    if force or not os.path.isfile(arch) or _sha256_file(arch) != pack.sha256:
        r = resolve_url(pack)
        st, body = _http("GET", r.url, r.headers)
        if st != 200:
            raise RuntimeError(f"pack {pack.ref()}: GET answered {st}")
        if pack.bytes and len(body) != pack.bytes:
            raise RuntimeError(f"pack {pack.ref()}: got {len(body)} bytes, declared {pack.bytes}")
        got = hashlib.sha256(body).hexdigest()
        if got != pack.sha256:
            raise RuntimeError(f"pack {pack.ref()}: sha256 mismatch (got {got})")
        tmp = arch + ".partial"
        with open(tmp, "wb") as f:
            f.write(body)
        os.replace(tmp, arch)
    ex = extract_dir(pack)
    if force or not os.path.isfile(os.path.join(ex, ".ok")):
        _extract(arch, ex)
    materialise(ex, dest)
    with open(os.path.join(dest, ".pack_ok"), "w") as f:
        f.write(f"{pack.ref()} {pack.sha256}\n")
    return dest


def pack_bytes_on_disk(pack: Pack, into_dir: str) -> int:
    total = 0
    for root, _d, files in os.walk(os.path.join(into_dir, pack.dest)):
        for fn in files:
            total += os.path.getsize(os.path.join(root, fn))
    return total
