"""``assets.kv``: a flat key=value file in which every ``pack=`` line opens a record and the keys after it belong to
that record, so one file describes several packs without nesting.

    schema_version=1

    pack=unitree_g1@v1
    provider=hf
    url=https://huggingface.co/datasets/Org/assets/resolve/main/unitree_g1.tar.gz
    sha256=9f1c...
    bytes=19923456
    dest=assets/unitree_g1

``provider`` names the ACCESS PATTERN (which credential, if any, goes where), not a URL scheme:
``https`` = plain GET of ``url`` (optionally a bearer token from the variable named by ``token_env``), ``hf`` = GET of
``url`` with ``HF_TOKEN`` as the bearer, ``noeira`` = ``id`` is looked up in the catalog service with
``NOEIRA_CLOUD_API_KEY`` and the answer is a presigned URL that is fetched WITHOUT any credential.
Reference: noeira/assets/pack.mojo:67-267.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass, field
from typing import List

SCHEMA_VERSION = "1"
PROVIDER_HTTPS = "https"
PROVIDER_HF = "hf"
PROVIDER_NOEIRA = "noeira"
_PROVIDERS = (PROVIDER_HTTPS, PROVIDER_HF, PROVIDER_NOEIRA)
_KEYS = ("provider", "url", "id", "sha256", "bytes", "dest", "token_env")


@dataclass
class Pack:
    name: str = ""
    version: str = ""
    provider: str = PROVIDER_HTTPS
    url: str = ""
    id: str = ""
    sha256: str = ""
    bytes: int = 0
    dest: str = ""
    token_env: str = ""

    def ref(self) -> str:
        return f"{self.name}@{self.version}" if self.version else self.name

    def validate(self) -> None:
        what = f"pack {self.ref()!r}"
        if not self.name or not re.fullmatch(r"[A-Za-z0-9_.-]+", self.name):
            raise ValueError(f"{what}: bad name")
        if self.provider not in _PROVIDERS:
            raise ValueError(f"{what}: provider must be one of {_PROVIDERS}, got {self.provider!r}")
        if self.provider == PROVIDER_NOEIRA:
            if not self.id:
                raise ValueError(f"{what}: provider=noeira needs id=")
            if self.url:
                raise ValueError(f"{what}: provider=noeira takes id=, not url= (the URL is presigned per request)")
        else:
            if not self.url.startswith(("https://", "http://")):
                raise ValueError(f"{what}: provider={self.provider} needs an http(s) url=")
            if self.id:
                raise ValueError(f"{what}: id= belongs to provider=noeira")
        if self.token_env and self.provider != PROVIDER_HTTPS:
            raise ValueError(f"{what}: token_env= is only for provider=https (the other providers choose their secret)")
        if not re.fullmatch(r"[0-9a-f]{64}", self.sha256):
            raise ValueError(f"{what}: sha256 must be 64 lower-case hex digits")
        if self.bytes < 0:
            raise ValueError(f"{what}: bytes must be >= 0")
        if not self.dest or os.path.isabs(self.dest) or ".." in self.dest.replace("\\", "/").split("/"):
            raise ValueError(f"{what}: dest must be a relative path inside the project")


@dataclass
class PackFile:
    dir: str = ""
    packs: List[Pack] = field(default_factory=list)

    def find(self, ref: str) -> Pack:
        for p in self.packs:
            if p.ref() == ref or p.name == ref:
                return p
        raise KeyError(f"no pack {ref!r} (have {[p.ref() for p in self.packs]})")

    def to_text(self) -> str:
        out = [f"schema_version={SCHEMA_VERSION}", ""]
        for p in self.packs:
            out.append(f"pack={p.ref()}")
            for k in _KEYS:
                v = getattr(p, k)
                if v not in ("", 0) or k == "provider":
                    out.append(f"{k}={v}")
            out.append("")
        return "\n".join(out)


def parse_packs(text: str, what: str = "<text>", dir: str = "") -> PackFile:
    pf = PackFile(dir=dir)
    cur = None
    seen_schema = False
    for ln, raw in enumerate(text.splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        if "=" not in line:
            raise ValueError(f"{what}:{ln}: expected key=value, got {raw!r}")
        key, val = (s.strip() for s in line.split("=", 1))
        if key == "schema_version":
            if val != SCHEMA_VERSION:
                raise ValueError(f"{what}:{ln}: schema_version {val!r} is not supported (this reader: {SCHEMA_VERSION})")
            seen_schema = True
        elif key == "pack":
            name, _, ver = val.partition("@")
            cur = Pack(name=name, version=ver)
            pf.packs.append(cur)
        elif key in _KEYS:
            if cur is None:
                raise ValueError(f"{what}:{ln}: {key}= before the first pack= line")
            setattr(cur, key, int(val) if key == "bytes" else val)
        else:
            raise ValueError(f"{what}:{ln}: unknown key {key!r}")
    if not seen_schema:
        raise ValueError(f"{what}: missing schema_version=")
    names = set()
    for p in pf.packs:
        p.validate()
        if p.ref() in names:
            raise ValueError(f"{what}: pack {p.ref()!r} declared twice")
        names.add(p.ref())
    return pf


def load_packs(path: str) -> PackFile:
    with open(path, "r", encoding="utf-8") as f:
        return parse_packs(f.read(), path, os.path.dirname(os.path.abspath(path)))
