"""Model / dataset hub client over the native HTTP(S) client: resolve URLs, cached downloads, listing, upload.

``HubClient(endpoint, token, cache_dir)``:
  ``url(repo, filename, revision, repo_type)``     ``<endpoint>/[datasets/]<repo>/resolve/<revision>/<filename>``
  ``download(repo, filename, ...)``                fetches once into ``<cache>/<repo_type>s--<org>--<name>/<revision>/<filename>`` (atomic
                                                   write, optional SHA-256 check), later calls return the cached path without a request
  ``list_files(repo, ...)``                        file names of a repository (``/api/<type>s/<repo>/tree/<revision>``)
  ``upload(repo, filename, data, ...)``            one file through the commit endpoint (JSON lines: header + base64 file)
  ``snapshot(repo, patterns)``                     every file that matches one of the glob patterns
The endpoint defaults to ``$HF_ENDPOINT`` or ``https://huggingface.co``; the token to ``$HF_TOKEN``.
(noeira/io: HF hub client / push over libcurl; here the C++ socket + OpenSSL client of ``csrc/host/http.cpp``.)
"""
from __future__ import annotations

import fnmatch
import hashlib
import json
import os
from typing import List, Optional, Sequence

from ..runtime.host import http_request, write_file_atomic


class HubError(RuntimeError):
    pass


class HubClient:
    def __init__(self, endpoint: str = None, token: str = None, cache_dir: str = None, timeout_ms: int = 60000):
        self.endpoint = (endpoint or os.environ.get("HF_ENDPOINT") or "https://huggingface.co").rstrip("/")
        self.token = token if token is not None else os.environ.get("HF_TOKEN")
        self.cache_dir = cache_dir or os.path.join(os.path.expanduser("~"), ".cache", "noeira_b200", "hub")
        self.timeout_ms = timeout_ms
        self.requests = 0

    def _headers(self, extra=None):
        h = {"User-Agent": "noeira_b200"}
        if self.token:
            h["Authorization"] = f"Bearer {self.token}"
        h.update(extra or {})
        return h

    def _get(self, url):
        self.requests += 1
        st, body = http_request("GET", url, self._headers(), timeout_ms=self.timeout_ms)
        if st != 200:
            raise HubError(f"GET {url}: HTTP {st}")
        return body

    @staticmethod
    def _prefix(repo_type):
        return {"model": "", "dataset": "datasets/", "space": "spaces/"}[repo_type]

    def url(self, repo: str, filename: str, revision: str = "main", repo_type: str = "model") -> str:
        return f"{self.endpoint}/{self._prefix(repo_type)}{repo}/resolve/{revision}/{filename}"

    def cached_path(self, repo, filename, revision="main", repo_type="model") -> str:
        return os.path.join(self.cache_dir, f"{repo_type}s--" + repo.replace("/", "--"), revision, *filename.split("/"))

    def download(self, repo: str, filename: str, revision: str = "main", repo_type: str = "model", sha256: Optional[str] = None,
                 force: bool = False) -> str:
        path = self.cached_path(repo, filename, revision, repo_type)
        if os.path.exists(path) and not force:
            return path
        body = self._get(self.url(repo, filename, revision, repo_type))
        if sha256 is not None and hashlib.sha256(body).hexdigest() != sha256.lower():
            raise HubError(f"{repo}/{filename}: SHA-256 mismatch")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        write_file_atomic(path, [body])
        return path

    def list_files(self, repo: str, revision: str = "main", repo_type: str = "model") -> List[str]:
        body = self._get(f"{self.endpoint}/api/{repo_type}s/{repo}/tree/{revision}?recursive=true")
        return sorted(e["path"] for e in json.loads(body) if e.get("type", "file") == "file")

    def snapshot(self, repo: str, patterns: Sequence[str] = ("*",), revision: str = "main", repo_type: str = "model") -> List[str]:
        names = [n for n in self.list_files(repo, revision, repo_type) if any(fnmatch.fnmatch(n, p) for p in patterns)]
        return [self.download(repo, n, revision, repo_type) for n in names]

    def upload(self, repo: str, filename: str, data: bytes, message: str = "upload", revision: str = "main", repo_type: str = "model"):
        """One small file through the commit endpoint (newline-delimited JSON: a header object, then one file object)."""
        import base64
        lines = [json.dumps({"key": "header", "value": {"summary": message}}),
                 json.dumps({"key": "file", "value": {"path": filename, "encoding": "base64", "content": base64.b64encode(data).decode()}})]
        self.requests += 1
        st, body = http_request("POST", f"{self.endpoint}/api/{repo_type}s/{repo}/commit/{revision}",
                                self._headers({"Content-Type": "application/x-ndjson"}), ("\n".join(lines) + "\n").encode(),
                                timeout_ms=self.timeout_ms)
        if st not in (200, 201):
            raise HubError(f"upload {repo}/{filename}: HTTP {st}")
        return json.loads(body) if body else {}
