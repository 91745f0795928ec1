"""Hosted-model chat client (OpenAI-compatible ``/v1/chat/completions`` JSON) and a server-sent-events parser, over the
native HTTP client.  ``http://`` endpoints only (a local gateway): the image has no TLS library.
(Reference: noeira/ai/ chat clients + SSE parser.)"""
from __future__ import annotations

import json
from typing import Dict, Iterator, List, Optional

from ..runtime import http_request


def parse_sse(stream: str) -> Iterator[Dict[str, str]]:
    """Events separated by blank lines; ``data:`` lines of one event are joined with newlines; comments (``:``) skipped."""
    ev: Dict[str, List[str]] = {}
    for line in stream.replace("\r\n", "\n").split("\n"):
        if line == "":
            if ev:
                yield {k: "\n".join(v) for k, v in ev.items()}
                ev = {}
            continue
        if line.startswith(":"):
            continue
        k, _, v = line.partition(":")
        ev.setdefault(k, []).append(v[1:] if v.startswith(" ") else v)
    if ev:
        yield {k: "\n".join(v) for k, v in ev.items()}


class ChatClient:
    def __init__(self, base_url: str, model: str, api_key: Optional[str] = None, timeout_ms: int = 30000):
        self.base_url, self.model, self.api_key, self.timeout_ms = base_url.rstrip("/"), model, api_key, timeout_ms

    def _headers(self):
        h = {"Content-Type": "application/json"}
        if self.api_key:
            h["Authorization"] = f"Bearer {self.api_key}"
        return h

    def complete(self, messages: List[Dict[str, str]], stream: bool = False, **params) -> str:
        body = json.dumps({"model": self.model, "messages": messages, "stream": stream, **params}).encode()
        status, data = http_request("POST", self.base_url + "/v1/chat/completions", self._headers(), body, self.timeout_ms)
        if status != 200:
            raise IOError(f"chat endpoint returned {status}: {data[:200]!r}")
        if not stream:
            return json.loads(data)["choices"][0]["message"]["content"]
        out = []
        for ev in parse_sse(data.decode()):
            d = ev.get("data", "")
            if d == "[DONE]":
                break
            delta = json.loads(d)["choices"][0].get("delta", {})
            out.append(delta.get("content", ""))
        return "".join(out)
