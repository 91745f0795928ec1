"""Hub client against a local HTTP server that speaks the hub's URL layout (no network)."""
import base64
import hashlib
import http.server
import json
import threading

import pytest

FILES = {"config.json": b'{"hidden": 512}', "model.safetensors": bytes(range(256)) * 40, "data/train-00000.parquet": b"PAR1....PAR1"}
SEEN = {"auth": [], "uploads": []}


class _Handler(http.server.BaseHTTPRequestHandler):
    def log_message(self, *a):
        pass

    def do_GET(self):
        SEEN["auth"].append(self.headers.get("Authorization"))
        if self.path.startswith("/api/models/org/demo/tree/main"):
            body = json.dumps([{"type": "file", "path": p} for p in FILES] + [{"type": "directory", "path": "data"}]).encode()
        elif self.path.startswith("/org/demo/resolve/main/") and self.path[len("/org/demo/resolve/main/"):] in FILES:
            body = FILES[self.path[len("/org/demo/resolve/main/"):]]
        elif self.path.startswith("/datasets/org/ds/resolve/v1/readme.md"):
            body = b"dataset card"
        else:
            self.send_response(404)
            self.end_headers()
            return
        self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_POST(self):
        n = int(self.headers.get("Content-Length", "0"))
        SEEN["uploads"].append((self.path, self.rfile.read(n)))
        body = b'{"commitOid": "abc"}'
        self.send_response(200)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)


def test_download_cache_listing_snapshot_upload(tmp_path):
    from noeira_b200.io.hub import HubClient, HubError
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        hub = HubClient(f"http://127.0.0.1:{srv.server_address[1]}", token="secret", cache_dir=str(tmp_path / "cache"))
        assert hub.url("org/demo", "config.json") == f"{hub.endpoint}/org/demo/resolve/main/config.json"
        assert hub.url("org/ds", "a.parquet", "v1", "dataset").endswith("/datasets/org/ds/resolve/v1/a.parquet")
        p = hub.download("org/demo", "model.safetensors", sha256=hashlib.sha256(FILES["model.safetensors"]).hexdigest())
        assert open(p, "rb").read() == FILES["model.safetensors"] and "models--org--demo" in p and SEEN["auth"][-1] == "Bearer secret"
        n = hub.requests
        assert hub.download("org/demo", "model.safetensors") == p and hub.requests == n          # served from the cache
        with pytest.raises(HubError):
            hub.download("org/demo", "config.json", sha256="00" * 32)
        with pytest.raises(HubError):
            hub.download("org/demo", "missing.bin")
        assert hub.list_files("org/demo") == sorted(FILES)
        got = hub.snapshot("org/demo", patterns=["*.json", "data/*"])
        assert [g.split("main/")[1] for g in got] == ["config.json", "data/train-00000.parquet"]
        assert open(hub.download("org/ds", "readme.md", "v1", "dataset"), "rb").read() == b"dataset card"
        out = hub.upload("org/demo", "eval/results.json", b'{"success": 0.9}', message="results")
        assert out == {"commitOid": "abc"}
        path, body = SEEN["uploads"][-1]
        lines = [json.loads(x) for x in body.decode().splitlines()]
        assert path == "/api/models/org/demo/commit/main" and lines[0]["value"]["summary"] == "results"
        assert base64.b64decode(lines[1]["value"]["content"]) == b'{"success": 0.9}' and lines[1]["value"]["path"] == "eval/results.json"
    finally:
        srv.shutdown()
