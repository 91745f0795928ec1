"""Asset packs: declaration parsing / validation, and fetch → verify → extract → link against a local HTTP server."""
import hashlib
import http.server
import io
import os
import tarfile
import threading

import pytest


def _tar_bytes(files):
    buf = io.BytesIO()
    with tarfile.open(fileobj=buf, mode="w:gz") as tf:
        for name, data in files.items():
            ti = tarfile.TarInfo(name)
            ti.size = len(data)
            tf.addfile(ti, io.BytesIO(data))
    return buf.getvalue()


def test_parse_and_validate():
    from noeira_b200.assets import parse_packs
    sha = "ab" * 32
    text = f"""schema_version=1

pack=robot@v2
provider=hf
url=https://example.org/robot.tar.gz
sha256={sha}
bytes=10
dest=assets/robot

pack=arm@v1
provider=noeira
id=arm-assets@v1
sha256={sha}
dest=assets/arm
"""
    pf = parse_packs(text)
    assert [p.ref() for p in pf.packs] == ["robot@v2", "arm@v1"]
    assert pf.find("arm").id == "arm-assets@v1" and pf.find("robot@v2").bytes == 10
    assert parse_packs(pf.to_text()).packs == pf.packs
    with pytest.raises(ValueError, match="token_env"):
        parse_packs(text.replace("provider=hf", "provider=hf\ntoken_env=X"))
    with pytest.raises(ValueError, match="dest"):
        parse_packs(text.replace("dest=assets/robot", "dest=../outside"))
    with pytest.raises(ValueError, match="id="):
        parse_packs(text.replace("id=arm-assets@v1\n", ""))
    with pytest.raises(ValueError, match="schema_version"):
        parse_packs(text.replace("schema_version=1", "schema_version=9"))
    with pytest.raises(ValueError, match="before the first"):
        parse_packs("schema_version=1\nurl=https://x\n")


def test_pull_pack_from_local_server(tmp_path, monkeypatch):
    from noeira_b200.assets import Pack, pack_bytes_on_disk, pack_status, pull_pack
    blob = _tar_bytes({"meshes/base.stl": b"solid base" * 10, "textures/skin.png": b"\x89PNG fake"})
    sha = hashlib.sha256(blob).hexdigest()
    hits = {"n": 0, "auth": None}

    class H(http.server.BaseHTTPRequestHandler):
        def do_GET(self):
            hits["n"] += 1
            hits["auth"] = self.headers.get("Authorization")
            self.send_response(200)
            self.send_header("Content-Length", str(len(blob)))
            self.end_headers()
            self.wfile.write(blob)

        def log_message(self, *a):
            pass

    srv = http.server.HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        monkeypatch.setenv("NOEIRA_CACHE", str(tmp_path / "cache"))
        monkeypatch.setenv("MY_TOKEN", "s3cret")
        url = f"http://127.0.0.1:{srv.server_address[1]}/robot.tar.gz"
        pack = Pack(name="robot", version="v1", provider="https", url=url, sha256=sha, bytes=len(blob),
                    dest="assets/robot", token_env="MY_TOKEN")
        proj = str(tmp_path / "proj")
        assert pack_status(pack, proj) == "absent"
        dest = pull_pack(pack, proj)
        assert open(os.path.join(dest, "meshes", "base.stl"), "rb").read() == b"solid base" * 10
        assert hits == {"n": 1, "auth": "Bearer s3cret"}
        assert pack_status(pack, proj) == "linked"
        assert pack_bytes_on_disk(pack, proj) > 100
        pull_pack(pack, proj)                       # idempotent: no second download
        assert hits["n"] == 1
        # a second project shares the cached archive and extraction
        pull_pack(pack, str(tmp_path / "proj2"))
        assert hits["n"] == 1
        # same inode = hard link into the cache
        a = os.stat(os.path.join(dest, "meshes", "base.stl")).st_ino
        b = os.stat(os.path.join(str(tmp_path / "proj2"), "assets/robot/meshes/base.stl")).st_ino
        assert a == b
        bad = Pack(name="robot", version="v2", provider="https", url=url, sha256="0" * 64, dest="assets/r2")
        with pytest.raises(RuntimeError, match="sha256 mismatch"):
            pull_pack(bad, proj)
    finally:
        srv.shutdown()
