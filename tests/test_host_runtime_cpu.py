"""Host C++ runtime: ring + sink thread, serial over a pty pair, HTTP against a local server, hull, file IO, loader."""
import gzip
import hashlib
import http.server
import os
import threading

import numpy as np
import pytest

from noeira_b200 import runtime as rt


def test_ring_and_filesink(tmp_path):
    r = rt.SpscRing(1 << 12)
    assert r.pop() is None
    msgs = [bytes([i % 251]) * (1 + i % 97) for i in range(200)]
    got = []

    def consumer():
        while len(got) < len(msgs):
            m = r.pop()
            if m is not None:
                got.append(m)

    t = threading.Thread(target=consumer)
    t.start()
    for m in msgs:
        while not r.push(m):
            pass
    t.join(10)
    assert got == msgs
    r.close()
    sink = rt.FileSink(str(tmp_path / "log.csv"))
    for i in range(1000):
        sink.write(f"{i},{i * i}\n".encode())
    assert sink.close() == 1000
    lines = (tmp_path / "log.csv").read_text().splitlines()
    assert len(lines) == 1000 and lines[999] == "999,998001"


def test_serial_over_pty():
    master, slave = os.openpty()
    port = rt.SerialPort(fd=slave, baud=115200)
    os.write(master, b"\xff\xff\x01\x02\x03")
    assert port.read(5, 500) == b"\xff\xff\x01\x02\x03"
    port.write(b"\x0a\x0d\x00ping")          # raw mode: no newline translation, NUL passes
    assert os.read(master, 16) == b"\x0a\x0d\x00ping"
    assert port.read(4, 50) == b""            # timeout returns what arrived
    port.close()
    os.close(master)
    with pytest.raises(OSError):
        rt.SerialPort("/dev/nonexistent-tty", 115200)


class _H(http.server.BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, *a):
        pass

    def do_GET(self):
        if self.path == "/gz":
            body = gzip.compress(b"hello " * 1000)
            self.send_response(200)
            self.send_header("Content-Encoding", "gzip")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)
        elif self.path == "/chunked":
            self.send_response(200)
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()
            for part in (b"abc", b"defgh", b"i" * 300):
                self.wfile.write(b"%x\r\n%s\r\n" % (len(part), part))
            self.wfile.write(b"0\r\n\r\n")
        else:
            self.send_response(404)
            self.send_header("Content-Length", "0")
            self.end_headers()

    def do_POST(self):
        n = int(self.headers["Content-Length"])
        data = self.rfile.read(n)
        out = data[::-1] + self.headers.get("X-Tag", "").encode()
        self.send_response(201)
        self.send_header("Content-Length", str(len(out)))
        self.end_headers()
        self.wfile.write(out)


def test_http_client_local_server():
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{srv.server_address[1]}"
    try:
        assert rt.http_request("GET", base + "/gz") == (200, b"hello " * 1000)
        assert rt.http_request("GET", base + "/chunked") == (200, b"abcdefgh" + b"i" * 300)
        assert rt.http_request("GET", base + "/nope")[0] == 404
        assert rt.http_request("POST", base + "/p", {"X-Tag": "t1"}, b"12345") == (201, b"54321t1")
        with pytest.raises(OSError):
            rt.http_request("GET", "https://127.0.0.1:9/")          # nothing listens there
    finally:
        srv.shutdown()
    assert rt.gzip_inflate(gzip.compress(b"xyz" * 50)) == b"xyz" * 50


def _self_signed(tmp_path, host="localhost"):
    import datetime
    import ipaddress
    from cryptography import x509
    from cryptography.hazmat.primitives import hashes, serialization
    from cryptography.hazmat.primitives.asymmetric import rsa
    from cryptography.x509.oid import NameOID
    key = rsa.generate_private_key(public_exponent=65537, key_size=2048)
    name = x509.Name([x509.NameAttribute(NameOID.COMMON_NAME, host)])
    now = datetime.datetime.now(datetime.timezone.utc)
    cert = (x509.CertificateBuilder().subject_name(name).issuer_name(name).public_key(key.public_key())
            .serial_number(x509.random_serial_number()).not_valid_before(now - datetime.timedelta(days=1))
            .not_valid_after(now + datetime.timedelta(days=2))
            .add_extension(x509.SubjectAlternativeName([x509.DNSName(host), x509.IPAddress(ipaddress.ip_address("127.0.0.1"))]), False)
            .add_extension(x509.BasicConstraints(ca=True, path_length=None), True).sign(key, hashes.SHA256()))
    cp, kp = str(tmp_path / "cert.pem"), str(tmp_path / "key.pem")
    open(cp, "wb").write(cert.public_bytes(serialization.Encoding.PEM))
    open(kp, "wb").write(key.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.TraditionalOpenSSL,
                                           serialization.NoEncryption()))
    return cp, kp


def test_https_client_verifies_the_server_certificate(tmp_path, monkeypatch):
    import ssl
    cp, kp = _self_signed(tmp_path)
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _H)
    ctx = ssl.SSLContext(ssl.PROTOCOL_TLS_SERVER)
    ctx.load_cert_chain(cp, kp)
    srv.socket = ctx.wrap_socket(srv.socket, server_side=True)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    base = f"https://127.0.0.1:{srv.server_address[1]}"
    try:
        monkeypatch.delenv("NOEIRA_TLS_INSECURE", raising=False)
        monkeypatch.delenv("NOEIRA_TLS_CA_FILE", raising=False)
        with pytest.raises(OSError):                                   # unknown issuer: refused
            rt.http_request("GET", base + "/gz")
        monkeypatch.setenv("NOEIRA_TLS_CA_FILE", cp)                    # trusted explicitly: verified, host name matches the SAN
        assert rt.http_request("GET", base + "/gz") == (200, b"hello " * 1000)
        assert rt.http_request("POST", base + "/p", {"X-Tag": "t2"}, b"abc") == (201, b"cbat2")
        monkeypatch.delenv("NOEIRA_TLS_CA_FILE")
        monkeypatch.setenv("NOEIRA_TLS_INSECURE", "1")
        assert rt.http_request("GET", base + "/chunked") == (200, b"abcdefgh" + b"i" * 300)
    finally:
        srv.shutdown()


def test_convex_hull_cube_and_random():
    cube = np.array([[x, y, z] for x in (0, 1) for y in (0, 1) for z in (0, 1)], dtype=float)
    pts = np.vstack([cube, np.random.default_rng(0).uniform(0.1, 0.9, (50, 3))])
    tri = rt.convex_hull(pts)
    assert len(tri) == 12 and set(tri.flatten()) == set(range(8))
    # closed, outward: volume from signed tetrahedra = 1, every point behind every face
    vol = sum(np.dot(pts[a], np.cross(pts[b], pts[c])) for a, b, c in tri) / 6
    assert abs(vol - 1.0) < 1e-9
    rng = np.random.default_rng(1)
    p = rng.normal(size=(300, 3))
    tri = rt.convex_hull(p)
    for a, b, c in tri:
        n = np.cross(p[b] - p[a], p[c] - p[a])
        assert ((p - p[a]) @ n).max() < 1e-7
    V, F = len(set(tri.flatten())), len(tri)
    assert V - 3 * F // 2 + F == 2            # Euler characteristic of a closed triangulated surface
    with pytest.raises(OSError):
        rt.convex_hull(np.zeros((10, 3)))


def test_file_io_and_sha256(tmp_path):
    a, b = os.urandom(100_003), np.arange(1000, dtype=np.float32)
    path = str(tmp_path / "blob.bin")
    rt.write_file_atomic(path, [a, b])
    raw = open(path, "rb").read()
    assert raw == a + b.tobytes()
    assert rt.read_file_range(path, 100_003 + 8, 8) == b[2:4].tobytes()
    assert not [f for f in os.listdir(tmp_path) if ".tmp." in f]
    for msg in (b"", b"abc", os.urandom(55), os.urandom(56), os.urandom(64), os.urandom(1000)):
        assert rt.sha256(msg) == hashlib.sha256(msg).hexdigest()


def test_record_loader_epochs(tmp_path):
    n, rec = 1000, 24
    data = np.arange(n * rec // 4, dtype=np.int32).reshape(n, rec // 4)
    path = str(tmp_path / "records.bin")
    with open(path, "wb") as f:
        f.write(b"HDR!" * 4)
        f.write(data.tobytes())
    ld = rt.RecordLoader(path, rec, n, batch=64, header_bytes=16, slots=3, threads=3, seed=5, shuffle=True, drop_last=False)
    out = np.zeros((64, rec // 4), dtype=np.int32)
    seen, order0 = [], []
    while True:
        cnt, idx = ld.next_into(out)
        if cnt == 0:
            break
        assert (out[:cnt] == data[idx.astype(np.int64)]).all()
        seen.extend(idx.tolist())
        order0.extend(idx.tolist())
    assert sorted(seen) == list(range(n)) and seen != list(range(n))
    ld.reset(0)
    again = []
    while True:
        cnt, idx = ld.next_into(out)
        if cnt == 0:
            break
        again.extend(idx.tolist())
    assert again == order0                     # same (seed, epoch) → same order
    ld.reset(1)
    cnt, idx = ld.next_into(out)
    assert idx.tolist() != order0[:64]
    ld.close()


def test_record_loader_reset_mid_epoch(tmp_path):
    """Abandon an epoch after one batch while the readers are still filling slots: every record delivered in the
    next epoch must match its index (no buffer is written by a reader of the old epoch)."""
    n, rec = 4096, 512
    data = np.arange(n * rec // 4, dtype=np.int32).reshape(n, rec // 4)
    path = str(tmp_path / "records.bin")
    with open(path, "wb") as f:
        f.write(data.tobytes())
    ld = rt.RecordLoader(path, rec, n, batch=256, slots=4, threads=4, seed=9, shuffle=True, drop_last=True)
    out = np.zeros((256, rec // 4), dtype=np.int32)
    for epoch in range(1, 30):
        cnt, idx = ld.next_into(out)
        assert cnt == 256 and (out == data[idx.astype(np.int64)]).all()
        ld.reset(epoch)
        for _ in range(2):
            cnt, idx = ld.next_into(out)
            assert cnt == 256 and (out == data[idx.astype(np.int64)]).all(), epoch
    ld.close()
