import http.server
import json
import os
import threading

import numpy as np


def test_npy_png_wav_roundtrip(tmp_path):
    from noeira_b200.io import formats as F
    for a in (np.arange(12, dtype=np.float32).reshape(3, 4), np.array([1, 2, 3], np.int64), np.random.rand(2, 3, 4)):
        F.save_npy(str(tmp_path / "a.npy"), a)
        assert np.array_equal(np.load(str(tmp_path / "a.npy")), a) and np.array_equal(F.load_npy(str(tmp_path / "a.npy")), a)
    np.save(str(tmp_path / "b.npy"), np.eye(3, dtype=np.float64))
    assert np.array_equal(F.load_npy(str(tmp_path / "b.npy")), np.eye(3))
    rng = np.random.default_rng(0)
    for shape in ((9, 7), (5, 6, 3), (4, 4, 4)):
        img = rng.integers(0, 256, shape, dtype=np.uint8)
        F.save_png(str(tmp_path / "i.png"), img)
        assert np.array_equal(F.load_png(str(tmp_path / "i.png")), img)
    t = np.linspace(0, 1, 800, dtype=np.float32)
    F.save_wav(str(tmp_path / "s.wav"), np.sin(2 * np.pi * 440 * t), 8000)
    s, rate = F.load_wav(str(tmp_path / "s.wav"))
    assert rate == 8000 and s.dtype == np.int16 and len(s) == 800 and abs(int(s.max()) - 32767) < 400
    assert F.b64decode(F.b64encode(b"\x00\xffabc")) == b"\x00\xffabc"
    F.write_jsonl(str(tmp_path / "r.jsonl"), [{"a": 1}, {"b": [1, 2]}])
    assert F.read_jsonl(str(tmp_path / "r.jsonl")) == [{"a": 1}, {"b": [1, 2]}]


def test_feetech_bus_against_fake_servo():
    from noeira_b200 import runtime as rt
    from noeira_b200.robot import FeetechBus, decode_packet, encode_packet
    from noeira_b200.robot.feetech import radians_to_ticks, ticks_to_radians
    assert encode_packet(1, 0x01) == bytes([0xFF, 0xFF, 0x01, 0x02, 0x01, 0xFB])
    assert decode_packet(encode_packet(3, 0, [0x10, 0x20])) == (3, 0, b"\x10\x20", 8)
    assert radians_to_ticks(ticks_to_radians(3000)) == 3000
    master, slave = os.openpty()
    mem = {5: bytearray(64)}
    mem[5][56:58] = (1234).to_bytes(2, "little")
    stop = threading.Event()

    def servo():
        buf = b""
        while not stop.is_set():
            try:
                buf += os.read(master, 64)
            except OSError:
                return
            while True:
                r = decode_packet(buf)
                if r is None:
                    break
                sid, instr, params, used = r
                buf = buf[used:]
                if instr == 0x83:                                  # sync write: no reply
                    addr, n = params[0], params[1]
                    for k in range(2, len(params), n + 1):
                        if params[k] in mem:
                            mem[params[k]][addr: addr + n] = params[k + 1: k + 1 + n]
                elif sid in mem:
                    if instr == 0x01:
                        os.write(master, encode_packet(sid, 0))
                    elif instr == 0x02:
                        os.write(master, encode_packet(sid, 0, mem[sid][params[0]: params[0] + params[1]]))
                    elif instr == 0x03:
                        mem[sid][params[0]: params[0] + len(params) - 1] = params[1:]
                        os.write(master, encode_packet(sid, 0))

    th = threading.Thread(target=servo, daemon=True)
    th.start()
    bus = FeetechBus(rt.SerialPort(fd=slave, baud=1000000), timeout_ms=200)
    assert bus.ping(5) and not bus.ping(9)
    assert bus.read_position(5) == 1234
    bus.write(5, 40, [1])
    assert mem[5][40] == 1
    bus.sync_write_positions({5: 2049, 6: 100})
    import time
    for _ in range(100):
        if int.from_bytes(mem[5][42:44], "little") == 2049:
            break
        time.sleep(0.01)
    assert int.from_bytes(mem[5][42:44], "little") == 2049
    stop.set()
    os.close(master)


def test_chat_client_and_sse():
    from noeira_b200.ai import ChatClient, parse_sse
    evs = list(parse_sse("event: a\ndata: 1\ndata: 2\n\n: comment\ndata: x\n\n"))
    assert evs == [{"event": "a", "data": "1\n2"}, {"data": "x"}]

    class H(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            req = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            assert self.headers["Authorization"] == "Bearer k" and req["model"] == "m"
            if req["stream"]:
                body = "".join(f"data: {json.dumps({'choices': [{'delta': {'content': w}}]})}\n\n" for w in ("hel", "lo")) + "data: [DONE]\n\n"
            else:
                body = json.dumps({"choices": [{"message": {"content": req["messages"][-1]["content"].upper()}}]})
            b = body.encode()
            self.send_response(200)
            self.send_header("Content-Length", str(len(b)))
            self.end_headers()
            self.wfile.write(b)

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    c = ChatClient(f"http://127.0.0.1:{srv.server_address[1]}", "m", "k")
    assert c.complete([{"role": "user", "content": "hi"}]) == "HI"
    assert c.complete([{"role": "user", "content": "hi"}], stream=True) == "hello"
    srv.shutdown()
