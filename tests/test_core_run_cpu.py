import http.server
import json
import threading

from noeira_b200 import core


def test_run_context_writes_kv_and_csv(tmp_path):
    with core.RunContext(str(tmp_path), "proj", "ppo", {"lr": 3e-4, "envs": 4096}) as run:
        kv0 = core.read_kv(run.path("run.kv"))
        assert kv0["status"] == "running" and kv0["config.envs"] == 4096
        for s in range(50):
            run.log(s, {"loss": 1.0 / (s + 1), "reward": float(s)})
    kv1 = core.read_kv(run.path("run.kv"))
    assert kv1["status"] == "finished" and kv1["final.reward"] == 49.0 and kv1["duration_s"] >= 0
    rows = open(run.path("metrics.csv")).read().splitlines()
    assert rows[0] == "step,loss,reward" and len(rows) == 51 and rows[-1].startswith("49,0.02,")
    from noeira_b200.core.run import list_runs
    assert [r["run_id"] for r in list_runs(str(tmp_path), "proj")] == [run.run_id]
    try:
        with core.RunContext(str(tmp_path), "proj", "bad", logger=core.NoOpLogger()) as r2:
            raise ValueError("boom")
    except ValueError:
        pass
    assert core.read_kv(r2.path("run.kv"))["status"] == "failed"


def test_remote_and_composite_logger(tmp_path):
    got = []

    class H(http.server.BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = self.rfile.read(int(self.headers["Content-Length"]))
            got.extend(json.loads(l) for l in body.decode().splitlines())
            self.send_response(204)
            self.send_header("Content-Length", "0")
            self.end_headers()

    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    remote = core.RemoteLogger(f"http://127.0.0.1:{srv.server_address[1]}/ingest", "r1", flush_every=4)
    lg = core.CompositeLogger(remote, core.CsvLogger(str(tmp_path / "m.csv")), core.NoOpLogger())
    for s in range(10):
        lg.log(s, {"x": s * 0.5})
    lg.close()
    srv.shutdown()
    assert remote.sent == 10 and remote.failed == 0 and [g["step"] for g in got] == list(range(10)) and got[3]["x"] == 1.5
    dead = core.RemoteLogger("http://127.0.0.1:1/none", flush_every=1, timeout_ms=200)
    dead.log(0, {"x": 1.0})
    assert dead.failed == 1


def test_metrics_and_timer():
    m = core.Metrics()
    m.add("a", 2.0)
    m.add("a", 4.0, n=3)
    assert m.mean("a") == 3.5 and m.last["a"] == 4.0
    t = core.PerfTimer()
    for _ in range(3):
        with t.section("s"):
            sum(range(1000))
    r = t.report()
    assert r["s"]["calls"] == 3 and r["s"]["total_ms"] > 0
