"""Run registry, key-value run files, loggers, metrics and timers.

``RunContext(root, project, name)`` creates ``<root>/<project>/<run id>/`` and writes ``run.kv`` immediately (status
``running``, start time, config) and again at close (status, end time, final metrics), so that a crashed run still
leaves a record (noeira/core/run.mojo:1-40).  ``Logger`` implementations: ``NoOpLogger``, ``CsvLogger`` (rows go
through the native SPSC ring + sink thread, the training loop never blocks on the file system), ``RemoteLogger``
(JSON lines POSTed with the native HTTP client, buffered), ``CompositeLogger`` (noeira/core/logger.mojo).
``Metrics`` keeps running sums / counts and last values (metrics.mojo); ``PerfTimer`` accumulates named wall-clock
or CUDA-event sections (perf_timer.mojo).
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional


# ------------------------------------------------------------------------------------------ kv files
def write_kv(path: str, d: Dict[str, object]):
    """``key = value`` lines, keys sorted; values are JSON scalars / lists so the file round-trips."""
    from ..runtime import write_file_atomic
    text = "".join(f"{k} = {json.dumps(d[k])}\n" for k in sorted(d))
    write_file_atomic(path, [text.encode()])


def read_kv(path: str) -> Dict[str, object]:
    out = {}
    for ln in open(path, encoding="utf-8"):
        ln = ln.strip()
        if not ln or ln.startswith("#") or "=" not in ln:
            continue
        k, v = ln.split("=", 1)
        try:
            out[k.strip()] = json.loads(v.strip())
        except json.JSONDecodeError:
            out[k.strip()] = v.strip()
    return out


# ------------------------------------------------------------------------------------------ loggers
class Logger:
    def log(self, step: int, values: Dict[str, float]):
        raise NotImplementedError

    def close(self):
        pass


class NoOpLogger(Logger):
    def log(self, step, values):
        pass


class CsvLogger(Logger):
    """Columns are fixed by the first row; later rows fill missing keys with an empty cell."""

    def __init__(self, path: str):
        from ..runtime import FileSink
        self.path, self.cols = path, None
        self.sink = FileSink(path)

    def log(self, step, values):
        if self.cols is None:
            self.cols = sorted(values)
            self.sink.write(("step," + ",".join(self.cols) + "\n").encode())
        row = [str(step)] + ["" if values.get(c) is None else repr(float(values[c])) for c in self.cols]
        self.sink.write((",".join(row) + "\n").encode())

    def close(self):
        if self.sink is not None:
            self.sink.close()
            self.sink = None


class RemoteLogger(Logger):
    """Buffers rows and POSTs them as JSON lines to ``url`` every ``flush_every`` rows; failures are counted, never raised
    (a logging endpoint that is down must not stop training)."""

    def __init__(self, url: str, run_id: str = "", flush_every: int = 20, timeout_ms: int = 2000):
        self.url, self.run_id, self.flush_every, self.timeout_ms = url, run_id, flush_every, timeout_ms
        self.buf: List[str] = []
        self.sent = self.failed = 0

    def log(self, step, values):
        self.buf.append(json.dumps({"run": self.run_id, "step": step, **{k: float(v) for k, v in values.items()}}))
        if len(self.buf) >= self.flush_every:
            self.flush()

    def flush(self):
        if not self.buf:
            return
        from ..runtime import http_request
        body = ("\n".join(self.buf) + "\n").encode()
        try:
            st, _ = http_request("POST", self.url, {"Content-Type": "application/x-ndjson"}, body, self.timeout_ms)
            if 200 <= st < 300:
                self.sent += len(self.buf)
            else:
                self.failed += len(self.buf)
        except OSError:
            self.failed += len(self.buf)
        self.buf = []

    def close(self):
        self.flush()


class CompositeLogger(Logger):
    def __init__(self, *loggers: Logger):
        self.loggers = list(loggers)

    def log(self, step, values):
        for lg in self.loggers:
            lg.log(step, values)

    def close(self):
        for lg in self.loggers:
            lg.close()


# ------------------------------------------------------------------------------------------ metrics / timers
class Metrics:
    def __init__(self):
        self.sum: Dict[str, float] = {}
        self.count: Dict[str, int] = {}
        self.last: Dict[str, float] = {}

    def add(self, name: str, value: float, n: int = 1):
        self.sum[name] = self.sum.get(name, 0.0) + float(value) * n
        self.count[name] = self.count.get(name, 0) + n
        self.last[name] = float(value)

    def mean(self, name: str) -> float:
        return self.sum[name] / max(self.count[name], 1)

    def means(self) -> Dict[str, float]:
        return {k: self.mean(k) for k in self.sum}

    def reset(self):
        self.sum.clear()
        self.count.clear()


class PerfTimer:
    """``with timer.section("update"): …`` — wall clock by default, CUDA events when ``cuda=True`` (read at ``report``)."""

    def __init__(self, cuda: bool = False):
        self.cuda = cuda
        self.total: Dict[str, float] = {}
        self.calls: Dict[str, int] = {}
        self._pending = []

    class _Section:
        def __init__(self, timer, name):
            self.t, self.name = timer, name

        def __enter__(self):
            from ..utils.trace import nvtx_range
            self._nv = nvtx_range(self.name).__enter__()
            if self.t.cuda:
                import torch
                self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.e0.record()
            else:
                self.t0 = time.perf_counter()
            return self

        def __exit__(self, *exc):
            self._nv.__exit__(*exc)
            if self.t.cuda:
                self.e1.record()
                self.t._pending.append((self.name, self.e0, self.e1))
            else:
                self.t._add(self.name, (time.perf_counter() - self.t0) * 1e3)
            return False

    def section(self, name: str):
        return PerfTimer._Section(self, name)

    def _add(self, name, ms):
        self.total[name] = self.total.get(name, 0.0) + ms
        self.calls[name] = self.calls.get(name, 0) + 1

    def report(self) -> Dict[str, Dict[str, float]]:
        if self._pending:
            import torch
            torch.cuda.synchronize()
            for name, e0, e1 in self._pending:
                self._add(name, e0.elapsed_time(e1))
            self._pending = []
        return {k: {"total_ms": self.total[k], "calls": self.calls[k], "mean_ms": self.total[k] / self.calls[k]} for k in self.total}


# ------------------------------------------------------------------------------------------ runs
class RunContext:
    def __init__(self, root: str, project: str, name: str = "run", config: Optional[dict] = None, logger: Logger = None):
        self.project, self.name = project, name
        self.run_id = f"{name}-{time.strftime('%Y%m%d-%H%M%S')}-{os.getpid()}"
        self.dir = os.path.join(root, project, self.run_id)
        os.makedirs(self.dir, exist_ok=True)
        self.config = dict(config or {})
        self.t0 = time.time()
        self.kv = {"run_id": self.run_id, "project": project, "name": name, "status": "running", "start_time": self.t0,
                   **{f"config.{k}": v for k, v in self.config.items()}}
        write_kv(self.path("run.kv"), self.kv)
        self.logger = logger if logger is not None else CsvLogger(self.path("metrics.csv"))
        self.metrics = Metrics()

    def path(self, *parts) -> str:
        return os.path.join(self.dir, *parts)

    def log(self, step: int, values: Dict[str, float]):
        for k, v in values.items():
            self.metrics.add(k, v)
        self.logger.log(step, values)

    def close(self, status: str = "finished", **final):
        self.logger.close()
        self.kv.update({"status": status, "end_time": time.time(), "duration_s": time.time() - self.t0,
                        **{f"final.{k}": v for k, v in {**self.metrics.last, **final}.items()}})
        write_kv(self.path("run.kv"), self.kv)

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        self.close("failed" if et is not None else "finished")
        return False


def list_runs(root: str, project: str) -> List[dict]:
    base = os.path.join(root, project)
    out = []
    for d in sorted(os.listdir(base)) if os.path.isdir(base) else []:
        kv = os.path.join(base, d, "run.kv")
        if os.path.exists(kv):
            out.append(read_kv(kv))
    return out
