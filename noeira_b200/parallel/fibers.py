"""RankFibers: run N ranks of a step function as threads of ONE process with deterministic collectives.

This is the bit-exact simulator used by the distributed gates (the reference's shared-context backend,
noeira/nn/distributed/process_group.mojo:15-21,379-393, and RankFibers, fibers.mojo:328-382): every collective is
a rendezvous; the last rank to arrive performs the operation for all ranks, reducing in rank order 0..N-1, so
results are reproducible and identical on every rank.  Failure semantics mirror the reference's: a rank that
raises, or a rank that reaches a different collective (or none) while the others wait, turns into an error on
EVERY rank instead of a hang (fibers.mojo:44-49,204-231).
"""
from __future__ import annotations

import threading
from typing import Callable, List

import torch


class CollectiveMismatch(RuntimeError):
    pass


class RankFailed(RuntimeError):
    pass


class ThreadComm:
    """Per-rank handle; all handles of a group share one ``_Hub``."""

    def __init__(self, hub, rank):
        self.hub, self.rank, self.world = hub, rank, hub.n

    def all_reduce(self, t: torch.Tensor):
        self.hub.rendezvous(self.rank, "all_reduce", t)

    def reduce_scatter(self, out: torch.Tensor, inp: torch.Tensor):
        self.hub.rendezvous(self.rank, "reduce_scatter", (out, inp))

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor):
        self.hub.rendezvous(self.rank, "all_gather", (out, inp))

    def broadcast(self, t: torch.Tensor, src: int = 0):
        self.hub.rendezvous(self.rank, f"broadcast{src}", t)

    def barrier(self):
        self.hub.rendezvous(self.rank, "barrier", None)


class _Hub:
    def __init__(self, n, timeout):
        self.n, self.timeout = n, timeout
        self.cv = threading.Condition()
        self.slots = [None] * n
        self.arrived = 0
        self.gen = 0
        self.error = None
        self.done_ranks = 0

    def fail(self, err):
        with self.cv:
            if self.error is None:
                self.error = err
            self.cv.notify_all()

    def depart(self):
        with self.cv:
            self.done_ranks += 1
            if self.arrived > 0 and self.arrived + self.done_ranks >= self.n and self.error is None:
                self.error = CollectiveMismatch("a rank finished while others wait in a collective")
            self.cv.notify_all()

    def rendezvous(self, rank, op, payload):
        with self.cv:
            if self.error is not None:
                raise RankFailed(str(self.error))
            gen = self.gen
            self.slots[rank] = (op, payload)
            self.arrived += 1
            if self.arrived + self.done_ranks >= self.n and self.arrived < self.n:
                self.error = CollectiveMismatch("a rank finished while others wait in a collective")
                self.cv.notify_all()
                raise RankFailed(str(self.error))
            if self.arrived == self.n:
                ops = {s[0] for s in self.slots}
                if len(ops) != 1:
                    self.error = CollectiveMismatch(f"ranks disagree on the collective: {sorted(ops)}")
                else:
                    try:
                        self._execute(op)
                    except Exception as e:  # noqa: BLE001
                        self.error = e
                self.arrived = 0
                self.slots = [None] * self.n
                self.gen += 1
                self.cv.notify_all()
            else:
                ok = self.cv.wait_for(lambda: self.gen != gen or self.error is not None, timeout=self.timeout)
                if not ok and self.error is None:
                    self.error = CollectiveMismatch(f"rank {rank} waited {self.timeout}s in {op}: a peer never arrived")
                    self.cv.notify_all()
            if self.error is not None:
                raise RankFailed(str(self.error))

    def _execute(self, op):
        p = [s[1] for s in self.slots]
        with torch.no_grad():
            if op == "all_reduce":
                acc = p[0].clone()
                for r in range(1, self.n):
                    acc += p[r]
                for r in range(self.n):
                    p[r].copy_(acc)
            elif op == "reduce_scatter":
                k = p[0][0].numel()
                for dst in range(self.n):
                    acc = p[0][1].reshape(-1)[dst * k:(dst + 1) * k].clone()
                    for r in range(1, self.n):
                        acc += p[r][1].reshape(-1)[dst * k:(dst + 1) * k]
                    p[dst][0].reshape(-1).copy_(acc)
            elif op == "all_gather":
                k = p[0][1].numel()
                for dst in range(self.n):
                    for r in range(self.n):
                        p[dst][0].reshape(-1)[r * k:(r + 1) * k].copy_(p[r][1].reshape(-1))
            elif op.startswith("broadcast"):
                src = int(op[len("broadcast"):])
                for r in range(self.n):
                    if r != src:
                        p[r].copy_(p[src])
            elif op == "barrier":
                pass
            else:
                raise CollectiveMismatch(op)


def run_ranks(n: int, body: Callable[[ThreadComm], object], timeout: float = 30.0) -> List[object]:
    """Run ``body(comm)`` on n rank-threads; returns the per-rank results or raises the first failure."""
    hub = _Hub(n, timeout)
    results, errors = [None] * n, [None] * n

    def runner(r):
        try:
            results[r] = body(ThreadComm(hub, r))
        except RankFailed as e:
            errors[r] = e
        except Exception as e:  # noqa: BLE001
            errors[r] = e
            hub.fail(e)
        finally:
            hub.depart()

    ts = [threading.Thread(target=runner, args=(r,), daemon=True) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout + 30)
    primary = [e for e in errors if e is not None and not isinstance(e, RankFailed)]
    if primary:
        raise primary[0]
    if any(errors):
        raise next(e for e in errors if e is not None)
    return results


class DistComm:
    """Same interface over torch.distributed (gloo on CPU, nccl on GPU)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def all_reduce(self, t):
        self.dist.all_reduce(t, group=self.group)

    def all_reduce_async(self, t):
        """Enqueues the reduction and returns a handle with ``wait()``; on NCCL it runs on the library's own stream,
        ordered after the work already enqueued on the caller's stream, so later kernels of the caller overlap it."""
        return self.dist.all_reduce(t, group=self.group, async_op=True)

    def reduce_scatter(self, out, inp):
        if self.dist.get_backend(self.group) == "gloo":
            tmp = inp.clone()
            self.dist.all_reduce(tmp, group=self.group)
            k = out.numel()
            out.reshape(-1).copy_(tmp.reshape(-1)[self.rank * k:(self.rank + 1) * k])
        else:
            self.dist.reduce_scatter_tensor(out, inp, group=self.group)

    def all_gather(self, out, inp):
        self.dist.all_gather_into_tensor(out, inp.contiguous(), group=self.group)

    def broadcast(self, t, src=0):
        self.dist.broadcast(t, src, group=self.group)

    def barrier(self):
        self.dist.barrier(group=self.group)
