"""Multi-GPU gates (run as child processes, one rank per GPU; skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _world_sizes():
    """Every power of two from 2 up to the number of GPUs of the box (2, 4, 8 on a full node)."""
    n, out = _ngpu(), []
    only = os.environ.get("NB_TEST_WORLDS")          # e.g. "4,8": restrict the sweep (each size is one torchrun launch)
    if only:
        return [int(x) for x in only.split(",") if int(x) <= n] or [2]
    w = 2
    while w <= min(n, 8):
        out.append(w)
        w *= 2
    return out or [2]


def _torchrun(script, world, port, timeout=900):
    # NVLS off: a rank that exits while bound to an NVLink multicast object can fault its peers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port),
                           os.path.join(ROOT, "tests", "mp", script)], capture_output=True, text=True, timeout=timeout, env=env)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", _world_sizes())
def test_fused_allreduce_adam_matches_nccl(world):
    r = _torchrun("ddp_worker.py", world, 29611 + world)
    assert "DDP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_bounded_wait_reports_timeout_and_context_survives():
    """A device wait on a flag that nothing sets runs out, records NB_ST_PEER_TIMEOUT and returns; the
    context stays usable (no trap, no hang)."""
    import ctypes
    from noeira_b200._native import check, cuda_lib, ptr, stream_ptr
    from noeira_b200.ops.status import DeviceStatusError, check_status, device_status
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    res = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    check(cuda_lib().nb_wait_flag_probe(ptr(flag), ctypes.c_uint(1), ctypes.c_uint(2000), ptr(device_status()), ptr(res),
                                        stream_ptr()), "probe")
    torch.cuda.synchronize()
    assert int(res.item()) == 0
    with pytest.raises(DeviceStatusError) as e:
        check_status()
    assert e.value.code == 2 and e.value.where == 99 and e.value.extra == 7
    # context still healthy, and a satisfied wait passes
    flag.fill_(5)
    check(cuda_lib().nb_wait_flag_probe(ptr(flag), ctypes.c_uint(3), ctypes.c_uint(2000), ptr(device_status()), ptr(res),
                                        stream_ptr()), "probe")
    torch.cuda.synchronize()
    assert int(res.item()) == 1
    check_status()


def test_tp_fused_kernels_single_rank():
    """world = 1: the fused kernels degenerate to GEMM (+ slot round trip) — exercises the tile pipeline."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "mp", "tp_worker.py")], capture_output=True, text=True,
                       timeout=600)
    assert "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", _world_sizes())
def test_tp_fused_kernels_match_nccl(world):
    r = _torchrun("tp_worker.py", world, 29621 + world)
    assert "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("world", _world_sizes())
def test_world_model_tp_matches_single_rank(world):
    """TP + SP world model (KV-head replica groups from 4 ranks up) against the same model on one rank."""
    r = _torchrun("wm_worker.py", world, 29641 + world)
    assert "WM_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
