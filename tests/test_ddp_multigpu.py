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


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_allreduce_adam_matches_nccl():
    n = min(_ngpu(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29611",
                        os.path.join(ROOT, "tests", "mp", "ddp_worker.py")], capture_output=True, text=True, timeout=600,
                       env=env)
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
def test_tp_fused_kernels_match_nccl():
    n = min(_ngpu(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29621",
                        os.path.join(ROOT, "tests", "mp", "tp_worker.py")], capture_output=True, text=True, timeout=600,
                       env=env)
    assert "TP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
