"""Runs with NOEIRA_B200_BOUNDS=1: index-driven kernels of the bounds-checked library on valid inputs (clean status) and
on out-of-range indices (NB_ST_BOUNDS recorded, access skipped, context still usable)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    assert os.environ.get("NOEIRA_B200_BOUNDS") == "1"
    from noeira_b200 import _native, nn
    from noeira_b200.data.replay import StoreReplayGpu
    from noeira_b200.ops.status import DeviceStatusError, check_status, device_status
    assert _native.cuda_lib()._name.endswith("libnoeira_b200_bounds.so")
    device_status()                                         # registers the status word with every checked unit
    emb = nn.Embedding(16, 32).to("cuda")
    out = emb.forward(torch.tensor([[1, 5, 15]], device="cuda"))
    torch.cuda.synchronize()
    check_status()
    ref = emb.weight.data[[1, 5, 15]].to(torch.bfloat16)
    assert torch.allclose(out[0].float(), ref.float(), atol=1e-2)
    emb.forward(torch.tensor([[2, 99]], device="cuda"))     # 99 >= vocab: reported, not read
    torch.cuda.synchronize()
    try:
        check_status()
        print("BOUNDS_FAIL: no report")
        return 1
    except DeviceStatusError as e:
        assert e.code == 3 and e.where == 601 and e.extra == 99, (e.code, e.where, e.extra)
    rb = StoreReplayGpu(64, 3, 1, prioritized=False)
    z = lambda *s: torch.zeros(*s, device="cuda")
    rb.store_batch(z(8, 3), z(8, 1), z(8), z(8, 3), z(8))
    rb.gather(torch.tensor([0, 3, 7], device="cuda"))
    torch.cuda.synchronize()
    check_status()
    rb.gather(torch.tensor([0, 64, 7], device="cuda"))      # 64 == capacity
    torch.cuda.synchronize()
    try:
        check_status()
        print("BOUNDS_FAIL: no report for the replay index")
        return 1
    except DeviceStatusError as e:
        assert e.code == 3 and e.where == 611 and e.extra == 64
    # the context is still healthy
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    check_status()
    print("BOUNDS_WORKER_OK")
    return 0


if __name__ == "__main__":
    sys.exit(main())
