import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N", [(16384, 256), (1000, 6), (37, 130), (128, 1)])
def test_colsum(M, N):
    from noeira_b200.nn.layers import colsum_into
    torch.manual_seed(0)
    Np = (N + 7) // 8 * 8
    x = torch.randn(M, Np, device="cuda").bfloat16()
    out = torch.ones(Np, device="cuda")
    colsum_into(x, out, N, accumulate=True)
    out2 = torch.ones(Np, device="cuda")
    colsum_into(x, out2, N, accumulate=True)
    torch.cuda.synchronize()
    ref = 1 + x[:, :N].float().sum(0)
    assert torch.allclose(out[:N], ref, atol=1e-2, rtol=1e-4)
    assert torch.equal(out, out2)
    if Np != N:
        assert (out[N:] == 1).all()
