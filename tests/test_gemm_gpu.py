"""tcgen05 GEMM against a plain fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 512), (300, 200, 136), (4096, 256, 256), (128, 64, 4096)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(0)
    Mp, Np, Kp = (M + 7) // 8 * 8, (N + 7) // 8 * 8, (K + 7) // 8 * 8
    a = (torch.randn(Kp if a_mn else Mp, Mp if a_mn else Kp, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(Kp if b_mn else Np, Np if b_mn else Kp, device="cuda") * 0.5).bfloat16()
    a_v = a[:K, :M] if a_mn else a[:M, :K]
    b_v = b[:K, :N] if b_mn else b[:N, :K]
    out = gemm(a_v, b_v, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    check_status()
    ref = _ref(a_v, b_v, a_mn, b_mn)
    err = (out - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_gemm_tile_widths(bn):
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(1)
    M, N, K = 512, 256, 320
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    out = gemm(a, b, bn=bn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    check_status()
    ref = a.float() @ b.float().t()
    assert (out - ref).abs().max().item() < 5e-2


@pytest.mark.parametrize("act", ["relu", "tanh", "gelu", "silu", "sigmoid"])
def test_gemm_epilogues(act):
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(2)
    M, N, K = 384, 192, 256
    a = (torch.randn(M, K, device="cuda") * 0.2).bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.2).bfloat16()  # [IN, OUT] layout → MN-major B
    bias = torch.randn(N, device="cuda")
    y = gemm(a, w, b_mn=True, bias=bias, act=act)
    pre = a.float() @ w.float() + bias
    f = dict(relu=torch.relu, tanh=torch.tanh, gelu=lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
             silu=torch.nn.functional.silu, sigmoid=torch.sigmoid)[act]
    ref = f(pre)
    torch.cuda.synchronize()
    check_status()
    assert (y.float() - ref).abs().max().item() < 3e-2
    # dgrad with fused activation derivative: dx = (dy · Wᵀ) ⊙ f'(saved)
    dy = (torch.randn(M, N, device="cuda") * 0.2).bfloat16()
    saved = (y if act in ("relu", "tanh", "sigmoid") else pre.bfloat16())
    # derivative wrt the PRE-activation of a previous layer of width K: use aux of shape [M, K]
    saved_k = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    if act == "relu":
        saved_k = saved_k.relu()
    if act == "tanh":
        saved_k = saved_k.float().tanh().bfloat16()
    if act == "sigmoid":
        saved_k = saved_k.float().sigmoid().bfloat16()
    dx = gemm(dy, w, b_mn=False, aux=saved_k, dact=act, out_dtype=torch.float32)
    s = saved_k.float()
    if act == "relu":
        d = (s > 0).float()
    elif act == "tanh":
        d = 1 - s * s
    elif act == "sigmoid":
        d = s * (1 - s)
    else:
        x = s.clone().requires_grad_(True)
        f(x).sum().backward()
        d = x.grad
    ref_dx = (dy.float() @ w.float().t()) * d
    torch.cuda.synchronize()
    check_status()
    assert (dx - ref_dx).abs().max().item() < 3e-2
    assert saved is not None


def test_gemm_wgrad_accumulate():
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(3)
    T, IN, OUT = 2048, 256, 192
    x = (torch.randn(T, IN, device="cuda") * 0.3).bfloat16()
    dy = (torch.randn(T, OUT, device="cuda") * 0.3).bfloat16()
    dW = torch.ones(IN, OUT, device="cuda")
    gemm(x, dy, a_mn=True, b_mn=True, out=dW, accumulate=True)  # dW[IN,OUT] += xᵀ·dy
    torch.cuda.synchronize()
    check_status()
    ref = 1.0 + x.float().t() @ dy.float()
    assert (dW - ref).abs().max().item() < 0.15, (dW - ref).abs().max().item()


def test_gemm_large_matches_and_times():
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(4)
    M = N = K = 4096
    a = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    out = gemm(a, b)
    ref = (a @ b.t()).float()
    torch.cuda.synchronize()
    check_status()
    assert (out.float() - ref).abs().max().item() < 0.1


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(256, 256, 16384, True, True), (17, 256, 16384, True, True),
                                             (256, 8, 8192, True, True), (128, 128, 4096, False, False),
                                             (384, 192, 2048, False, True)])
def test_gemm_split_k_deterministic(M, N, K, a_mn, b_mn):
    """Few tiles + deep K takes the split-K path (partials in the workspace, ordered fix-up)."""
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(5)
    Mp, Np = (M + 7) // 8 * 8, (N + 7) // 8 * 8
    a = (torch.randn((K, Mp) if a_mn else (Mp, K), device="cuda") * 0.3).bfloat16()
    b = (torch.randn((K, Np) if b_mn else (Np, K), device="cuda") * 0.3).bfloat16()
    a_v = a[:, :M] if a_mn else a[:M]
    b_v = b[:, :N] if b_mn else b[:N]
    outs = []
    for _ in range(2):
        out = torch.full((M, Np), 0.5, device="cuda")
        gemm(a_v, b_v, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=True, n=N)
        outs.append(out)
    torch.cuda.synchronize()
    check_status()
    ref = 0.5 + _ref(a_v, b_v, a_mn, b_mn)
    err = (outs[0][:, :N] - ref).abs().max().item()
    assert err < 2e-2 * ref.abs().max().item(), err
    assert torch.equal(outs[0], outs[1])


@pytest.fixture
def two_cta():
    from noeira_b200.ops.gemm import TWO_CTA_FORCE, set_two_cta_mode
    old = set_two_cta_mode(TWO_CTA_FORCE)
    yield
    set_two_cta_mode(old)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 768, 320), (1000, 520, 264), (4096, 1024, 512)])
def test_gemm_two_cta_tiles(M, N, K, a_mn, b_mn, two_cta):
    """256 x 256 tiles on CTA pairs (cta_group::2): all four operand layouts, ragged M / N / K edges."""
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(5)
    a = (torch.randn(K if a_mn else M, M if a_mn else K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(K if b_mn else N, N if b_mn else K, device="cuda") * 0.5).bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (out - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


def test_gemm_two_cta_epilogue_and_repeat(two_cta):
    """Bias + activation + bf16 store through the pair kernel; two runs are bit-identical."""
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(6)
    M, N, K = 768, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.2).bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.2).bfloat16()
    bias = torch.randn(N, device="cuda")
    y1 = gemm(a, w, b_mn=True, bias=bias, act="gelu")
    y2 = gemm(a, w, b_mn=True, bias=bias, act="gelu")
    torch.cuda.synchronize()
    check_status()
    ref = torch.nn.functional.gelu(a.float() @ w.float() + bias, approximate="tanh")
    assert torch.equal(y1, y2)
    assert (y1.float() - ref).abs().max().item() < 3e-2


def _tf32_round(x):
    """fp32 → TF32 by round-to-nearest-even on the 13 dropped mantissa bits (what the copy into shared memory does)."""
    i = x.contiguous().view(torch.int32)
    r = i + 0xFFF + ((i >> 13) & 1)
    return (r & ~0x1FFF).view(torch.float32)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (256, 256, 512), (300, 200, 132), (4096, 256, 256), (128, 64, 4096), (64, 16, 96)])
def test_gemm_tf32_layouts(M, N, K, a_mn, b_mn):
    """fp32 operands through the TF32 tensor-core path, all four operand layouts, against an fp32 reference on operands
    rounded to TF32 (tight) and on the raw operands (the 10-bit-mantissa error bound)."""
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(0)
    Mp, Np, Kp = (M + 3) // 4 * 4, (N + 3) // 4 * 4, (K + 3) // 4 * 4
    a = torch.randn(Kp if a_mn else Mp, Mp if a_mn else Kp, device="cuda") * 0.5
    b = torch.randn(Kp if b_mn else Np, Np if b_mn else Kp, device="cuda") * 0.5
    a_v = a[:K, :M] if a_mn else a[:M, :K]
    b_v = b[:K, :N] if b_mn else b[:N, :K]
    out = gemm(a_v, b_v, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    check_status()
    assert out.dtype == torch.float32
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        raw = _ref(a_v, b_v, a_mn, b_mn)
        rounded = _ref(_tf32_round(a_v), _tf32_round(b_v), a_mn, b_mn)
        trunc = _ref((a_v.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32),
                     (b_v.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32), a_mn, b_mn)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    scale = max(1.0, raw.abs().max().item())
    e_exact = min((out - rounded).abs().max().item(), (out - trunc).abs().max().item())
    assert e_exact < 2e-5 * scale * max(1.0, K / 512), (e_exact, (out - raw).abs().max().item())
    assert (out - raw).abs().max().item() < 2e-3 * scale * max(1.0, (K / 256) ** 0.5)


def test_gemm_tf32_epilogue_accumulate_and_split_k():
    from noeira_b200.ops import check_status, gemm
    torch.manual_seed(3)
    M, N, K = 384, 96, 160
    a, b = torch.randn(M, K, device="cuda") * 0.3, torch.randn(K, N, device="cuda") * 0.3
    bias = torch.randn(N, device="cuda")
    y = gemm(a, b, b_mn=True, bias=bias, act="tanh")
    ref = torch.tanh(_tf32_round(a) @ _tf32_round(b) + bias)
    assert (y - ref).abs().max().item() < 2e-3
    yb = gemm(a, b, b_mn=True, bias=bias, act="relu", out_dtype=torch.bfloat16, out=torch.empty(M, N, device="cuda", dtype=torch.bfloat16))
    assert (yb.float() - torch.relu(a @ b + bias)).abs().max().item() < 3e-2
    # weight-gradient form: accumulate x^T dy into fp32, deep K through the split-K path, bit-repeatable
    x, dy = torch.randn(16384, 64, device="cuda") * 0.1, torch.randn(16384, 128, device="cuda") * 0.1
    acc = torch.ones(64, 128, device="cuda")
    gemm(x, dy, a_mn=True, b_mn=True, out=acc, accumulate=True)
    acc2 = torch.ones(64, 128, device="cuda")
    gemm(x, dy, a_mn=True, b_mn=True, out=acc2, accumulate=True)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(acc, acc2)
    assert (acc - (1 + x.double().t() @ dy.double()).float()).abs().max().item() < 2e-2


def test_linear_tf32_precision_mode_matches_fp32_reference():
    """``set_attr("precision", "tf32")``: an MLP with fp32 activations on the TF32 path; forward, input gradient and
    parameter gradients against plain fp32 PyTorch on the same weights."""
    from noeira_b200 import nn
    from noeira_b200.ops import check_status
    nn.manual_seed(0)
    net = nn.Sequential(nn.LinearTanh(24, 96), nn.LinearGELU(96, 64), nn.Linear(64, 6)).to("cuda")
    net.set_attr("precision", "tf32")
    torch.manual_seed(1)
    x = torch.randn(300, 24, device="cuda")
    dy = torch.randn(300, 6, device="cuda")
    y = net.forward(x)
    dx = net.vjp(dy)
    torch.cuda.synchronize()
    check_status()
    assert y.dtype == torch.float32 and dx.dtype == torch.float32
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        xr = x.clone().requires_grad_(True)
        Ws = [(m.weight.data.clone().requires_grad_(True), m.bias.data.clone().requires_grad_(True)) for m in net.mods]
        h = torch.tanh(xr @ Ws[0][0] + Ws[0][1])
        h = torch.nn.functional.gelu(h @ Ws[1][0] + Ws[1][1], approximate="tanh")
        ref = h @ Ws[2][0] + Ws[2][1]
        ref.backward(dy)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert (y - ref).abs().max().item() < 5e-3
    assert (dx - xr.grad).abs().max().item() < 2e-2
    for m, (W, b) in zip(net.mods, Ws):
        assert (m.weight.grad - W.grad).abs().max().item() < 5e-2 * max(1.0, W.grad.abs().max().item())
        assert (m.bias.grad - b.grad).abs().max().item() < 1e-3 * max(1.0, b.grad.abs().max().item())
    # far closer to fp32 than the bf16 path of the same layers
    net.set_attr("precision", None)
    yb = net.forward(x.bfloat16()).float()
    assert (y - ref).abs().max().item() < 0.5 * (yb - ref).abs().max().item()
