"""Parameter-efficient fine-tuning and 4-bit weights.

``freeze_params(module, predicate)`` marks parameters frozen (no gradient, skipped by the optimizer).
``LoRALinear(base, rank, alpha)``: ``y = base(x) + (alpha / rank) · (x A) B`` with ``A [in, r]`` (Kaiming) and ``B [r, out]``
(zero), base frozen; parameter names ``base_layer.weight|bias``, ``lora_A.weight``, ``lora_B.weight`` (the PEFT layout);
``merge()`` folds the update into the base weight.  ``quantize_q4_0`` / ``dequantize_q4_0``: blocks of 32 values with
one fp16 scale.  ``QLinear``: a frozen Linear whose weight is stored in Q4_0 and expanded to bf16 by a CUDA kernel
before the GEMM; ``QLoRALinear = LoRALinear(QLinear)``.
Reference: noeira/nn/peft/freeze.mojo:39, lora.mojo:156,584, peft_io.mojo, quant/q4_0.mojo, qlinear.mojo:208, qlora.mojo:43.
"""
from __future__ import annotations

import ctypes

import torch

from .._native import check, cuda_lib, ptr, stream_ptr
from .init import Kaiming, Zero
from .layers import Linear
from .module import Module


def freeze_params(module: Module, predicate=lambda name, p: True) -> int:
    n = 0
    for name, p in module.named_params():
        if predicate(name, p):
            p.frozen = True
            n += 1
    return n


class LoRALinear(Module):
    def __init__(self, base: Module, rank: int = 16, alpha: float = 32.0):
        super().__init__()
        assert rank % 8 == 0, "rank must be a multiple of 8 (16-byte rows for the tensor-core path)"
        self.base = self.add_child("base_layer", base)
        for _, p in base.named_params():
            p.frozen = True
        self.rank, self.scale = rank, alpha / rank
        self.lora_a = self.add_child("lora_A", Linear(base.in_dim, rank, bias=False, init=Kaiming()))
        self.lora_b = self.add_child("lora_B", Linear(rank, base.out_dim, bias=False, init=Zero()))
        self.in_dim, self.out_dim = base.in_dim, base.out_dim
        self.merged = False

    def forward(self, x, residual=None):
        y = self.base.forward(x, residual=residual)
        if self.merged:
            return y
        u = self.lora_b.forward(self.lora_a.forward(x))
        return y + (u.to(y.dtype) * self.scale)

    def vjp(self, dy):
        dx = self.base.vjp(dy)
        if self.merged:
            return dx
        d = dy * self.scale
        dx2 = self.lora_a.vjp(self.lora_b.vjp(d))
        return dx2 if dx is None else dx + dx2.to(dx.dtype)

    @torch.no_grad()
    def merge(self):
        """W ← W + (alpha / r) · A B; afterwards the adapter costs nothing at inference."""
        w = self.base.weight
        w.data.add_(self.scale * (self.lora_a.weight.data.float() @ self.lora_b.weight.data.float()))
        w.version += 1
        self.merged = True


# ------------------------------------------------------------------------------------------ Q4_0
def quantize_q4_0(w: torch.Tensor):
    """fp32 [rows, cols] (cols % 32 == 0) → (codes uint8 [rows, cols / 2], scales fp16 [rows, cols / 32])."""
    rows, cols = w.shape
    assert cols % 32 == 0
    blk = w.float().reshape(rows, cols // 32, 32)
    amax_idx = blk.abs().argmax(-1, keepdim=True)
    mx = blk.gather(-1, amax_idx)                       # signed value of largest magnitude
    d = (mx / -8.0)
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.clamp(torch.floor(blk * inv + 8.5), 0, 15).to(torch.uint8)
    codes = (q[..., :16] | (q[..., 16:] << 4)).reshape(rows, cols // 2).contiguous()
    return codes, d.squeeze(-1).to(torch.float16).contiguous()


def dequantize_q4_0(codes: torch.Tensor, scales: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    rows = codes.shape[0]
    cols = codes.shape[1] * 2
    if codes.is_cuda:
        out = torch.empty(rows, cols, device=codes.device, dtype=torch.bfloat16)
        check(cuda_lib().nb_q4_0_dequant(ptr(codes), ptr(scales), ptr(out), ctypes.c_int(rows), ctypes.c_int(cols),
                                         ctypes.c_int(cols), stream_ptr()), "q4_0_dequant")
        return out if out_dtype == torch.bfloat16 else out.to(out_dtype)
    c = codes.reshape(rows, cols // 32, 16)
    q = torch.cat([c & 15, c >> 4], -1).float() - 8.0
    return (q * scales.float().unsqueeze(-1)).reshape(rows, cols).to(out_dtype)


def gptq_quantize_q4_0(w: torch.Tensor, x: torch.Tensor, damp: float = 0.01):
    """GPTQ for a Linear weight ``w [IN, OUT]`` (Q4_0 blocks of 32 along OUT) from calibration inputs ``x [n, IN]``:
    input rows are quantised one after the other and the rounding error of a row is pushed onto the rows not yet
    quantised through the inverse Hessian of the layer's squared output error (H = 2 XᵀX / n), so that ``x @ w`` is
    preserved far better than by rounding each weight on its own.  Returns ``(codes, scales)`` in the layout of
    ``quantize_q4_0``.  (Frantar et al., "GPTQ", 2023; reference: noeira/nn/quant/ GPTQ calibration.)"""
    IN, OUT = w.shape
    assert OUT % 32 == 0 and x.shape[1] == IN
    W = w.detach().double().cpu().clone()
    X = x.detach().double().cpu()
    H = 2.0 * (X.t() @ X) / max(X.shape[0], 1)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1.0
    W[dead] = 0.0
    H += damp * torch.diag(H).mean() * torch.eye(IN, dtype=torch.float64)
    Hinv = torch.cholesky_inverse(torch.linalg.cholesky(H))
    U = torch.linalg.cholesky(Hinv, upper=True)          # Hinv = Uᵀ U; row i of U drives the update of rows > i
    codes = torch.empty(IN, OUT // 2, dtype=torch.uint8)
    scales = torch.empty(IN, OUT // 32, dtype=torch.float16)
    for i in range(IN):
        c, sc = quantize_q4_0(W[i: i + 1].float())
        codes[i], scales[i] = c[0], sc[0]
        q = dequantize_q4_0(c, sc, torch.float32)[0].double()
        err = (W[i] - q) / U[i, i]
        if i + 1 < IN:
            W[i + 1:] -= U[i, i + 1:, None] * err[None, :]
    return codes, scales


class QLinear(Module):
    """Frozen Linear with a Q4_0 weight (0.5625 bytes per element).  The bias stays fp32."""

    def __init__(self, linear: Linear, calibration: torch.Tensor = None):
        """``calibration``: optional inputs ``[n, IN]`` of this layer; with them the weight is quantised by GPTQ."""
        super().__init__()
        self.in_dim, self.out_dim, self.act = linear.in_dim, linear.out_dim, linear.act
        assert self.out_dim % 32 == 0, "Q4_0 blocks run along the output dimension of the [IN, OUT] weight"
        wcpu = linear.weight.data.float().cpu()[: self.in_dim, : self.out_dim]
        if calibration is not None:
            codes, scales = gptq_quantize_q4_0(wcpu, calibration.float().cpu().reshape(-1, self.in_dim))
        else:
            codes, scales = quantize_q4_0(linear.weight.data.float().cpu())
        self.codes = self.add_state("qweight", codes.shape)
        self.codes.data = codes
        self.scales = self.add_state("scales", scales.shape)
        self.scales.data = scales
        self.bias = linear.bias
        if self.bias is not None:
            self._params["bias"] = self.bias
            self.bias.frozen = True
        self._w = None

    def _moved(self, device):
        self._w = None

    def weight_bf16(self):
        if self._w is None:          # expanded once: the weight never changes
            self._w = dequantize_q4_0(self.codes.data, self.scales.data, torch.bfloat16 if self.on_cuda else torch.float32)
        return self._w

    def forward(self, x, residual=None):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        W = self.weight_bf16()
        if self.on_cuda:
            from ..ops.gemm import gemm
            y = gemm(x2.to(torch.bfloat16), W, b_mn=True, bias=self.bias.storage if self.bias is not None else None, act=self.act)
        else:
            y = x2.float() @ W
            if self.bias is not None:
                y = y + self.bias.data
            if self.act is not None:
                from .layers import _ACT_CPU
                y = _ACT_CPU[self.act](y)
        self._saved = y
        y = y.reshape(*lead, self.out_dim)
        return y if residual is None else y + residual

    def vjp(self, dy):
        d2 = dy.reshape(-1, self.out_dim)
        if self.act is not None:
            from .layers import act_backward
            d2 = act_backward(d2.to(self._saved.dtype), self._saved, self.act)
        W = self.weight_bf16()
        if self.on_cuda:
            from ..ops.gemm import gemm
            dx = gemm(d2.to(torch.bfloat16).contiguous(), W)                 # dy [M, OUT] · Wᵀ, W is [IN, OUT] = [N, K]
        else:
            dx = d2.float() @ W.t()
        return dx.reshape(*dy.shape[:-1], self.in_dim)


def QLoRALinear(linear: Linear, rank: int = 16, alpha: float = 32.0) -> LoRALinear:
    return LoRALinear(QLinear(linear), rank, alpha)


# ------------------------------------------------------------------------------------------ adapter / quantisation slots
def replace_linears(module: Module, factory, predicate=lambda path, lin: True, prefix: str = "") -> int:
    """Replaces every plain ``Linear`` below ``module`` whose dotted path passes ``predicate`` by ``factory(linear)``: in
    the child registry and in every attribute (or list attribute) of the parent that holds the same object, so that model
    code written against ``self.q_proj`` / ``self.mods[i]`` picks the wrapper up.  Returns the number of replacements.
    (The reference gives each decoder linear an adapter slot and a quantised slot at compile time,
    noeira/deep_agents/smolvla/layer_weights.mojo:30-105; here the slot is filled at run time.)"""
    n = 0
    for key, child in list(module._children.items()):
        path = prefix + key
        if type(child) is Linear:
            if not predicate(path, child):
                continue
            new = factory(child)
            new.device = child.device
            module._children[key] = new
            for attr, val in list(vars(module).items()):
                if val is child:
                    setattr(module, attr, new)
                elif isinstance(val, list):
                    for i, v in enumerate(val):
                        if v is child:
                            val[i] = new
            n += 1
        else:
            n += replace_linears(child, factory, predicate, path + ".")
    return n


def add_lora(module: Module, rank: int = 16, alpha: float = 32.0, predicate=lambda path, lin: True) -> int:
    """LoRA adapters on the selected linears (their base weights are frozen); the adapters are the only trainable
    parameters they add: ``<path>.lora_A.weight``, ``<path>.lora_B.weight``."""
    return replace_linears(module, lambda lin: LoRALinear(lin, rank=rank, alpha=alpha), predicate)


def quantize_linears(module: Module, predicate=lambda path, lin: lin.out_dim % 32 == 0, calibration=None, lora_rank: int = 0,
                     alpha: float = 32.0) -> int:
    """Q4_0 weights on the selected linears (``calibration``: ``{path: inputs}`` quantises those layers by GPTQ); with
    ``lora_rank`` every quantised layer also carries a trainable adapter (QLoRA)."""
    cal, paths = calibration or {}, {}

    def pred(path, lin):
        ok = predicate(path, lin)
        if ok:
            paths[id(lin)] = path
        return ok

    def factory(lin):
        q = QLinear(lin, calibration=cal.get(paths.get(id(lin))))
        return LoRALinear(q, lora_rank, alpha) if lora_rank else q

    return replace_linears(module, factory, pred)
