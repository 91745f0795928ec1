"""Supervised trainers over device-resident data.

``Trainer``: classification / regression on a dataset that lives on the device (``x [N, …]``, ``y [N]``); each step
gathers a batch by index (indices drawn on the device by a keyed permutation of the epoch), runs forward, loss,
explicit backward, clip and the arena optimizer; the whole step is replayed from a CUDA graph when
``use_cuda_graph`` is set (noeira/nn/training/trainer.mojo:84: resident dataset, sub-buffer batch views, captured epoch).

``AutoregressiveTrainer``: next-token training of a language model on one resident token stream with device-side
window sampling, warm-up + cosine learning rate and gradient clipping
(noeira/nn/training/autoregressive_trainer.mojo:53).
"""
from __future__ import annotations

import math

import torch

from .. import nn
from ..nn import schedulers


class Trainer:
    def __init__(self, model, x: torch.Tensor, y: torch.Tensor, batch: int, loss: str = "cross_entropy", lr: float = 1e-3,
                 weight_decay: float = 0.0, max_grad_norm: float = 0.0, optimizer: str = "adamw", seed: int = 0,
                 use_cuda_graph: bool = False, grad_sync=None, augmenter=None):
        self.model, self.batch, self.loss_kind = model, batch, loss
        self.device = x.device
        # with an augmenter the trainer trains from a buffer that is rewritten from the raw set once per epoch (the
        # buffer keeps its address, so a captured step keeps working)
        self.augmenter = augmenter if augmenter is not None and not augmenter.is_noop else None
        self.raw_x = x
        self.seed = seed
        if self.augmenter is not None:
            x = torch.empty_like(x)
            self.augmenter.augment(x, self.raw_x, 0, seed)
        self.x, self.y = x, y
        self.n = x.shape[0]
        opt_cls = {"adamw": nn.AdamW, "adam": nn.Adam, "sgd": nn.SGD, "laprop": nn.LaProp}[optimizer]
        kw = {"weight_decay": weight_decay} if optimizer == "adamw" else {}
        self.opt = opt_cls(model.named_params(), lr=lr, **kw)
        self.opt.max_grad_norm = max_grad_norm
        self.grad_sync = grad_sync
        if grad_sync is not None:
            grad_sync.attach(self.opt)
        self.loss_acc = torch.zeros(1, device=self.device)
        self.correct = torch.zeros(1, device=self.device)
        self.gen = torch.Generator(device=self.device).manual_seed(seed)
        self.mse = nn.MSELoss()
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self._graphed = None
        self._idx = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.steps = 0

    def _step_body(self, idx):
        if self.device.type == "cuda":
            nn.advance_rng(self.device)
        xb, yb = self.x.index_select(0, idx), self.y.index_select(0, idx)
        out = self.model.forward(xb)
        if self.loss_kind == "cross_entropy":
            self.correct += (out.float().argmax(-1) == yb).float().sum()
            g = nn.cross_entropy(out if out.is_cuda and out.dtype == torch.bfloat16 else (out.to(torch.bfloat16) if out.is_cuda else out),
                                 yb, self.loss_acc)
        else:
            g = self.mse(out, yb.float().reshape(out.shape), self.loss_acc)
        self.model.vjp(g)
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(self.opt)
        else:
            if self.opt.max_grad_norm > 0:
                self.opt.clip()
            self.opt.step(zero_grad=True)
        return self.loss_acc

    def train_step(self, idx: torch.Tensor = None):
        if idx is None:
            idx = torch.randint(0, self.n, (self.batch,), device=self.device, generator=self.gen)
        self.steps += 1
        if not self.use_cuda_graph:
            return self._step_body(idx)
        if self._graphed is None:
            from ..utils.graphs import GraphedStep
            self._graphed = GraphedStep(self._step_body, [idx])
        return self._graphed(idx)

    def train_epoch(self, epoch: int = 0):
        """One pass in a shuffled order (device-side permutation); returns (mean loss, accuracy) read once at the end."""
        self.loss_acc.zero_()
        self.correct.zero_()
        if self.augmenter is not None:
            self.augmenter.augment(self.x, self.raw_x, epoch, self.seed)
        g = torch.Generator(device=self.device).manual_seed(1234567 + epoch)
        perm = torch.randperm(self.n, device=self.device, generator=g)
        nb = self.n // self.batch
        for b in range(nb):
            self.train_step(perm[b * self.batch: (b + 1) * self.batch])
        return float(self.loss_acc) / max(nb, 1), float(self.correct) / max(nb * self.batch, 1)

    @torch.no_grad()
    def evaluate(self, x, y):
        self.model.eval()
        out = self.model.forward(x)
        self.model.train()
        return float((out.float().argmax(-1) == y).float().mean())


class AutoregressiveTrainer:
    def __init__(self, model, tokens: torch.Tensor, batch: int, seq: int, lr: float = 3e-4, warmup: int = 100,
                 total_steps: int = 10000, min_lr_frac: float = 0.1, weight_decay: float = 0.1, max_grad_norm: float = 1.0,
                 seed: int = 0, use_cuda_graph: bool = False, grad_sync=None, rank: int = 0, world: int = 1):
        self.model, self.tokens, self.batch, self.seq = model, tokens, batch, seq
        self.device = tokens.device
        self.opt = nn.AdamW(model.named_params(), lr=lr, weight_decay=weight_decay)
        self.opt.max_grad_norm = max_grad_norm
        self.grad_sync = grad_sync
        if grad_sync is not None:
            grad_sync.attach(self.opt)
            if hasattr(grad_sync, "attach_model"):
                grad_sync.attach_model(model)        # overlapped reduction: the units' vjp launch their buckets
        self.schedule = schedulers.WarmupCosine(lr, warmup, total_steps, lr * min_lr_frac)
        self.loss_acc = torch.zeros(1, device=self.device)
        # every rank draws the GLOBAL batch of window starts from the same stream and keeps its slice, so that N ranks
        # at batch B/N see exactly the windows one rank at batch B would (global-batch-equivalent sharded sampler)
        self.gen = torch.Generator(device=self.device).manual_seed(seed)
        self.rank, self.world = rank, world
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self._graphed = None
        self._ar = torch.arange(seq + 1, device=self.device)
        self.step_no = 0

    def sample_windows(self):
        hi = self.tokens.numel() - self.seq - 1
        starts = torch.randint(0, hi, (self.batch * self.world,), device=self.device, generator=self.gen)
        return starts[self.rank * self.batch: (self.rank + 1) * self.batch]

    def _step_body(self, starts):
        if self.device.type == "cuda":
            nn.advance_rng(self.device)
        win = self.tokens[(starts[:, None] + self._ar[None]).reshape(-1)].reshape(self.batch, self.seq + 1)
        ids, tgt = win[:, :-1].contiguous(), win[:, 1:].contiguous()
        logits = self.model.forward(ids)
        g = nn.cross_entropy(logits, tgt, self.loss_acc)
        if self.world > 1 and self.grad_sync is not None:
            pass                                   # the sync averages over ranks; the loss is already a per-rank mean
        self.model.vjp(g)
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(self.opt)
        else:
            if self.opt.max_grad_norm > 0:
                self.opt.clip()
            self.opt.step(zero_grad=True)
        return self.loss_acc

    def train_step(self):
        schedulers.apply(self.schedule, self.opt, self.step_no)
        starts = self.sample_windows()
        self.step_no += 1
        if not self.use_cuda_graph:
            return self._step_body(starts)
        if self._graphed is None:
            from ..utils.graphs import GraphedStep
            self._graphed = GraphedStep(self._step_body, [starts])
        return self._graphed(starts)

    def mean_loss(self, reset=True):
        v = float(self.loss_acc)
        if reset:
            self.loss_acc.zero_()
        return v
