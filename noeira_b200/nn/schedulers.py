"""Learning-rate schedules: pure functions of the step, written into the optimizer's device-resident hyper block
(``opt.set_lr``), so a captured step reads the new rate without re-capture.
Reference: noeira/nn/optimizer/lr_scheduler.mojo:33-121 (Constant, LinearWarmup, Cosine, WarmupCosine, StepDecay)."""
from __future__ import annotations

import math


class Constant:
    def __init__(self, lr):
        self.lr = lr

    def __call__(self, step):
        return self.lr


class LinearWarmup:
    def __init__(self, lr, warmup_steps):
        self.lr, self.w = lr, max(int(warmup_steps), 1)

    def __call__(self, step):
        return self.lr * min(1.0, (step + 1) / self.w)


class Cosine:
    def __init__(self, lr, total_steps, min_lr=0.0):
        self.lr, self.T, self.min = lr, max(int(total_steps), 1), min_lr

    def __call__(self, step):
        t = min(step, self.T) / self.T
        return self.min + 0.5 * (self.lr - self.min) * (1 + math.cos(math.pi * t))


class WarmupCosine:
    def __init__(self, lr, warmup_steps, total_steps, min_lr=0.0):
        self.lr, self.w, self.T, self.min = lr, max(int(warmup_steps), 1), max(int(total_steps), 1), min_lr

    def __call__(self, step):
        if step < self.w:
            return self.lr * (step + 1) / self.w
        t = min(step - self.w, self.T - self.w) / max(self.T - self.w, 1)
        return self.min + 0.5 * (self.lr - self.min) * (1 + math.cos(math.pi * t))


class StepDecay:
    def __init__(self, lr, every, gamma=0.1):
        self.lr, self.every, self.gamma = lr, max(int(every), 1), gamma

    def __call__(self, step):
        return self.lr * self.gamma ** (step // self.every)


def apply(schedule, optimizer, step):
    lr = schedule(step)
    optimizer.set_lr(lr)
    return lr
