"""Reward shaping from a bound goal: a potential that is 0 exactly when the goal holds.

``ShapedGoalReward`` turns the goal tape's distance into the per-step reward
``success_bonus · [goal reached this step] + scale · (d_{t-1} − d_t) − step_cost`` (potential-based, so the shaped and
the sparse problem have the same optimal policies), and latches success per episode.
Reference: noeira/tasks/shaping.mojo:1-243.
"""
from __future__ import annotations

import torch

from .predicates import BoundGoal, GoalState, evaluate, evaluate_cuda


class ShapedGoalReward:
    def __init__(self, bound: BoundGoal, n: int, device, scale: float = 10.0, success_bonus: float = 5.0,
                 step_cost: float = 0.01):
        self.bound, self.scale, self.bonus, self.step_cost = bound, scale, success_bonus, step_cost
        self.prev = torch.zeros(n, device=device)
        self.done = torch.zeros(n, dtype=torch.bool, device=device)
        self.tape = bound.tensors(device)
        self.on_cuda = torch.device(device).type == "cuda"

    def _eval(self, st: GoalState):
        return evaluate_cuda(self.bound, st, self.tape) if self.on_cuda else evaluate(self.bound, st)

    def reset(self, st: GoalState, mask=None):
        _, d = self._eval(st)
        if mask is None:
            self.prev.copy_(d)
            self.done.zero_()
        else:
            self.prev = torch.where(mask, d, self.prev)
            self.done &= ~mask

    def step(self, st: GoalState):
        """→ (reward [N], success [N] bool: the goal holds now)."""
        ok, d = self._eval(st)
        first = ok & ~self.done
        r = self.scale * (self.prev - d) - self.step_cost + self.bonus * first.float()
        self.prev.copy_(d)
        self.done |= ok
        return r, ok
