"""Iterative LQR over a differentiable dynamics function.

``dynamics(x, u) -> x'`` and ``cost(x, u) -> scalar``, ``final_cost(x) -> scalar`` are PyTorch functions; their first
and second derivatives come from ``torch.func`` (jacobians of the dynamics, gradients and Hessians of the costs).
Backward pass: the standard Riccati recursion with Levenberg-Marquardt regularisation on ``Q_uu``; forward pass: line
search over the feed-forward scale.  (Reference: noeira/planners/trajectory/ilqr.mojo + ilqr_kernels.mojo.)
"""
from __future__ import annotations

from typing import Callable

import torch
from torch.func import hessian, jacrev


class ILQR:
    def __init__(self, dynamics: Callable, cost: Callable, final_cost: Callable, horizon: int, act_dim: int,
                 reg: float = 1e-3, max_reg: float = 1e6):
        self.f, self.l, self.lf, self.H, self.A = dynamics, cost, final_cost, horizon, act_dim
        self.reg, self.max_reg = reg, max_reg
        self.U = None

    def rollout(self, x0, U):
        X, c = [x0], torch.zeros(())
        for t in range(self.H):
            c = c + self.l(X[-1], U[t])
            X.append(self.f(X[-1], U[t]))
        return torch.stack(X), c + self.lf(X[-1])

    def plan(self, x0: torch.Tensor, iterations: int = 20, tol: float = 1e-6):
        x0 = x0.double()
        U = self.U if self.U is not None else torch.zeros(self.H, self.A, dtype=torch.float64)
        X, J = self.rollout(x0, U)
        reg = self.reg
        for _ in range(iterations):
            # derivatives along the trajectory
            fx = [jacrev(self.f, 0)(X[t], U[t]) for t in range(self.H)]
            fu = [jacrev(self.f, 1)(X[t], U[t]) for t in range(self.H)]
            lx = [jacrev(self.l, 0)(X[t], U[t]) for t in range(self.H)]
            lu = [jacrev(self.l, 1)(X[t], U[t]) for t in range(self.H)]
            lxx = [hessian(self.l, 0)(X[t], U[t]) for t in range(self.H)]
            luu = [hessian(self.l, 1)(X[t], U[t]) for t in range(self.H)]
            lux = [jacrev(jacrev(self.l, 1), 0)(X[t], U[t]) for t in range(self.H)]
            Vx, Vxx = jacrev(self.lf)(X[-1]), hessian(self.lf)(X[-1])
            k, K = [None] * self.H, [None] * self.H
            ok = True
            for t in reversed(range(self.H)):
                Qx, Qu = lx[t] + fx[t].T @ Vx, lu[t] + fu[t].T @ Vx
                Qxx = lxx[t] + fx[t].T @ Vxx @ fx[t]
                Quu = luu[t] + fu[t].T @ Vxx @ fu[t] + reg * torch.eye(self.A, dtype=torch.float64)
                Qux = lux[t] + fu[t].T @ Vxx @ fx[t]
                try:
                    L = torch.linalg.cholesky(Quu)
                except RuntimeError:
                    ok = False
                    break
                k[t] = -torch.cholesky_solve(Qu[:, None], L)[:, 0]
                K[t] = -torch.cholesky_solve(Qux, L)
                Vx = Qx + K[t].T @ Quu @ k[t] + K[t].T @ Qu + Qux.T @ k[t]
                Vxx = Qxx + K[t].T @ Quu @ K[t] + K[t].T @ Qux + Qux.T @ K[t]
                Vxx = 0.5 * (Vxx + Vxx.T)
            if not ok:
                reg = min(reg * 10, self.max_reg)
                continue
            improved = False
            for alpha in (1.0, 0.5, 0.25, 0.1, 0.03, 0.01):
                Xn, Un = [x0], []
                for t in range(self.H):
                    u = U[t] + alpha * k[t] + K[t] @ (Xn[-1] - X[t])
                    Un.append(u)
                    Xn.append(self.f(Xn[-1], u))
                Un = torch.stack(Un)
                Xn, Jn = self.rollout(x0, Un)
                if Jn < J:
                    improved = True
                    dJ = float(J - Jn)
                    X, U, J = Xn, Un, Jn
                    reg = max(reg / 5, 1e-8)
                    break
            if not improved:
                reg = min(reg * 10, self.max_reg)
                if reg >= self.max_reg:
                    break
            elif dJ < tol:
                break
        self.U = U
        return U, X, float(J)
