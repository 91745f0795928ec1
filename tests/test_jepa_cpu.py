"""The latent world model: the Gaussian-sketch regulariser, training without collapse, prediction beats copy-last,
planning in latent space."""
import math

import torch

from noeira_b200.experimental.jepa import JEPAConfig, JEPAWorldModel, random_directions, sigreg


def test_sigreg_is_small_for_a_standard_gaussian_and_large_otherwise():
    g = torch.Generator().manual_seed(0)
    dirs = random_directions(8, 128, g, "cpu")
    z = torch.randn(2048, 8, generator=g)
    base = float(sigreg(z, dirs))
    assert base < 2.0                                             # the statistic of a sample of the null is O(1)
    assert float(sigreg(torch.zeros(2048, 8), dirs)) > 50 * base                       # collapsed
    assert float(sigreg(z * 3.0, dirs)) > 20 * base                                    # too wide
    assert float(sigreg(z + 1.0, dirs)) > 20 * base                                    # shifted
    squashed = z.clone()
    squashed[:, 0] = 0.0
    assert float(sigreg(squashed, dirs)) > 5 * base                                     # one dead dimension
    # its gradient spreads a collapsed batch out
    c = (0.01 * torch.randn(256, 8, generator=g)).requires_grad_(True)
    sigreg(c, dirs).backward()
    assert float((c.grad * c.detach()).sum()) < 0                                        # descent moves points outward


class _Circle:
    """A point on a plane pushed by 2-D actions, seen through a fixed random nonlinear map to 16 values."""

    def __init__(self, seed=0):
        g = torch.Generator().manual_seed(seed)
        self.g = g
        self.a = torch.randn(2, 16, generator=g)
        self.b = torch.randn(16, generator=g)

    def observe(self, s):
        return torch.tanh(s @ self.a + self.b) + 0.3 * (s @ self.a)

    def batch(self, n):
        s = torch.rand(n, 2, generator=self.g) * 2 - 1
        a = torch.rand(n, 2, generator=self.g) * 2 - 1
        s2 = (s + 0.3 * a).clamp(-1.3, 1.3)
        return s, a, s2


def test_training_keeps_the_latents_spread_and_predicts_better_than_copy_last():
    env = _Circle()
    wm = JEPAWorldModel(JEPAConfig(latent_dim=4, hidden=64, lr=2e-3, projections=128, seed=1))
    first = None
    for step in range(500):
        s, a, s2 = env.batch(256)
        m = wm.train_step(env.observe(s), a, env.observe(s2))
        first = first or m
    s, a, s2 = env.batch(256)                                      # the statistic grows with the batch: same size as in training
    sg = float(wm.losses(env.observe(s), a, env.observe(s2))[2])
    assert sg < 0.2 * first["sigreg"]
    s, a, s2 = env.batch(1024)
    total, pl, _, copy_last = (float(v) for v in wm.losses(env.observe(s), a, env.observe(s2)))
    assert math.isfinite(total)
    z = wm.encode(env.observe(s))
    assert z.std(0).min() > 0.3 and z.std(0).max() < 3.0          # no dimension collapsed or blew up
    assert pl < 0.35 * copy_last                                   # the action-conditioned prediction carries information
    # the latents hold the state: a linear read-out recovers the position
    sol = torch.linalg.lstsq(torch.cat([z, torch.ones(1024, 1)], 1), s).solution
    resid = (torch.cat([z, torch.ones(1024, 1)], 1) @ sol - s).pow(2).mean() / s.var()
    assert float(resid) < 0.15
    # planning: shooting in latent space moves the point toward the goal
    start, goal = torch.tensor([[-0.6, -0.6]]), torch.tensor([[0.6, 0.5]])
    pos = start.clone()
    for _ in range(10):
        act = wm.plan(env.observe(pos), env.observe(goal), horizon=5, samples=256)
        pos = (pos + 0.3 * act.reshape(1, 2).cpu()).clamp(-1.3, 1.3)
    assert float((pos - goal).norm()) < 0.45 * float((start - goal).norm())
