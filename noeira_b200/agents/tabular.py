"""Tabular agents on small discrete MDPs (CPU): Q-learning, SARSA, Expected SARSA and Double Q-learning over a
``TabularEnv`` (``reset() -> s``, ``step(a) -> (s', r, done)``), plus a reference grid world.
(Reference: noeira/agents/ — the tabular family; the linear-function-approximation variants are not built.)"""
from __future__ import annotations

import numpy as np


class GridWorld:
    """``n x n`` grid, start top-left, goal bottom-right (+1), pits (−1) end the episode, step cost −0.01; actions
    0..3 = up, right, down, left; moves off the grid stay in place."""

    def __init__(self, n=5, pits=((1, 3), (3, 1)), max_steps=100):
        self.n, self.pits, self.max_steps = n, set(pits), max_steps
        self.n_states, self.n_actions = n * n, 4

    def reset(self):
        self.pos, self.t = (0, 0), 0
        return 0

    def step(self, a):
        dr, dc = ((-1, 0), (0, 1), (1, 0), (0, -1))[a]
        r, c = min(max(self.pos[0] + dr, 0), self.n - 1), min(max(self.pos[1] + dc, 0), self.n - 1)
        self.pos, self.t = (r, c), self.t + 1
        s = r * self.n + c
        if self.pos == (self.n - 1, self.n - 1):
            return s, 1.0, True
        if self.pos in self.pits:
            return s, -1.0, True
        return s, -0.01, self.t >= self.max_steps


class TabularAgent:
    def __init__(self, n_states, n_actions, kind="q_learning", alpha=0.2, gamma=0.98, eps=0.1, seed=0):
        assert kind in ("q_learning", "sarsa", "expected_sarsa", "double_q")
        self.kind, self.alpha, self.gamma, self.eps = kind, alpha, gamma, eps
        self.rng = np.random.default_rng(seed)
        self.q = np.zeros((n_states, n_actions))
        self.q2 = np.zeros((n_states, n_actions)) if kind == "double_q" else None

    def values(self, s):
        return self.q[s] if self.q2 is None else self.q[s] + self.q2[s]

    def act(self, s, greedy=False):
        if not greedy and self.rng.random() < self.eps:
            return int(self.rng.integers(self.q.shape[1]))
        v = self.values(s)
        return int(self.rng.choice(np.flatnonzero(v == v.max())))

    def learn(self, s, a, r, s2, done, a2=None):
        g = 0.0 if done else self.gamma
        if self.kind == "q_learning":
            target = r + g * self.q[s2].max()
        elif self.kind == "sarsa":
            target = r + g * self.q[s2, a2]
        elif self.kind == "expected_sarsa":
            nA = self.q.shape[1]
            pi = np.full(nA, self.eps / nA)
            pi[self.q[s2].argmax()] += 1 - self.eps
            target = r + g * float(pi @ self.q[s2])
        else:
            if self.rng.random() < 0.5:
                self.q, self.q2 = self.q2, self.q
            target = r + g * self.q2[s2, self.q[s2].argmax()]
        self.q[s, a] += self.alpha * (target - self.q[s, a])

    def train(self, env, episodes):
        returns = []
        for _ in range(episodes):
            s, done, G = env.reset(), False, 0.0
            a = self.act(s)
            while not done:
                s2, r, done = env.step(a)
                a2 = self.act(s2)
                self.learn(s, a, r, s2, done, a2)
                s, a, G = s2, a2, G + r
            returns.append(G)
        return returns
