"""Two-player line games on a grid as batched tensor programs: tic-tac-toe and connect four.

A position is stored in canonical form, from the point of view of the player to move: ``+1`` own stone, ``−1`` opponent
stone, ``0`` empty, flattened row-major to ``[n, rows·cols]``.  ``step`` places a stone of the mover, reports ``+1`` when
that completes a line of ``k`` (the mover wins; there is no other non-zero reward), and hands the position to the
opponent by flipping the signs.  All functions are pure and work on any batch on any device, so a tree search can use
them as its transition model.  (The reference's AlphaZero examples play the same two games:
noeira/deep_agents/alphazero/.)
"""
from __future__ import annotations

import torch


class LineGame:
    def __init__(self, rows: int, cols: int, k: int, gravity: bool, device="cpu"):
        self.rows, self.cols, self.k, self.gravity = rows, cols, k, gravity
        self.cells = rows * cols
        self.n_actions = cols if gravity else self.cells
        lines = []
        for r in range(rows):
            for c in range(cols):
                for dr, dc in ((0, 1), (1, 0), (1, 1), (1, -1)):
                    rr, cc = r + (k - 1) * dr, c + (k - 1) * dc
                    if 0 <= rr < rows and 0 <= cc < cols:
                        row = torch.zeros(self.cells)
                        for i in range(k):
                            row[(r + i * dr) * cols + c + i * dc] = 1.0
                        lines.append(row)
        self.lines = torch.stack(lines).to(device)                      # [n_lines, cells]
        self.device = torch.device(device)

    def to(self, device):
        self.lines, self.device = self.lines.to(device), torch.device(device)
        return self

    def initial(self, n: int) -> torch.Tensor:
        return torch.zeros(n, self.cells, device=self.device)

    def legal(self, board: torch.Tensor) -> torch.Tensor:
        if self.gravity:
            return board[:, : self.cols] == 0                            # row 0 is the top row
        return board == 0

    def _cell(self, board, action):
        if not self.gravity:
            return action
        col = board.reshape(-1, self.rows, self.cols)[torch.arange(board.shape[0], device=board.device), :, action]   # [n, rows]
        depth = (col == 0).sum(1) - 1                                   # lowest empty row of the column
        return depth.clamp(min=0) * self.cols + action

    def step(self, board: torch.Tensor, action: torch.Tensor):
        """→ (next position seen by the opponent, reward of the mover, done)."""
        ar = torch.arange(board.shape[0], device=board.device)
        nb = board.clone()
        nb[ar, self._cell(board, action)] = 1.0
        win = (((nb > 0).float() @ self.lines.t()) >= self.k).any(1)
        full = (nb != 0).all(1)
        return -nb, win.float(), win | full


def TicTacToe(device="cpu") -> LineGame:
    return LineGame(3, 3, 3, gravity=False, device=device)


def ConnectFour(device="cpu") -> LineGame:
    return LineGame(6, 7, 4, gravity=True, device=device)
