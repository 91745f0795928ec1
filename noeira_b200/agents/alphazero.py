"""AlphaZero: self-play with a tree search over the TRUE game model, a policy / value network trained on its outcomes.

The search is the batched PUCT search of ``planners.mcts`` with the game itself as the transition function: the search's
"latent" is the canonical position plus a finished flag, ``recurrent`` plays the move, evaluates the network on the new
position and masks illegal moves; positions are always seen by the player to move, so the tree runs with discount −1
(a child's value counts negatively for its parent: negamax backup).  Finished positions are absorbing with value 0.
Training: ``loss = CE(π_search, p) + (z − v)²`` on positions drawn from a ring of recent self-play games, with z the final
outcome from the mover's point of view.
(noeira/deep_agents/alphazero/: self-play driver, masked expansion and negated backup kernels of the tree search,
loss kernels loss_ops.mojo:41-68.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from .. import nn
from ..planners.mcts import BatchedMCTS, MCTSConfig

_NEG = -1e9


@dataclass
class AlphaZeroConfig:
    hidden: int = 128
    n_simulations: int = 50
    lr: float = 2e-3
    batch: int = 256
    buffer: int = 20000
    temperature_moves: int = 4          # moves per game sampled from the visit counts; greedy afterwards
    root_noise_frac: float = 0.25
    dirichlet_alpha: float = 0.6
    value_coef: float = 1.0
    max_grad_norm: float = 5.0
    seed: int = 0


class AlphaZeroAgent:
    def __init__(self, game, cfg: AlphaZeroConfig = None, device="cpu"):
        self.game, self.cfg = game.to(device), cfg or AlphaZeroConfig()
        c, self.device = self.cfg, torch.device(device)
        nn.manual_seed(c.seed)
        C, A = game.cells, game.n_actions
        self.trunk = nn.Sequential(nn.LinearReLU(C, c.hidden, need_input_grad=False), nn.LinearReLU(c.hidden, c.hidden)).to(self.device)
        self.policy = nn.Linear(c.hidden, A, out_fp32=True).to(self.device)
        self.value = nn.Linear(c.hidden, 1, out_fp32=True).to(self.device)
        self.opt = nn.Adam(list(self.trunk.named_params("trunk.")) + list(self.policy.named_params("policy.")) +
                           list(self.value.named_params("value.")), lr=c.lr)
        self.opt.max_grad_norm = c.max_grad_norm
        self.gen = torch.Generator(device=self.device).manual_seed(c.seed + 1)
        mk = lambda noise: BatchedMCTS(MCTSConfig(n_actions=A, n_simulations=c.n_simulations, discount=-1.0,
                                                   root_noise_frac=noise, dirichlet_alpha=c.dirichlet_alpha,
                                                   max_depth=game.cells + 1), self._initial, self._recurrent)
        self.mcts, self.mcts_eval = mk(c.root_noise_frac), mk(0.0)
        z = dict(device=self.device)
        self.buf_s = torch.zeros(c.buffer, C, **z)
        self.buf_pi = torch.zeros(c.buffer, A, **z)
        self.buf_z = torch.zeros(c.buffer, **z)
        self.size = self.pos = 0
        self.last: Dict[str, float] = {}

    # ---- network
    def _inp(self, x):
        return x.to(torch.bfloat16) if self.device.type == "cuda" else x.float()

    def net(self, board):
        h = self.trunk.forward(self._inp(board))
        return self.policy.forward(h).float(), torch.tanh(self.value.forward(h).float()[:, 0])

    # ---- model functions of the search: latent = [board | finished]
    def _initial(self, board):
        logits, v = self.net(board)
        logits = torch.where(self.game.legal(board), logits, torch.full_like(logits, _NEG))
        return torch.cat([board, torch.zeros(board.shape[0], 1, device=board.device)], 1), logits, v

    def _recurrent(self, latent, action):
        board, fin = latent[:, :-1], latent[:, -1] > 0.5
        legal_move = self.game.legal(board).gather(1, action[:, None])[:, 0]
        nb, r, done = self.game.step(board, action)
        stay = fin | ~legal_move                                   # absorbing: finished games and (zero-prior) illegal edges
        nb = torch.where(stay[:, None], board, nb)
        r = torch.where(stay, torch.zeros_like(r), r)
        fin2 = fin | done | ~legal_move
        logits, v = self.net(nb)
        logits = torch.where(self.game.legal(nb), logits, torch.full_like(logits, _NEG))
        logits = torch.where(fin2[:, None], torch.zeros_like(logits), logits)
        v = torch.where(fin2, torch.zeros_like(v), v)
        return torch.cat([nb, fin2.float()[:, None]], 1), r, logits, v

    @torch.no_grad()
    def act(self, board, temperature: float = 0.0, explore: bool = False):
        """(visit-count policy, root value, move) for a batch of positions."""
        m = self.mcts if explore else self.mcts_eval
        return m.search(board, legal=self.game.legal(board), temperature=temperature, generator=self.gen)

    # ---- self-play
    @torch.no_grad()
    def self_play(self, n_games: int) -> int:
        """Plays ``n_games`` games in lock step and appends every position with its search policy and final outcome
        (from the mover's side) to the ring.  Returns the number of stored positions."""
        g, c = self.game, self.cfg
        board = g.initial(n_games)
        alive = torch.ones(n_games, dtype=torch.bool, device=self.device)
        hist = []                                                   # (board, π, alive-at-that-ply)
        outcome_ply = torch.full((n_games,), -1, device=self.device)
        won = torch.zeros(n_games, device=self.device)
        ply = 0
        while bool(alive.any()):
            pi, _, a = self.act(board, temperature=1.0 if ply < c.temperature_moves else 0.0, explore=True)
            hist.append((board.clone(), pi, alive.clone()))
            nb, r, done = g.step(board, a)
            ended = alive & done
            outcome_ply = torch.where(ended, torch.full_like(outcome_ply, ply), outcome_ply)
            won = torch.where(ended, r, won)                        # 1: the mover at ``outcome_ply`` won; 0: draw
            board = torch.where(alive[:, None], nb, board)
            alive = alive & ~done
            ply += 1
        stored = 0
        for t, (b, pi, live) in enumerate(hist):
            sign = 1.0 - 2.0 * ((outcome_ply - t) % 2).float()      # same side as the last mover: +, other side: −
            z = won * sign
            idx = live.nonzero(as_tuple=False)[:, 0]
            k = idx.numel()
            slot = (self.pos + torch.arange(k, device=self.device)) % c.buffer
            self.buf_s[slot], self.buf_pi[slot], self.buf_z[slot] = b[idx], pi[idx], z[idx]
            self.pos = (self.pos + k) % c.buffer
            self.size = min(c.buffer, self.size + k)
            stored += k
        return stored

    # ---- training
    def loss_and_grads(self, logits, v, pi, z):
        """CE(π, softmax(logits)) + c_v (z − v)²; returns loss, d/dlogits, d/d(value pre-activation)."""
        B = logits.shape[0]
        logp = torch.log_softmax(logits, -1)
        pl = -(pi * logp).sum(-1).mean()
        vl = ((z - v) ** 2).mean()
        dlogits = (logp.exp() * pi.sum(-1, keepdim=True) - pi) / B
        dvpre = self.cfg.value_coef * 2 * (v - z) * (1 - v * v) / B
        return pl + self.cfg.value_coef * vl, dlogits, dvpre, pl, vl

    def train_step(self):
        c = self.cfg
        idx = torch.randint(0, self.size, (min(c.batch, self.size),), device=self.device, generator=self.gen)
        s, pi, z = self.buf_s[idx], self.buf_pi[idx], self.buf_z[idx]
        h = self.trunk.forward(self._inp(s))
        logits = self.policy.forward(h).float()
        logits = torch.where(self.game.legal(s), logits, torch.full_like(logits, _NEG))
        v = torch.tanh(self.value.forward(h).float()[:, 0])
        loss, dlogits, dvpre, pl, vl = self.loss_and_grads(logits, v, pi, z)
        dh = self.policy.vjp(dlogits) + self.value.vjp(dvpre[:, None])
        self.trunk.vjp(dh)
        if c.max_grad_norm > 0:
            self.opt.clip()
        self.opt.step(zero_grad=True)
        self.last = dict(loss=float(loss), policy_loss=float(pl), value_loss=float(vl))
        return self.last

    # ---- evaluation
    @torch.no_grad()
    def play_vs_random(self, n_games: int, agent_first: bool = True, use_search: bool = True):
        """→ (wins, draws, losses) of the agent against a uniformly random legal mover."""
        g = self.game
        board = g.initial(n_games)
        alive = torch.ones(n_games, dtype=torch.bool, device=self.device)
        result = torch.zeros(n_games, device=self.device)           # +1 agent won, −1 agent lost
        agent_turn = agent_first
        while bool(alive.any()):
            if agent_turn:
                if use_search:
                    _, _, a = self.act(board)
                else:
                    lg, _ = self.net(board)
                    a = torch.where(g.legal(board), lg, torch.full_like(lg, _NEG)).argmax(1)
            else:
                p = g.legal(board).float() + 1e-9
                a = torch.multinomial(p, 1, generator=self.gen)[:, 0]
            nb, r, done = g.step(board, a)
            result = torch.where(alive & (r > 0), torch.full_like(result, 1.0 if agent_turn else -1.0), result)
            board = torch.where(alive[:, None], nb, board)
            alive = alive & ~done
            agent_turn = not agent_turn
        return int((result > 0).sum()), int((result == 0).sum()), int((result < 0).sum())

    def save(self, path):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.trunk.named_params("trunk.")) + list(self.policy.named_params("policy.")) +
                        list(self.value.named_params("value.")), [], {})
