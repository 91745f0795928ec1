"""Batched Monte Carlo tree search (PUCT, MuZero-style) with one tree per environment, all trees advanced in lock step.

Per simulation, for all environments at once: (1) SELECT — descend from the root by the PUCT score
``Q̂(s,a) + c(N) · P(s,a) · sqrt(N(s)) / (1 + N(s,a))`` (Q normalised by the tree's running min / max) until an unexpanded
edge; (2) one BATCHED model call for the leaves (``recurrent(latent, action) → latent', reward, policy logits, value``);
(3) EXPAND — append the node, softmax its priors (legal-action mask optional); (4) BACKUP — discounted return along the
path.  The tree lives in preallocated tensors; on CUDA select / expand / backup are one kernel each
(``csrc/mcts.cu``, one thread per tree, no host synchronisation inside a search); the tensor-program versions below run
anywhere and are the oracle of the GPU test.
Reference: noeira/planners/tree_search/mcts_gpu.mojo:1-60 (root parallelisation, per-simulation kernel sequence),
noeira/planners/tree_search/model_traits.mojo (Representation / Dynamics / Prediction), mcts_cpu.mojo.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch


@dataclass
class MCTSConfig:
    n_actions: int
    n_simulations: int = 50
    discount: float = 0.997
    pb_c_base: float = 19652.0
    pb_c_init: float = 1.25
    dirichlet_alpha: float = 0.3
    root_noise_frac: float = 0.0        # 0.25 for self-play exploration
    max_depth: int = 32
    # Gumbel root search (``search_gumbel``): actions considered at the root, and the σ transform of completed Q values
    gumbel_considered: int = 16
    gumbel_c_visit: float = 50.0
    gumbel_c_scale: float = 1.0


class MCTSTree:
    """Tree storage of ``n`` independent searches with at most ``n_simulations + 1`` nodes each."""

    def __init__(self, n: int, cfg: MCTSConfig, latent_dim: int, device):
        N, A = cfg.n_simulations + 1, cfg.n_actions
        z = dict(device=device)
        self.n, self.cfg, self.N, self.A, self.L = n, cfg, N, A, latent_dim
        self.children = torch.full((n, N, A), -1, dtype=torch.int32, **z)
        self.prior = torch.zeros(n, N, A, **z)
        self.visit = torch.zeros(n, N, **z)
        self.value_sum = torch.zeros(n, N, **z)
        self.reward = torch.zeros(n, N, **z)
        self.parent = torch.full((n, N), -1, dtype=torch.int32, **z)
        self.latent = torch.zeros(n, N, latent_dim, **z)
        self.n_nodes = torch.ones(n, dtype=torch.int32, **z)
        self.minmax = torch.stack([torch.full((n,), float("inf"), **z), torch.full((n,), float("-inf"), **z)], dim=1).contiguous()
        self.leaf_parent = torch.zeros(n, dtype=torch.int32, **z)
        self.leaf_action = torch.zeros(n, dtype=torch.int32, **z)

    def reset(self):
        self.children.fill_(-1); self.prior.zero_(); self.visit.zero_(); self.value_sum.zero_(); self.reward.zero_()
        self.parent.fill_(-1); self.n_nodes.fill_(1)
        self.minmax[:, 0] = float("inf"); self.minmax[:, 1] = float("-inf")


def _softmax_masked(logits, legal):
    if legal is not None:
        logits = logits.masked_fill(~legal, float("-inf"))
    return torch.softmax(logits.float(), dim=-1)


# ------------------------------------------------------------------------------------------ tensor-program tree ops
def select_torch(t: MCTSTree):
    cfg, ar = t.cfg, torch.arange(t.n, device=t.visit.device)
    node = torch.zeros(t.n, dtype=torch.long, device=t.visit.device)
    done = torch.zeros(t.n, dtype=torch.bool, device=t.visit.device)
    lp = torch.zeros_like(node)
    la = torch.zeros_like(node)
    lo, hi = t.minmax[:, 0], t.minmax[:, 1]
    span_ok = hi > lo
    for _ in range(cfg.max_depth):
        ch = t.children[ar, node].long()                                  # [n, A]
        expanded = ch >= 0
        chc = ch.clamp(min=0)
        nc = torch.where(expanded, t.visit[ar[:, None], chc], torch.zeros_like(t.prior[:, 0]))
        q_raw = t.reward[ar[:, None], chc] + cfg.discount * t.value_sum[ar[:, None], chc] / nc.clamp(min=1)
        qn = torch.where(span_ok[:, None], (q_raw - lo[:, None]) / (hi - lo).clamp(min=1e-8)[:, None], q_raw)
        q = torch.where(expanded & (nc > 0), qn, torch.zeros_like(qn))
        np_ = t.visit[ar, node]
        c = torch.log((np_ + cfg.pb_c_base + 1) / cfg.pb_c_base) + cfg.pb_c_init
        u = c[:, None] * t.prior[ar, node] * torch.sqrt(np_.clamp(min=1))[:, None] / (1 + nc)
        score = q + u
        score = torch.where(t.prior[ar, node] > 0, score, torch.full_like(score, float("-inf")))   # illegal actions
        a = score.argmax(dim=1)
        child = ch[ar, a]
        stop = (child < 0) & ~done
        lp = torch.where(stop, node, lp)
        la = torch.where(stop, a, la)
        done |= stop
        node = torch.where(done, node, child.clamp(min=0))
    # a path that reached max_depth without an unexpanded edge re-expands its last edge target (rare; bounded trees)
    lp = torch.where(done, lp, node)
    t.leaf_parent.copy_(lp.int())
    t.leaf_action.copy_(la.int())


def expand_torch(t: MCTSTree, latent, reward, logits, value, legal=None):
    ar = torch.arange(t.n, device=t.visit.device)
    new = t.n_nodes.long().clamp(max=t.N - 1)
    lp, la = t.leaf_parent.long(), t.leaf_action.long()
    t.children[ar, lp, la] = new.int()
    t.parent[ar, new] = lp.int()
    t.latent[ar, new] = latent.float()
    t.reward[ar, new] = reward.float()
    t.prior[ar, new] = _softmax_masked(logits, legal)
    t.n_nodes.copy_((new + 1).int())
    return new


def backup_torch(t: MCTSTree, leaf, value):
    cfg, ar = t.cfg, torch.arange(t.n, device=t.visit.device)
    node = leaf.clone()
    g = value.float().clone()
    alive = torch.ones(t.n, dtype=torch.bool, device=t.visit.device)
    for _ in range(t.N):                      # a path has at most one node per simulation
        t.value_sum[ar, node] += torch.where(alive, g, torch.zeros_like(g))
        t.visit[ar, node] += alive.float()
        q = t.reward[ar, node] + cfg.discount * (t.value_sum[ar, node] / t.visit[ar, node].clamp(min=1))
        isroot = node == 0
        upd = alive & ~isroot
        t.minmax[:, 0] = torch.where(upd, torch.minimum(t.minmax[:, 0], q), t.minmax[:, 0])
        t.minmax[:, 1] = torch.where(upd, torch.maximum(t.minmax[:, 1], q), t.minmax[:, 1])
        g = t.reward[ar, node] + cfg.discount * g
        alive = alive & ~isroot
        node = t.parent[ar, node].long().clamp(min=0)
        if not bool(alive.any()):
            break


# ------------------------------------------------------------------------------------------ CUDA tree ops
def _cuda_select(t):
    from .._native import check, cuda_lib, ptr, stream_ptr
    c, cfg = ctypes, t.cfg
    check(cuda_lib().nb_mcts_select(ptr(t.children), ptr(t.prior), ptr(t.visit), ptr(t.value_sum), ptr(t.reward), ptr(t.minmax),
                                    c.c_int(t.n), c.c_int(t.N), c.c_int(t.A), c.c_float(cfg.discount), c.c_float(cfg.pb_c_base),
                                    c.c_float(cfg.pb_c_init), c.c_int(cfg.max_depth), ptr(t.leaf_parent), ptr(t.leaf_action),
                                    stream_ptr()), "mcts_select")


def _cuda_expand_backup(t, latent, reward, logits, value, legal):
    from .._native import check, cuda_lib, ptr, stream_ptr
    c, cfg = ctypes, t.cfg
    lg = legal.to(torch.uint8).contiguous() if legal is not None else None
    check(cuda_lib().nb_mcts_expand_backup(ptr(t.children), ptr(t.prior), ptr(t.visit), ptr(t.value_sum), ptr(t.reward), ptr(t.parent),
                                           ptr(t.latent), ptr(t.n_nodes), ptr(t.minmax), ptr(t.leaf_parent), ptr(t.leaf_action),
                                           ptr(latent.float().contiguous()), ptr(reward.float().contiguous()),
                                           ptr(logits.float().contiguous()), ptr(value.float().contiguous()), ptr(lg), c.c_int(t.n),
                                           c.c_int(t.N), c.c_int(t.A), c.c_int(t.L), c.c_float(cfg.discount), c.c_int(cfg.max_depth),
                                           stream_ptr()), "mcts_expand_backup")


class BatchedMCTS:
    """``initial(obs) → (latent [n,L], logits [n,A], value [n])``; ``recurrent(latent, action) → (latent', reward [n],
    logits [n,A], value [n])``.  ``search`` returns (visit-count policy [n,A], root value [n], chosen action [n])."""

    def __init__(self, cfg: MCTSConfig, initial: Callable, recurrent: Callable, use_kernels: Optional[bool] = None):
        self.cfg, self.initial, self.recurrent, self.use_kernels = cfg, initial, recurrent, use_kernels
        self.tree: Optional[MCTSTree] = None

    @torch.no_grad()
    def search(self, obs, legal=None, temperature: float = 0.0, generator=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        cfg = self.cfg
        latent, logits, value = self.initial(obs)
        n, dev = latent.shape[0], latent.device
        kern = self.use_kernels if self.use_kernels is not None else dev.type == "cuda"
        if self.tree is None or self.tree.n != n or self.tree.L != latent.shape[1] or self.tree.visit.device != dev:
            self.tree = MCTSTree(n, cfg, latent.shape[1], dev)
        t = self.tree
        t.reset()
        pri = _softmax_masked(logits, legal)
        if cfg.root_noise_frac > 0:
            noise = torch.distributions.Dirichlet(torch.full((cfg.n_actions,), cfg.dirichlet_alpha, device=dev)).sample((n,))
            pri = (1 - cfg.root_noise_frac) * pri + cfg.root_noise_frac * noise
            if legal is not None:
                pri = pri * legal
                pri = pri / pri.sum(-1, keepdim=True).clamp(min=1e-8)
        t.prior[:, 0] = pri
        t.latent[:, 0] = latent.float()
        t.visit[:, 0] = 1.0
        t.value_sum[:, 0] = value.float()
        ar = torch.arange(n, device=dev)
        for _ in range(cfg.n_simulations):
            (_cuda_select if kern else select_torch)(t)
            lat = t.latent[ar, t.leaf_parent.long()]
            nl, r, lg, v = self.recurrent(lat, t.leaf_action.long())
            if kern:
                _cuda_expand_backup(t, nl, r, lg, v, None)
            else:
                new = expand_torch(t, nl, r, lg, v, None)
                backup_torch(t, new, v)
        ch = t.children[:, 0].long()
        counts = torch.where(ch >= 0, t.visit[ar[:, None], ch.clamp(min=0)], torch.zeros_like(t.prior[:, 0]))
        policy = counts / counts.sum(-1, keepdim=True).clamp(min=1)
        root_value = t.value_sum[:, 0] / t.visit[:, 0]
        if temperature <= 0:
            action = counts.argmax(-1)
        else:
            p = counts.pow(1.0 / temperature)
            action = torch.multinomial(p / p.sum(-1, keepdim=True), 1, generator=generator).squeeze(-1)
        return policy, root_value, action


    # ------------------------------------------------------------------ Gumbel root search with sequential halving
    def _simulate(self, t, kern, ar):
        (_cuda_select if kern else select_torch)(t)
        lat = t.latent[ar, t.leaf_parent.long()]
        nl, r, lg, v = self.recurrent(lat, t.leaf_action.long())
        if kern:
            _cuda_expand_backup(t, nl, r, lg, v, None)
        else:
            backup_torch(t, expand_torch(t, nl, r, lg, v, None), v)

    @torch.no_grad()
    def search_gumbel(self, obs, legal=None, generator=None, greedy: bool = False):
        """Policy improvement by planning with Gumbel (Danihelka et al.): sample Gumbel noise g, consider the top-m actions
        by g + logits, split the simulation budget over ⌈log₂ m⌉ halving phases (every surviving action gets the same
        number of visits in a phase; the root action of a simulation is forced by a one-hot root prior, below the root the
        usual PUCT descent runs), drop the worse half by g + logits + σ(q̂) after each phase.  Returns the improved policy
        softmax(logits + σ(completed Q)) — the training target —, the root value, and the surviving action.
        ``greedy``: no noise (evaluation)."""
        cfg = self.cfg
        latent, logits, value = self.initial(obs)
        n, dev, A = latent.shape[0], latent.device, cfg.n_actions
        kern = self.use_kernels if self.use_kernels is not None else dev.type == "cuda"
        if self.tree is None or self.tree.n != n or self.tree.L != latent.shape[1] or self.tree.visit.device != dev:
            self.tree = MCTSTree(n, cfg, latent.shape[1], dev)
        t = self.tree
        t.reset()
        logits = logits.float()
        if legal is not None:
            logits = logits.masked_fill(~legal, -1e9)
        pri = torch.softmax(logits, -1)
        t.latent[:, 0] = latent.float()
        t.visit[:, 0] = 1.0
        t.value_sum[:, 0] = value.float()
        ar = torch.arange(n, device=dev)
        if greedy:
            g = torch.zeros(n, A, device=dev)
        else:
            u = torch.rand(n, A, device=dev, generator=generator).clamp(1e-9, 1 - 1e-9)
            g = -torch.log(-torch.log(u))
        m = min(cfg.gumbel_considered, A)
        cand = (g + logits).topk(m, dim=1).indices                                  # [n, m], best first
        budget, used = cfg.n_simulations, 0
        phases = max(1, int(torch.ceil(torch.log2(torch.tensor(float(m)))).item()))
        eye = torch.eye(A, device=dev)

        def q_and_counts():
            ch = t.children[:, 0].long()
            nc = torch.where(ch >= 0, t.visit[ar[:, None], ch.clamp(min=0)], torch.zeros(n, A, device=dev))
            q = t.reward[ar[:, None], ch.clamp(min=0)] + cfg.discount * t.value_sum[ar[:, None], ch.clamp(min=0)] / nc.clamp(min=1)
            return torch.where(nc > 0, q, torch.zeros_like(q)), nc

        def sigma(q, nc):
            lo = torch.where(nc > 0, q, torch.full_like(q, float("inf"))).min(1, keepdim=True).values
            hi = torch.where(nc > 0, q, torch.full_like(q, float("-inf"))).max(1, keepdim=True).values
            lo, hi = torch.minimum(lo, value.float()[:, None]), torch.maximum(hi, value.float()[:, None])
            qn = (q - lo) / (hi - lo).clamp(min=1e-6)
            return (cfg.gumbel_c_visit + nc.max(1, keepdim=True).values) * cfg.gumbel_c_scale * qn

        cur = m
        for ph in range(phases):
            per = max(1, budget // (phases * cur))
            for rep in range(per):
                for k in range(cur):
                    if used >= budget:
                        break
                    t.prior[:, 0] = eye[cand[:, k]]
                    self._simulate(t, kern, ar)
                    used += 1
            if cur == 1:
                break
            q, nc = q_and_counts()
            score = (g + logits + sigma(q, nc)).gather(1, cand[:, :cur])
            order = score.argsort(dim=1, descending=True)
            cand = torch.cat([cand[:, :cur].gather(1, order), cand[:, cur:]], 1)
            cur = max(1, cur // 2)
        while used < budget:                                                        # leftover budget goes to the survivor
            t.prior[:, 0] = eye[cand[:, 0]]
            self._simulate(t, kern, ar)
            used += 1
        q, nc = q_and_counts()
        score = (g + logits + sigma(q, nc)).gather(1, cand[:, :cur])
        action = cand[:, :cur].gather(1, score.argmax(1, keepdim=True))[:, 0]
        # completed Q: visited actions keep their estimate, the others take the root value
        completed = torch.where(nc > 0, q, value.float()[:, None].expand(n, A))
        improved = torch.softmax(logits + sigma(completed, torch.where(nc > 0, nc, torch.ones_like(nc)) * (nc.max(1, keepdim=True).values > 0)), -1)
        t.prior[:, 0] = pri
        root_value = t.value_sum[:, 0] / t.visit[:, 0]
        return improved, root_value, action


class SampledMCTS:
    """Tree search over continuous (or very large) action spaces: every node carries ``K`` actions SAMPLED from the policy at
    that node, and the tree branches over those K slots (Sampled MuZero).  The priors of the slots are uniform — the
    samples already follow the policy, so the visit counts of the slots estimate the improved policy relative to it.

    ``initial(obs) → (latent, policy_params, value)``, ``recurrent(latent, action [n, act_dim]) → (latent', reward, policy_params',
    value')``, ``sample(policy_params, K, generator) → actions [n, K, act_dim]``.  ``search`` returns the root's sampled actions,
    their visit-count weights, the root value and the chosen action vector."""

    def __init__(self, cfg: MCTSConfig, initial: Callable, recurrent: Callable, sample: Callable, act_dim: int,
                 use_kernels: Optional[bool] = None):
        self.K, self.act_dim, self.sample = cfg.n_actions, act_dim, sample
        self._initial, self._recurrent = initial, recurrent
        self.node_actions = None
        self._gen = None
        self.inner = BatchedMCTS(cfg, self._init_cb, self._rec_cb, use_kernels)

    def _init_cb(self, obs):
        latent, params, value = self._initial(obs)
        n, dev = latent.shape[0], latent.device
        N = self.inner.cfg.n_simulations + 1
        if self.node_actions is None or self.node_actions.shape[0] != n or self.node_actions.device != dev:
            self.node_actions = torch.zeros(n, N, self.K, self.act_dim, device=dev)
        self.node_actions[:, 0] = self.sample(params, self.K, self._gen)
        return latent, torch.zeros(n, self.K, device=dev), value

    def _rec_cb(self, latent, slot):
        t = self.inner.tree
        ar = torch.arange(latent.shape[0], device=latent.device)
        action = self.node_actions[ar, t.leaf_parent.long(), slot]
        nl, r, params, v = self._recurrent(latent, action)
        new = t.n_nodes.long().clamp(max=t.N - 1)                       # the index the expansion is about to use
        self.node_actions[ar, new] = self.sample(params, self.K, self._gen)
        return nl, r, torch.zeros(latent.shape[0], self.K, device=latent.device), v

    @torch.no_grad()
    def search(self, obs, temperature: float = 0.0, generator=None):
        self._gen = generator
        weights, value, slot = self.inner.search(obs, temperature=temperature, generator=generator)
        actions = self.node_actions[:, 0].clone()
        chosen = actions[torch.arange(actions.shape[0], device=actions.device), slot]
        return actions, weights, value, chosen
