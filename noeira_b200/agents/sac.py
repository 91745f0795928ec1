"""SAC and TD3 (continuous control, off-policy) on the explicit-VJP nn layer; run on CPU (fp32) or GPU (bf16).

Pipeline of one update (noeira/deep_agents/sac/trainer.mojo:11-19,604-703):
    sample → target y = r + γ(1−d)(min Q_targ(s′,a′) − α log π(a′|s′)) → twin-critic MSE step →
    actor loss mean(α log π − min Q(s, a_π)) with the critics' parameters held fixed → temperature step
    (ScalarAdam on ln α, gradient −(mean log π + H_target), H_target = −ACT, α₀ = 0.2) → Polyak(τ).
Networks (noeira/deep_agents/sac/config.mojo:52-74): actor = StochasticActor(trunk 2×LinearReLU, heads μ / ln σ),
critic = Sequential(LinearReLU(OBS+ACT,H), LinearReLU(H,H), Linear(H,1)), two of them with Polyak targets.
Squashed Gaussian (noeira/deep_agents/loss/squashed_gaussian.mojo): ln σ clamped to [−5, 2] with zero gradient
where clamped; u = μ + σ z, a = c·tanh u, log π = Σ(−½z² − ln σ − ½ ln 2π − ln(c(1−tanh²u) + 1e-6)).
Checkpoint layout: actor, critic 1, critic 2 in pack order in ONE file without prefixes plus K scalars
``alpha.*`` / ``total_train_steps`` (noeira/deep_agents/sac/trainer.mojo:1083-1103).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from ..data.replay import StoreReplay

LOG2PI = math.log(2 * math.pi)


@dataclass
class SACConfig:
    obs_dim: int = 17
    act_dim: int = 6
    hidden: int = 256
    batch: int = 256
    actor_lr: float = 3e-4
    critic_lr: float = 3e-4
    alpha_lr: float = 3e-4
    gamma: float = 0.99
    tau: float = 0.005
    init_alpha: float = 0.2
    action_scale: float = 1.0
    auto_entropy: bool = True
    seed: int = 0


def make_sac_actor(obs, act, hidden):
    return nn.StochasticActor(nn.Sequential(nn.LinearReLU(obs, hidden, need_input_grad=False), nn.LinearReLU(hidden, hidden)),
                              hidden, act)


def make_critic(obs, act, hidden):
    return nn.Sequential(nn.LinearReLU(obs + act, hidden), nn.LinearReLU(hidden, hidden), nn.Linear(hidden, 1, out_fp32=True))


class SquashedGaussian:
    """Reparameterised tanh-Gaussian with explicit backward."""

    LS_MIN, LS_MAX = -5.0, 2.0

    def __init__(self, act_dim, scale=1.0):
        self.A, self.c = act_dim, scale

    def forward(self, packed, z):
        p = packed.float()
        mu, ls_raw = p[:, : self.A], p[:, self.A: 2 * self.A]
        ls = ls_raw.clamp(self.LS_MIN, self.LS_MAX)
        self._free = ((ls_raw > self.LS_MIN) & (ls_raw < self.LS_MAX)).float()
        sd = ls.exp()
        u = mu + sd * z
        y = torch.tanh(u)
        self._sd_z, self._y = sd * z, y
        a = self.c * y
        logp = (-0.5 * z * z - ls - 0.5 * LOG2PI - torch.log(self.c * (1 - y * y) + 1e-6)).sum(1)
        return a, logp

    def vjp(self, da, dlogp):
        """da [B, A] (dL/da), dlogp [B] (dL/dlogπ) → gradient of the packed [μ | ln σ]."""
        y = self._y
        one = 1 - y * y
        gu = 2 * self.c * y * one / (self.c * one + 1e-6)          # d logπ / du
        du = da * self.c * one + dlogp[:, None] * gu
        dls = (du * self._sd_z - dlogp[:, None]) * self._free
        return torch.cat([du, dls], 1)


class SACTrainer:
    def __init__(self, cfg: SACConfig = None, device="cpu"):
        self.cfg = cfg = cfg or SACConfig()
        self.device = torch.device(device)
        nn.manual_seed(cfg.seed)
        O, A, H = cfg.obs_dim, cfg.act_dim, cfg.hidden
        self.actor = make_sac_actor(O, A, H).to(self.device)
        self.q1, self.q2 = make_critic(O, A, H).to(self.device), make_critic(O, A, H).to(self.device)
        self.q1t, self.q2t = make_critic(O, A, H).to(self.device), make_critic(O, A, H).to(self.device)
        self.q1t.copy_from(self.q1)
        self.q2t.copy_from(self.q2)
        self.actor_opt = nn.Adam(self.actor.named_params(), lr=cfg.actor_lr)
        self.critic_opt = nn.Adam(list(self.q1.named_params("q1.")) + list(self.q2.named_params("q2.")), lr=cfg.critic_lr)
        self.target_arena = nn.ParamArena(list(self.q1t.named_params("q1.")) + list(self.q2t.named_params("q2.")),
                                          with_moments=False)
        self.alpha_opt = nn.ScalarAdam(cfg.init_alpha, cfg.alpha_lr, device=self.device)
        self.target_entropy = -float(A)
        self.dist = SquashedGaussian(A, cfg.action_scale)
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.total_train_steps = 0
        self.metrics = {}
        self._pad = (O + A + 7) // 8 * 8 if self.device.type == "cuda" else O + A

    # ------------------------------------------------------------------ helpers
    def _act_in(self, x):
        if self.device.type == "cuda":
            w = (x.shape[1] + 7) // 8 * 8
            out = torch.zeros(x.shape[0], w, device=self.device, dtype=torch.bfloat16)
            out[:, : x.shape[1]] = x
            return out[:, : x.shape[1]]
        return x

    def _sa(self, s, a):
        return self._act_in(torch.cat([s.float(), a.float()], 1))

    def _noise(self, n):
        return torch.randn(n, self.cfg.act_dim, device=self.device, generator=self.gen)

    @property
    def alpha(self):
        return self.alpha_opt.alpha

    def select_action(self, obs, deterministic=False):
        packed = self.actor.forward(self._act_in(obs))
        if deterministic:
            return self.cfg.action_scale * torch.tanh(packed.float()[:, : self.cfg.act_dim])
        a, _ = self.dist.forward(packed, self._noise(obs.shape[0]))
        return a

    # ------------------------------------------------------------------ update
    # ------------------------------------------------------------------ update on the device: GEMMs + glue kernels only
    def _glue(self, B):
        """Buffers of the kernel path for batch size ``B`` (allocated once: a captured update keeps their addresses)."""
        g = getattr(self, "_glue_buf", None)
        if g is None or g["B"] != B:
            c, dev = self.cfg, self.device
            f = dict(device=dev, dtype=torch.float32)
            h = dict(device=dev, dtype=torch.bfloat16)
            nblk = (B + 255) // 256
            g = self._glue_buf = dict(
                B=B, sa=torch.zeros(B, self._pad, **h), sa2=torch.zeros(B, self._pad, **h), act=torch.zeros(B, c.act_dim, **f),
                logp=torch.zeros(B, **f), logp2=torch.zeros(B, **f), y=torch.zeros(B, **f),
                ysq=torch.zeros(B, c.act_dim, **f), sdz=torch.zeros(B, c.act_dim, **f),
                free=torch.zeros(B, c.act_dim, device=dev, dtype=torch.uint8), dq1=torch.zeros(B, 8, **h), dq2=torch.zeros(B, 8, **h),
                dpacked=torch.zeros(B, (2 * c.act_dim + 7) // 8 * 8, **h), partials=torch.zeros(3 * nblk + 8, **f),
                closs=torch.zeros(1, **f), stats=torch.zeros(3, **f))
        return g

    def _update_kernels(self, s, a, r, sp, d):
        """The same update as ``update`` with every elementwise stage in ``csrc/sac_kernels.cu``: sample + log-probability +
        critic input rows in one launch, target, critic gradients, critic choice for the actor loss, and the squashed
        Gaussian's backward; reductions are two-pass and deterministic."""
        import ctypes
        from .._native import check, cuda_lib, ptr, stream_ptr
        cfg, lib, B = self.cfg, cuda_lib(), s.shape[0]
        O, A, ci = cfg.obs_dim, cfg.act_dim, ctypes.c_int
        g = self._glue(B)
        s, a, sp = s.float().contiguous(), a.float().contiguous(), sp.float().contiguous()
        r, d = r.float().contiguous(), d.float().contiguous()
        alpha = self.alpha_opt.alpha
        st = stream_ptr()
        scale = ctypes.c_float(cfg.action_scale)

        def sample(obs, noise, sa, logp, save):
            packed = self.actor.forward(self._act_in(obs))
            packed = packed if packed.dtype == torch.float32 else packed.float()
            check(lib.nb_sac_sample(ptr(packed), ci(packed.stride(0)), ptr(noise), ptr(obs), ci(obs.stride(0)), ptr(g["act"]), ptr(logp),
                                    ptr(g["ysq"]) if save else None, ptr(g["sdz"]) if save else None, ptr(g["free"]) if save else None,
                                    ptr(sa), ci(sa.stride(0)), ci(B), ci(O), ci(A), scale, st), "sac_sample")

        def qpair(q1, q2, sa):
            x = sa[:, : O + A]
            return q1.forward(x), q2.forward(x)

        # ---- target
        sample(sp, self._noise(B), g["sa"], g["logp"], False)
        q1t, q2t = qpair(self.q1t, self.q2t, g["sa"])
        check(lib.nb_sac_target(ptr(q1t), ci(q1t.stride(0)), ptr(q2t), ci(q2t.stride(0)), ptr(g["logp"]), ptr(r), ptr(d), ptr(alpha),
                                ctypes.c_float(cfg.gamma), ptr(g["y"]), ci(B), st), "sac_target")
        # ---- critics
        check(lib.nb_sac_pack_sa(ptr(s), ci(s.stride(0)), ptr(a), ci(a.stride(0)), ptr(g["sa2"]), ci(g["sa2"].stride(0)), ci(B), ci(O),
                                 ci(A), st), "sac_pack_sa")
        q1v, q2v = qpair(self.q1, self.q2, g["sa2"])
        check(lib.nb_sac_critic_grad(ptr(q1v), ci(q1v.stride(0)), ptr(q2v), ci(q2v.stride(0)), ptr(g["y"]), ptr(g["dq1"]), ptr(g["dq2"]),
                                     ci(8), ptr(g["partials"]), ptr(g["closs"]), ci(B), st), "sac_critic_grad")
        self.q1.vjp(g["dq1"][:, :1])
        self.q2.vjp(g["dq2"][:, :1])
        self.critic_opt.step(zero_grad=True)
        # ---- actor (critic parameters fixed)
        sample(s, self._noise(B), g["sa"], g["logp2"], True)
        q1v, q2v = qpair(self.q1, self.q2, g["sa"])
        check(lib.nb_sac_actor_qgrad(ptr(q1v), ci(q1v.stride(0)), ptr(q2v), ci(q2v.stride(0)), ptr(g["logp2"]), ptr(alpha), ptr(g["dq1"]),
                                     ptr(g["dq2"]), ci(8), ptr(g["partials"]), ptr(g["stats"]), ci(B), st), "sac_actor_qgrad")
        ps = [p for q in (self.q1, self.q2) for p in q.params()]
        for p in ps:
            p.frozen = True
        d1 = self.q1.vjp(g["dq1"][:, :1])
        d2 = self.q2.vjp(g["dq2"][:, :1])
        for p in ps:
            p.frozen = False
        d1 = d1 if d1.dtype == torch.bfloat16 else d1.to(torch.bfloat16)
        d2 = d2 if d2.dtype == torch.bfloat16 else d2.to(torch.bfloat16)
        check(lib.nb_sac_dist_bwd(ptr(d1), ci(d1.stride(0)), ptr(d2), ci(d2.stride(0)), ptr(g["ysq"]), ptr(g["sdz"]), ptr(g["free"]),
                                  ptr(alpha), ptr(g["dpacked"]), ci(g["dpacked"].stride(0)), ci(B), ci(O), ci(A), scale, st),
              "sac_dist_bwd")
        self.actor.vjp(g["dpacked"][:, : 2 * A])
        self.actor_opt.step(zero_grad=True)
        if cfg.auto_entropy:
            self.alpha_opt.step_alpha(g["stats"][1:2], self.target_entropy)
        nn.polyak(self.target_arena, self.critic_opt.arena, cfg.tau)
        self.total_train_steps += 1
        self.metrics = dict(critic_loss=g["closs"][0], actor_loss=g["stats"][0], mean_q=g["stats"][2], mean_logp=g["stats"][1])
        return self.metrics

    def update(self, s, a, r, sp, d):
        cfg = self.cfg
        if self.device.type == "cuda" and getattr(self, "use_kernels", True):
            return self._update_kernels(s, a, r, sp, d)
        B = s.shape[0]
        alpha = float(self.alpha) if self.device.type == "cpu" else self.alpha
        # ---- target
        ap, logpp = self.dist.forward(self.actor.forward(self._act_in(sp)), self._noise(B))
        sap = self._sa(sp, ap)
        qt = torch.minimum(self.q1t.forward(sap).float()[:, 0], self.q2t.forward(sap).float()[:, 0])
        y = r + cfg.gamma * (1 - d) * (qt - alpha * logpp)
        # ---- critics
        sa = self._sa(s, a)
        closs = 0.0
        for q in (self.q1, self.q2):
            qv = q.forward(sa).float()[:, 0]
            diff = qv - y
            closs = closs + (diff * diff).mean()
            q.vjp((2.0 / B * diff)[:, None])
        self.critic_opt.step(zero_grad=True)
        # ---- actor (critic parameters fixed)
        packed = self.actor.forward(self._act_in(s))
        api, logpi = self.dist.forward(packed, self._noise(B))
        sapi = self._sa(s, api)
        q1v, q2v = self.q1.forward(sapi).float()[:, 0], self.q2.forward(sapi).float()[:, 0]
        use1 = (q1v <= q2v).float()
        aloss = (alpha * logpi - torch.minimum(q1v, q2v)).mean()
        ps = [p for q in (self.q1, self.q2) for p in q.params()]
        for p in ps:
            p.frozen = True
        d1 = self.q1.vjp((-use1 / B)[:, None])
        d2 = self.q2.vjp((-(1 - use1) / B)[:, None])
        for p in ps:
            p.frozen = False
        da = (d1.float() + d2.float())[:, cfg.obs_dim: cfg.obs_dim + cfg.act_dim]
        dpacked = self.dist.vjp(da, torch.full((B,), 1.0, device=self.device) * alpha / B)
        self.actor.vjp(dpacked if self.device.type == "cpu" else dpacked.to(torch.bfloat16))
        self.actor_opt.step(zero_grad=True)
        # ---- temperature
        if cfg.auto_entropy:
            self.alpha_opt.step_alpha(logpi.mean().reshape(1) if self.device.type == "cuda" else logpi.mean(), self.target_entropy)
        # ---- Polyak
        nn.polyak(self.target_arena, self.critic_opt.arena, cfg.tau)
        self.total_train_steps += 1
        self.metrics = dict(critic_loss=closs, actor_loss=aloss, mean_q=q1v.mean(), mean_logp=logpi.mean())
        return self.metrics

    def update_captured(self, s, a, r, sp, d):
        """The same update replayed from one CUDA graph (captured on the third call; batch shape fixed).  The noise
        generator is registered with the graph, so every replay draws fresh samples
        (noeira/deep_agents/sac/trainer.mojo:604-703 ``train_device_kernels`` is the reference's capture body)."""
        if self.device.type != "cuda":
            return self.update(s, a, r, sp, d)
        if getattr(self, "_graphed", None) is None:
            from ..utils.graphs import GraphedStep
            self._graphed = GraphedStep(self.update, [s, a, r, sp, d], generators=[self.gen])
        before = self.total_train_steps
        out = self._graphed(s, a, r, sp, d)
        self.total_train_steps = before + 1
        return out

    # ------------------------------------------------------------------ persistence (reference layout)
    def save(self, path, with_moments: bool = True):
        """Actor, critic 1, critic 2 in pack order plus the temperature state and the step counter as K scalars
        (noeira/deep_agents/sac/trainer.mojo:1083-1103).  ``with_moments=False`` writes exactly the reference's
        sections (its resume re-warms the moments and restarts the targets from the online critics).
        ``with_moments=True`` is the exact-resume form: Adam's m / v, the optimizers' step counters and
        bias-correction products, and the two target critics (two more modules after critic 2) are stored as well,
        so a resumed run continues bit for bit."""
        from ..io.checkpoint import save_params_multi
        st = self.alpha_opt.state.cpu().tolist()
        sc = {"alpha.log_alpha": st[0], "alpha.m": st[1], "alpha.v": st[2], "alpha.b1t": st[3], "alpha.b2t": st[4],
              "alpha.alpha": st[5], "total_train_steps": float(self.total_train_steps)}
        mods = [self.actor, self.q1, self.q2]
        if with_moments:
            sc.update({f"actor_opt.{k}": v for k, v in self.actor_opt.scalars().items()})
            sc.update({f"critic_opt.{k}": v for k, v in self.critic_opt.scalars().items()})
            mods += [self.q1t, self.q2t]
        save_params_multi(path, mods, sc, with_moments=with_moments)

    def load(self, path):
        from ..io.checkpoint import CheckpointError, load_params_multi
        try:
            sc = load_params_multi(path, [self.actor, self.q1, self.q2, self.q1t, self.q2t], load_moments=True)
            exact = "actor_opt.t" in sc
        except CheckpointError:
            sc = load_params_multi(path, [self.actor, self.q1, self.q2], load_moments=False)
            exact = False
        if "alpha.log_alpha" in sc:
            self.alpha_opt.state.copy_(torch.tensor([sc[k] for k in ("alpha.log_alpha", "alpha.m", "alpha.v", "alpha.b1t",
                                                                     "alpha.b2t", "alpha.alpha")]))
        self.total_train_steps = int(sc.get("total_train_steps", 0))
        if exact:
            # moments are only meaningful together with their step counters: both are restored, or neither
            self.actor_opt.load_scalars({k.split(".", 1)[1]: v for k, v in sc.items() if k.startswith("actor_opt.")})
            self.critic_opt.load_scalars({k.split(".", 1)[1]: v for k, v in sc.items() if k.startswith("critic_opt.")})
        else:
            self.q1t.copy_from(self.q1)
            self.q2t.copy_from(self.q2)
        for o in (self.actor_opt, self.critic_opt):
            if o.arena.shadow is not None:
                o.arena.refresh_shadow()
        if getattr(self.target_arena, "shadow", None) is not None:
            self.target_arena.refresh_shadow()


class SACAgent:
    """Facade: drives a BatchedEnv with a replay buffer (noeira/deep_agents/sac/agent.mojo:58,
    run_offpolicy_train_batched noeira/deep_agents/training/driver_offpolicy.mojo:823)."""

    def __init__(self, env, cfg: SACConfig = None, capacity=1_000_000, learning_starts=1000, utd=1):
        self.env = env
        cfg = cfg or SACConfig(obs_dim=env.obs_dim, act_dim=env.act_dim)
        self.trainer = SACTrainer(cfg, device=env.device)
        self.replay = StoreReplay(capacity, env.obs_dim, env.act_dim, device=env.device, seed=cfg.seed)
        self.learning_starts, self.utd = learning_starts, utd

    def train(self, total_env_steps, logger=None, log_every=1000, checkpoint_path: str = "", checkpoint_every: int = 0):
        """Runs the generic off-policy driver (``training.rl.run_offpolicy_train_batched``)."""
        from ..training.rl import run_offpolicy_train_batched

        class _Scalars:
            def __init__(self, inner):
                self.inner = inner

            def log_scalars(self, step, row):
                (self.inner.log_scalars if hasattr(self.inner, "log_scalars") else self.inner.log)(step, row)
        self.log = run_offpolicy_train_batched(self.trainer, self.env, self.replay, total_env_steps,
                                               learning_starts=self.learning_starts, utd=self.utd, batch_size=self.trainer.cfg.batch,
                                               print_every=log_every, logger=_Scalars(logger) if logger is not None else None,
                                               checkpoint_every=checkpoint_every, checkpoint_path=checkpoint_path)
        return self.trainer.metrics


# ------------------------------------------------------------------------------------------ TD3
@dataclass
class TD3Config:
    obs_dim: int = 17
    act_dim: int = 6
    hidden: int = 256
    batch: int = 256
    actor_lr: float = 3e-4
    critic_lr: float = 3e-4
    gamma: float = 0.99
    tau: float = 0.005
    policy_noise: float = 0.2
    noise_clip: float = 0.5
    policy_delay: int = 2
    explore_noise: float = 0.1
    action_scale: float = 1.0
    seed: int = 0


class TD3Trainer:
    """Deterministic actor + Gaussian exploration, target-policy smoothing, delayed actor / target updates
    (noeira/deep_agents/td3/trainer.mojo:84, target_y_block.mojo:79, blocks/delayed_actor_polyak_step.mojo:28)."""

    def __init__(self, cfg: TD3Config = None, device="cpu"):
        self.cfg = cfg = cfg or TD3Config()
        self.device = torch.device(device)
        nn.manual_seed(cfg.seed)
        O, A, H = cfg.obs_dim, cfg.act_dim, cfg.hidden
        mk_actor = lambda: nn.Sequential(nn.LinearReLU(O, H, need_input_grad=False), nn.LinearReLU(H, H),
                                         nn.Linear(H, A, act="tanh", out_fp32=False))
        self.actor, self.actor_t = mk_actor().to(self.device), mk_actor().to(self.device)
        self.actor_t.copy_from(self.actor)
        self.q1, self.q2 = make_critic(O, A, H).to(self.device), make_critic(O, A, H).to(self.device)
        self.q1t, self.q2t = make_critic(O, A, H).to(self.device), make_critic(O, A, H).to(self.device)
        self.q1t.copy_from(self.q1)
        self.q2t.copy_from(self.q2)
        self.actor_opt = nn.Adam(self.actor.named_params(), lr=cfg.actor_lr)
        self.critic_opt = nn.Adam(list(self.q1.named_params("q1.")) + list(self.q2.named_params("q2.")), lr=cfg.critic_lr)
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed + 1)
        self.total_train_steps = 0

    _act_in = SACTrainer._act_in
    _sa = SACTrainer._sa

    def select_action(self, obs, explore=True):
        a = self.cfg.action_scale * self.actor.forward(self._act_in(obs)).float()
        if explore:
            a = (a + self.cfg.explore_noise * torch.randn(a.shape, device=self.device, generator=self.gen)).clamp(
                -self.cfg.action_scale, self.cfg.action_scale)
        return a

    def _update_kernels(self, s, a, r, sp, d):
        """The same update with the elementwise stages in ``csrc/sac_kernels.cu`` (smoothed target action + critic input rows,
        target, critic gradients, actor gradient, deterministic loss reductions)."""
        import ctypes
        from .._native import check, cuda_lib, ptr, stream_ptr
        cfg, lib, B = self.cfg, cuda_lib(), s.shape[0]
        O, A, ci, cf = cfg.obs_dim, cfg.act_dim, ctypes.c_int, ctypes.c_float
        g = getattr(self, "_glue_buf", None)
        if g is None or g["B"] != B:
            f = dict(device=self.device, dtype=torch.float32)
            h = dict(device=self.device, dtype=torch.bfloat16)
            pad = (O + A + 7) // 8 * 8
            g = self._glue_buf = dict(B=B, sa=torch.zeros(B, pad, **h), sa2=torch.zeros(B, pad, **h), y=torch.zeros(B, **f),
                                      dq1=torch.zeros(B, 8, **h), dq2=torch.zeros(B, 8, **h), dqa=torch.zeros(B, 8, **h),
                                      da=torch.zeros(B, (A + 7) // 8 * 8, **h), partials=torch.zeros((B + 255) // 256 + 8, **f),
                                      closs=torch.zeros(1, **f), aloss=torch.zeros(1, **f))
            g["dqa"][:, 0] = -1.0 / B
        s, a, sp = s.float().contiguous(), a.float().contiguous(), sp.float().contiguous()
        r, d = r.float().contiguous(), d.float().contiguous()
        st = stream_ptr()
        z = torch.randn(B, A, device=self.device, generator=self.gen)
        at = self.actor_t.forward(self._act_in(sp))
        check(lib.nb_td3_pack(ptr(sp), ci(sp.stride(0)), ptr(at), ci(at.stride(0)), ptr(z) if cfg.policy_noise > 0 else None,
                              cf(cfg.policy_noise), cf(cfg.noise_clip), cf(cfg.action_scale), ptr(g["sa"]), ci(g["sa"].stride(0)), ci(B),
                              ci(O), ci(A), st), "td3_pack")
        x = g["sa"][:, : O + A]
        q1t, q2t = self.q1t.forward(x), self.q2t.forward(x)
        check(lib.nb_sac_target(ptr(q1t), ci(q1t.stride(0)), ptr(q2t), ci(q2t.stride(0)), None, ptr(r), ptr(d), None, cf(cfg.gamma),
                                ptr(g["y"]), ci(B), st), "td3_target")
        check(lib.nb_sac_pack_sa(ptr(s), ci(s.stride(0)), ptr(a), ci(a.stride(0)), ptr(g["sa2"]), ci(g["sa2"].stride(0)), ci(B), ci(O),
                                 ci(A), st), "sac_pack_sa")
        x2 = g["sa2"][:, : O + A]
        q1v, q2v = self.q1.forward(x2), self.q2.forward(x2)
        check(lib.nb_sac_critic_grad(ptr(q1v), ci(q1v.stride(0)), ptr(q2v), ci(q2v.stride(0)), ptr(g["y"]), ptr(g["dq1"]), ptr(g["dq2"]),
                                     ci(8), ptr(g["partials"]), ptr(g["closs"]), ci(B), st), "sac_critic_grad")
        self.q1.vjp(g["dq1"][:, :1])
        self.q2.vjp(g["dq2"][:, :1])
        self.critic_opt.step(zero_grad=True)
        self.total_train_steps += 1
        out = dict(critic_loss=g["closs"][0])
        if self.total_train_steps % cfg.policy_delay == 0:
            api = self.actor.forward(self._act_in(s))
            check(lib.nb_td3_pack(ptr(s), ci(s.stride(0)), ptr(api), ci(api.stride(0)), None, cf(0.0), cf(0.0), cf(cfg.action_scale),
                                  ptr(g["sa"]), ci(g["sa"].stride(0)), ci(B), ci(O), ci(A), st), "td3_pack")
            q1pi = self.q1.forward(g["sa"][:, : O + A])
            check(lib.nb_column_sum(ptr(q1pi), ci(q1pi.stride(0)), ptr(g["partials"]), ptr(g["aloss"]), cf(-1.0 / B), ci(B), st), "column_sum")
            ps = self.q1.params()
            for p in ps:
                p.frozen = True
            dsa = self.q1.vjp(g["dqa"][:, :1])
            for p in ps:
                p.frozen = False
            dsa = dsa if dsa.dtype == torch.bfloat16 else dsa.to(torch.bfloat16)
            check(lib.nb_td3_actor_grad(ptr(dsa), ci(dsa.stride(0)), ptr(g["da"]), ci(g["da"].stride(0)), ci(B), ci(O), ci(A),
                                        cf(cfg.action_scale), st), "td3_actor_grad")
            self.actor.vjp(g["da"][:, :A])
            self.actor_opt.step(zero_grad=True)
            for t, o in ((self.actor_t, self.actor), (self.q1t, self.q1), (self.q2t, self.q2)):
                t.polyak_from(o, cfg.tau)
            out["actor_loss"] = g["aloss"][0]
        return out

    def update(self, s, a, r, sp, d):
        cfg, B = self.cfg, s.shape[0]
        if self.device.type == "cuda" and getattr(self, "use_kernels", True):
            return self._update_kernels(s, a, r, sp, d)
        noise = (torch.randn(B, cfg.act_dim, device=self.device, generator=self.gen) * cfg.policy_noise).clamp(
            -cfg.noise_clip, cfg.noise_clip)
        ap = (cfg.action_scale * self.actor_t.forward(self._act_in(sp)).float() + noise).clamp(-cfg.action_scale, cfg.action_scale)
        sap = self._sa(sp, ap)
        y = r + cfg.gamma * (1 - d) * torch.minimum(self.q1t.forward(sap).float()[:, 0], self.q2t.forward(sap).float()[:, 0])
        sa = self._sa(s, a)
        closs = 0.0
        for q in (self.q1, self.q2):
            diff = q.forward(sa).float()[:, 0] - y
            closs = closs + (diff * diff).mean()
            q.vjp((2.0 / B * diff)[:, None])
        self.critic_opt.step(zero_grad=True)
        self.total_train_steps += 1
        out = dict(critic_loss=closs)
        if self.total_train_steps % cfg.policy_delay == 0:
            api = self.actor.forward(self._act_in(s))
            q1v = self.q1.forward(self._sa(s, cfg.action_scale * api.float()))
            ps = self.q1.params()
            for p in ps:
                p.frozen = True
            dsa = self.q1.vjp(torch.full((B, 1), -1.0 / B, device=self.device))
            for p in ps:
                p.frozen = False
            da = dsa.float()[:, cfg.obs_dim: cfg.obs_dim + cfg.act_dim] * cfg.action_scale
            self.actor.vjp(da if self.device.type == "cpu" else da.to(torch.bfloat16))
            self.actor_opt.step(zero_grad=True)
            for t, o in ((self.actor_t, self.actor), (self.q1t, self.q1), (self.q2t, self.q2)):
                t.polyak_from(o, cfg.tau)
            out["actor_loss"] = -q1v.float().mean()
        return out


def DDPGTrainer(cfg: TD3Config = None, device="cpu") -> TD3Trainer:
    """DDPG = TD3 without target-policy smoothing and without the delayed actor update; the twin critic stays (its
    minimum only makes the target more conservative).  (noeira/deep_agents/ddpg/)"""
    import dataclasses
    cfg = dataclasses.replace(cfg or TD3Config(), policy_noise=0.0, noise_clip=0.0, policy_delay=1)
    return TD3Trainer(cfg, device)
