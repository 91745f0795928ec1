"""PPO (continuous actions) with an on-device rollout.

Pipeline per iteration (the host only enqueues; nothing is copied to the host inside it):

    rollout   T × { actor fwd, critic fwd (tcgen05 GEMMs, fused bias+tanh) → sample kernel →
                    fused physics env step writing reward/done/next-obs straight into slot t and the
                    post-reset observation into slot t+1 }
    gae       critic fwd over all T·N bootstrap states → reverse-scan GAE kernel
    update    E·K × { gather minibatch by a keyed bijective shuffle → actor fwd → clipped-surrogate
                      kernel (loss + dμ + d ln σ) → actor vjp → [fused gradient all-reduce +] Adam →
                      critic fwd → value-loss kernel → critic vjp → Adam }

Each of the three phases is captured once in a CUDA graph and replayed; counters that change between
replays (minibatch index, rollout index, RNG offset, Adam step / β powers) live on the device.

Reference: PPOTrainer noeira/deep_agents/ppo/trainer.mojo:185 (device rollout :933-940, update
:837-915), driver noeira/deep_agents/training/driver_onpolicy.mojo:479,1005-1091, preset
noeira/deep_agents/ppo/config.mojo:51-134 (separate Adam per net, actor lr 3e-4, critic lr 1e-3,
γ 0.99, λ 0.95, clip 0.2, ln σ init −0.5).  Parameter names: ``actor.{0,1,2}.*`` (+ ``actor.2.log_std``),
``critic.{0,1,2}.*``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import nn
from .. import _native
from .._native import check, cuda_lib, ptr, stream_ptr
from ..ops.streams import Branch


@dataclass
class PPOConfig:
    n_envs: int = 4096
    rollout_len: int = 32
    n_epochs: int = 4
    n_minibatches: int = 8
    hidden: int = 256
    actor_lr: float = 3e-4
    critic_lr: float = 1e-3
    gamma: float = 0.99
    gae_lambda: float = 0.95
    clip_eps: float = 0.2
    entropy_coef: float = 0.0
    action_scale: float = 1.0
    log_std_init: float = -0.5
    max_grad_norm: float = 0.0
    seed: int = 0
    use_cuda_graphs: bool = True
    fused_mlp: bool = True     # actor / critic forward as one fused three-layer kernel when the shapes allow it
    precision: str = "bf16"    # "tf32": fp32 activations and master weights on the TF32 tensor-core path, layer by layer


def make_actor(obs_dim, act_dim, hidden, log_std_init=-0.5):
    return nn.Sequential(nn.LinearTanh(obs_dim, hidden, need_input_grad=False), nn.LinearTanh(hidden, hidden),
                         nn.GaussianHead(hidden, act_dim, log_std_init=log_std_init))


def make_critic(obs_dim, hidden):
    return nn.Sequential(nn.LinearTanh(obs_dim, hidden, need_input_grad=False), nn.LinearTanh(hidden, hidden),
                         nn.Linear(hidden, 1, out_fp32=True))


class PPOTrainer:
    def __init__(self, env, cfg: PPOConfig = None, grad_sync=None):
        """``grad_sync``: optional object with ``reduce_and_step(optimizer)`` that replaces the local
        optimizer step by a fused cross-GPU reduce + update (``noeira_b200.parallel.DataParallel``)."""
        self.env = env
        self.cfg = cfg = cfg or PPOConfig(n_envs=env.n_envs)
        assert cfg.n_envs == env.n_envs
        if cfg.use_cuda_graphs and not getattr(env, "graph_safe", True):
            # an environment stepped by tensor operations with its own random generator cannot sit in a captured stream
            import dataclasses
            self.cfg = cfg = dataclasses.replace(cfg, use_cuda_graphs=False)
        self.device = env.device
        self.lib = cuda_lib()
        nn.manual_seed(cfg.seed)
        self.actor = make_actor(env.obs_dim, env.act_dim, cfg.hidden, cfg.log_std_init).to(self.device)
        self.critic = make_critic(env.obs_dim, cfg.hidden).to(self.device)
        self.actor_opt = nn.Adam(self.actor.named_params("actor."), lr=cfg.actor_lr)
        self.critic_opt = nn.Adam(self.critic.named_params("critic."), lr=cfg.critic_lr)
        self.actor_opt.max_grad_norm = self.critic_opt.max_grad_norm = cfg.max_grad_norm
        self.grad_sync = grad_sync
        T, N, OP = cfg.rollout_len, cfg.n_envs, env.obs_pad
        self.AP = AP = (env.act_dim + 7) // 8 * 8
        self.pool = T * N
        assert self.pool % cfg.n_minibatches == 0
        self.mb = self.pool // cfg.n_minibatches
        f = dict(device=self.device, dtype=torch.float32)
        h = dict(device=self.device, dtype=torch.bfloat16)
        # [obs_0 .. obs_T | next_obs_0 .. next_obs_{T-1}] in one allocation: the critic evaluates the whole pool
        # in a single 3-GEMM chain after the rollout instead of 3 small GEMMs per step
        self.obs_all = torch.zeros(2 * T + 1, N, OP, **h)
        self.obs_buf = self.obs_all[: T + 1]
        self.next_obs_buf = self.obs_all[T + 1:]
        self.act_buf = torch.zeros(T, N, AP, **f)
        self.env_action = torch.zeros(N, AP, **f)
        self.logp_buf = torch.zeros(T, N, **f)
        self.rew_buf = torch.zeros(T, N, **f)
        self.done_buf = torch.zeros(T, N, **f)
        self.term_buf = torch.zeros(T, N, **f)
        self.adv_buf = torch.zeros(T, N, **f)
        self.ret_buf = torch.zeros(T, N, **f)
        # minibatch staging
        self.mb_obs = torch.zeros(self.mb, OP, **h)
        self.mb_act = torch.zeros(self.mb, AP, **f)
        self.mb_logp = torch.zeros(self.mb, **f)
        self.mb_adv = torch.zeros(self.mb, **f)
        self.mb_ret = torch.zeros(self.mb, **f)
        self.dmu = torch.zeros(self.mb, AP, **h)
        self.dv = torch.zeros(self.mb, 8, **h)
        nblk = (self.mb + 255) // 256
        self.partials = torch.zeros(max(nblk * 2, nblk * env.act_dim, nblk * 4) + 16, **f)
        self.partials2 = torch.zeros(nblk * 4 + 16, **f)
        self.partials_v = torch.zeros(nblk * 4 + 16, **f)
        self._critic_branch = Branch(torch.cuda.Stream(device=self.device), 1) if self.device.type == "cuda" else None
        self._cap_stream = torch.cuda.Stream(device=self.device)
        self._actor_pg = Branch(torch.cuda.Stream(device=self.device), 2)     # parameter-gradient branches
        self._critic_pg = Branch(torch.cuda.Stream(device=self.device), 3)
        self.actor.set_attr("grad_branch", self._actor_pg)
        self.critic.set_attr("grad_branch", self._critic_pg)
        self.adv_stats = torch.zeros(2, **f)
        # device counters: [0] minibatch index, [1] rollout index, [2] rng offset
        self.counters = torch.zeros(4, device=self.device, dtype=torch.int64)
        # metrics: [0] Σ policy loss [1] Σ KL [2] Σ clipfrac [3] Σ entropy [4] samples [5] Σ value loss·MB
        self.metrics = torch.zeros(8, **f)
        self._graphs = {}
        self._fused = {}
        self._tf32 = cfg.precision == "tf32" and self.device.type == "cuda"
        if self._tf32:
            self.actor.set_attr("precision", "tf32")
            self.critic.set_attr("precision", "tf32")
        if cfg.fused_mlp and self.device.type == "cuda" and not self._tf32:
            from ..ops.mlp import fusable
            for net in (self.actor, self.critic):
                self._fused[id(net)] = fusable(*self._layers(net))
        # fused update path: both networks through one grouped forward launch, one grouped data-gradient launch and
        # six parameter-gradient branches (one per layer) — see ops/mlp.py
        self._train_pass = None
        if self._fused.get(id(self.actor)) and self._fused.get(id(self.critic)) and not self._tf32:
            from ..ops.mlp import Mlp3Pass
            self._train_pass = (Mlp3Pass(*self._layers(self.actor), self.mb, self.device),
                                Mlp3Pass(*self._layers(self.critic), self.mb, self.device))
            self._layer_pg = [[Branch(torch.cuda.Stream(device=self.device), 4 + 3 * i + j) for j in range(3)] for i in range(2)]
        self._graph_launches = {}
        self.iteration = 0
        self.env.reset_batch()
        self.obs_buf[0].copy_(self.env.obs_bf16)

    # ------------------------------------------------------------------ phases
    def _layers(self, net):
        a, b, c = net.mods
        return a, b, (c.lin if hasattr(c, "lin") else c)

    def _forward(self, net, x, save):
        """Forward of the actor or the critic: the fused three-layer kernel when it applies, else layer by layer."""
        if self._fused.get(id(net)) and x.shape[0] >= 1024:     # one launch instead of three
            from ..ops.mlp import mlp3_forward
            l1, l2, l3 = self._layers(net)
            y = mlp3_forward(x, l1, l2, l3, save=save)
            if hasattr(net.mods[2], "lin"):
                net.mods[2]._mu = y
            return y
        return net.forward(x)          # both heads write fp32 rows (what the sampling / loss / GAE kernels read) on either path

    def _rollout(self):
        cfg, env, lib = self.cfg, self.env, self.lib
        head = self.actor.mods[2]
        for t in range(cfg.rollout_len):
            obs = self.obs_buf[t]
            mu = self._forward(self.actor, obs, save=False)
            check(lib.nb_ppo_sample(ptr(mu), ctypes.c_int(mu.stride(0)), ptr(head.log_std.storage), None,
                                    ctypes.c_int(0), ptr(self.act_buf[t]), ctypes.c_int(self.AP),
                                    ptr(self.env_action), ctypes.c_int(self.AP), ptr(self.logp_buf[t]),
                                    None, ctypes.c_int(cfg.n_envs), ctypes.c_int(env.act_dim),
                                    ctypes.c_float(cfg.action_scale), ctypes.c_ulonglong(cfg.seed * 7919 + 13),
                                    ptr(self.counters), ctypes.c_int(t), ctypes.c_int(0), stream_ptr()), "ppo_sample")
            env.engine.step(self.env_action, self.rew_buf[t], self.done_buf[t], self.term_buf[t],
                            obs_bf16=self.obs_buf[t + 1], next_obs_bf16=self.next_obs_buf[t], ep_stats=env.ep_stats)
        check(lib.nb_ppo_counter_add(ptr(self.counters), ctypes.c_int(2), ctypes.c_int(cfg.rollout_len), stream_ptr()), "counter")

    def _gae(self):
        cfg = self.cfg
        T, N = cfg.rollout_len, cfg.n_envs
        v_all = self.critic.forward(self.obs_all.view((2 * T + 1) * N, -1))      # V(obs_t), V(obs_T), V(next_obs_t)
        vnext = v_all[(T + 1) * N:]
        check(self.lib.nb_ppo_gae(ptr(self.rew_buf), ptr(self.done_buf), ptr(self.term_buf), ptr(v_all),
                                  ctypes.c_int(v_all.stride(0)),
                                  ptr(vnext), ctypes.c_int(vnext.stride(0)), ptr(self.adv_buf), ptr(self.ret_buf),
                                  ctypes.c_int(cfg.rollout_len), ctypes.c_int(cfg.n_envs), ctypes.c_float(cfg.gamma),
                                  ctypes.c_float(cfg.gae_lambda), stream_ptr()), "ppo_gae")
        self.obs_buf[0].copy_(self.obs_buf[T])

    def _opt_step(self, opt):
        if self.grad_sync is not None:
            self.grad_sync.reduce_and_step(opt)
            return
        if opt.max_grad_norm > 0:
            opt.clip()
        opt.step(zero_grad=True)

    def _minibatch(self):
        cfg, env, lib = self.cfg, self.env, self.lib
        head = self.actor.mods[2]
        if self._train_pass is not None:
            return self._minibatch_fused()
        check(lib.nb_ppo_gather(ptr(self.obs_buf), ctypes.c_int(env.obs_pad * 2), ptr(self.act_buf), ctypes.c_int(self.AP),
                                ptr(self.logp_buf), ptr(self.adv_buf), ptr(self.ret_buf), ptr(self.mb_obs),
                                ptr(self.mb_act), ptr(self.mb_logp), ptr(self.mb_adv), ptr(self.mb_ret),
                                ptr(self.partials), ptr(self.adv_stats), ctypes.c_int(self.pool), ctypes.c_int(self.mb),
                                ctypes.c_int(cfg.n_minibatches), ctypes.c_ulonglong(cfg.seed * 104729 + 7),
                                ptr(self.counters), stream_ptr()), "ppo_gather")
        # ---- critic forward / backward on a side stream, overlapping the actor chain
        br = self._critic_branch
        with br:
            v = self._forward(self.critic, self.mb_obs, save=True)
            check(lib.nb_ppo_value_loss(ptr(v), ctypes.c_int(v.stride(0)), ptr(self.mb_ret), ptr(self.dv), ctypes.c_int(8),
                                        ptr(self.partials_v), ptr(self.metrics[5:]), ctypes.c_int(self.mb),
                                        ctypes.c_float(1.0 / self.mb), stream_ptr()), "ppo_value_loss")
            self.critic.vjp(self.dv[:, :1])
            self._critic_pg.join()
        # ---- actor
        mu = self._forward(self.actor, self.mb_obs, save=True)
        check(lib.nb_ppo_objective(ptr(mu), ctypes.c_int(mu.stride(0)), ptr(head.log_std.storage), ptr(self.mb_act),
                                   ctypes.c_int(self.AP), ptr(self.mb_logp), ptr(self.mb_adv), ptr(self.adv_stats),
                                   ptr(self.dmu), ctypes.c_int(self.AP), ptr(self.partials), ptr(self.partials2),
                                   ptr(head.log_std.grad_storage), ptr(self.metrics), ctypes.c_int(self.mb),
                                   ctypes.c_int(env.act_dim), ctypes.c_float(cfg.clip_eps),
                                   ctypes.c_float(cfg.entropy_coef), ctypes.c_float(1.0 / self.mb), stream_ptr()),
              "ppo_objective")
        self.actor.vjp(self.dmu[:, : env.act_dim])
        self._actor_pg.join()
        # the optimizer steps stay on the main stream; with a gradient sync both arenas are reduced and updated by one
        # cross-GPU kernel (every rank runs its cross-GPU kernels in the same order)
        br.join()
        if self.grad_sync is not None and hasattr(self.grad_sync, "reduce_and_step_many"):
            self.grad_sync.reduce_and_step_many([self.actor_opt, self.critic_opt])
        else:
            self._opt_step(self.actor_opt)
            self._opt_step(self.critic_opt)
        check(lib.nb_ppo_counter(ptr(self.counters), ctypes.c_int(0), ctypes.c_int(0), stream_ptr()), "counter")

    def _gather(self):
        cfg, env = self.cfg, self.env
        check(self.lib.nb_ppo_gather(ptr(self.obs_buf), ctypes.c_int(env.obs_pad * 2), ptr(self.act_buf), ctypes.c_int(self.AP),
                                     ptr(self.logp_buf), ptr(self.adv_buf), ptr(self.ret_buf), ptr(self.mb_obs),
                                     ptr(self.mb_act), ptr(self.mb_logp), ptr(self.mb_adv), ptr(self.mb_ret),
                                     ptr(self.partials), ptr(self.adv_stats), ctypes.c_int(self.pool), ctypes.c_int(self.mb),
                                     ctypes.c_int(cfg.n_minibatches), ctypes.c_ulonglong(cfg.seed * 104729 + 7),
                                     ptr(self.counters), stream_ptr()), "ppo_gather")

    def _minibatch_fused(self):
        """One minibatch update with the fused kernels: gather → grouped forward (actor + critic, one launch) → the two
        loss kernels → grouped data-gradient chain (one launch) → six parameter-gradient chains on side streams →
        optimizer (with a gradient sync: one cross-GPU kernel for both arenas)."""
        from ..ops.mlp import mlp3_backward_group, mlp3_forward_group, mlp3_param_grads
        cfg, env, lib = self.cfg, self.env, self.lib
        head = self.actor.mods[2]
        pa, pc = self._train_pass
        self._gather()
        x = self.mb_obs
        mu, v = mlp3_forward_group([pa, pc], [x, x])
        # the two loss chains are independent (value loss + its reduction, objective + its finalisation): the value side
        # runs on a branch next to the objective instead of in front of it
        with self._critic_branch:
            check(lib.nb_ppo_value_loss(ptr(v), ctypes.c_int(v.stride(0)), ptr(self.mb_ret), ptr(self.dv), ctypes.c_int(8),
                                        ptr(self.partials_v), ptr(self.metrics[5:]), ctypes.c_int(self.mb),
                                        ctypes.c_float(1.0 / self.mb), stream_ptr()), "ppo_value_loss")
        check(lib.nb_ppo_objective(ptr(mu), ctypes.c_int(mu.stride(0)), ptr(head.log_std.storage), ptr(self.mb_act),
                                   ctypes.c_int(self.AP), ptr(self.mb_logp), ptr(self.mb_adv), ptr(self.adv_stats),
                                   ptr(self.dmu), ctypes.c_int(self.AP), ptr(self.partials), ptr(self.partials2),
                                   ptr(head.log_std.grad_storage), ptr(self.metrics), ctypes.c_int(self.mb),
                                   ctypes.c_int(env.act_dim), ctypes.c_float(cfg.clip_eps),
                                   ctypes.c_float(cfg.entropy_coef), ctypes.c_float(1.0 / self.mb), stream_ptr()),
              "ppo_objective")
        self._critic_branch.join()
        mlp3_backward_group([pa, pc], [x, x], [self.dmu, self.dv])
        mlp3_param_grads(pa, x, self.dmu, self._layer_pg[0])
        mlp3_param_grads(pc, x, self.dv, self._layer_pg[1])
        for brs in self._layer_pg:
            for b in brs:
                b.join()
        if self.grad_sync is not None and hasattr(self.grad_sync, "reduce_and_step_many"):
            self.grad_sync.reduce_and_step_many([self.actor_opt, self.critic_opt])
        elif self.grad_sync is None:
            from ..nn.optim import step_many
            step_many([self.actor_opt, self.critic_opt], zero_grad=True)
        else:
            self._opt_step(self.actor_opt)
            self._opt_step(self.critic_opt)
        check(lib.nb_ppo_counter(ptr(self.counters), ctypes.c_int(0), ctypes.c_int(0), stream_ptr()), "counter")

    def _update(self):
        cfg = self.cfg
        check(self.lib.nb_ppo_counter(ptr(self.counters), ctypes.c_int(0), ctypes.c_int(1), stream_ptr()), "counter")
        for _ in range(cfg.n_epochs * cfg.n_minibatches):
            self._run("minibatch", self._minibatch)
        check(self.lib.nb_ppo_counter(ptr(self.counters), ctypes.c_int(1), ctypes.c_int(0), stream_ptr()), "counter")

    # ------------------------------------------------------------------ graphs
    def _run(self, key, fn):
        if not self.cfg.use_cuda_graphs:
            fn()
            return
        g = self._graphs.get(key)
        if g is None:
            # eager warm-up on a side stream (lazy allocations, kernel attribute set-up), then capture
            s = self._cap_stream          # warm-up and capture on ONE stream: workspaces are reused at stable addresses
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                fn()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = _native.launch_count()
            with torch.cuda.graph(g, stream=s):
                fn()
            self._graph_launches[key] = _native.launch_count() - n0
            _native.add_launches(-self._graph_launches[key])  # the capture pass launches nothing
            self._graphs[key] = g
            return  # the warm-up already did this call's work
        g.replay()
        _native.add_launches(self._graph_launches[key])

    # ------------------------------------------------------------------ public
    def collect(self):
        self._run("rollout", self._rollout)
        self._run("gae", self._gae)

    def update(self):
        self._update()

    def train_iteration(self, read_metrics: bool = True):
        from ..utils.trace import nvtx_range
        self.metrics.zero_()
        self.env.ep_stats.zero_()
        with nvtx_range("ppo.collect"):
            self.collect()
        with nvtx_range("ppo.update"):
            self.update()
        self.iteration += 1
        return self.read_metrics() if read_metrics else None

    def read_metrics(self):
        m = self.metrics.cpu().tolist()
        e = self.env.ep_stats.cpu().tolist()
        n = max(m[4], 1.0)
        nup = self.cfg.n_epochs * self.cfg.n_minibatches
        return {"policy_loss": m[0] / n, "approx_kl": m[1] / n, "clip_frac": m[2] / n, "entropy": m[3] / n,
                "value_loss": m[5] / max(nup * self.mb, 1), "mean_step_reward": e[2] / self.pool,
                "episodes": e[1], "mean_episode_return": e[0] / e[1] if e[1] > 0 else float("nan")}

    @property
    def env_steps_per_iteration(self) -> int:
        return self.pool

    # ------------------------------------------------------------------ persistence
    def named_params(self):
        yield from self.actor.named_params("actor.")
        yield from self.critic.named_params("critic.")

    def save(self, path: str):
        from ..io.checkpoint import save_checkpoint
        save_checkpoint(path, list(self.named_params()), [], {
            "iteration": float(self.iteration),
            **{f"actor_opt.{k}": v for k, v in self.actor_opt.scalars().items()},
            **{f"critic_opt.{k}": v for k, v in self.critic_opt.scalars().items()}}, with_moments=True)

    def load(self, path: str):
        from ..io.checkpoint import load_checkpoint
        sc = load_checkpoint(path, list(self.named_params()), [])
        self.iteration = int(sc.get("iteration", 0))
        self.actor_opt.load_scalars({k.split(".", 1)[1]: v for k, v in sc.items() if k.startswith("actor_opt.")})
        self.critic_opt.load_scalars({k.split(".", 1)[1]: v for k, v in sc.items() if k.startswith("critic_opt.")})
        for o in (self.actor_opt, self.critic_opt):
            if o.arena.shadow is not None:
                o.arena.refresh_shadow()


class PPOAgent:
    """Facade: ``PPOAgent(env, cfg).train(total_env_steps)`` (noeira/deep_agents/ppo/agent.mojo:41)."""

    def __init__(self, env, cfg: PPOConfig = None, logger=None, grad_sync=None):
        self.trainer = PPOTrainer(env, cfg, grad_sync=grad_sync)
        self.logger = logger

    def train(self, total_env_steps: int, log_every: int = 1, checkpoint_path: str = None, checkpoint_every: int = 0):
        """Runs the generic on-policy driver (``training.rl.run_onpolicy_train_batched``) over the device rollout;
        ``log_every`` / ``checkpoint_every`` count iterations.  Returns the last metrics read."""
        from ..training.rl import run_onpolicy_train_batched
        tr = self.trainer
        per = tr.env_steps_per_iteration
        last = {}

        def keep(step, m):
            last.clear()
            last.update(m)
        run_onpolicy_train_batched(tr, tr.env, total_env_steps, print_every=per * max(log_every, 1), logger=self.logger,
                                   checkpoint_every=per * checkpoint_every, checkpoint_path=checkpoint_path or "",
                                   on_iteration=keep, read_metrics_every=max(log_every, 1))
        return last

    def select_greedy_action(self, obs_bf16):
        return self.trainer.actor.forward(obs_bf16)
