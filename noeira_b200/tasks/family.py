"""A task family as a batched environment, and the family drivers.

``TabletopFamilyEnv`` is the kinematic counterpart of the reference's composed tabletop scenes: a velocity-controlled
gripper, the family's slots as objects that can be grasped, carried and released (released objects settle on the
surface below them: a region's site, another object's top, or the floor), several tasks of ONE family mixed across the
lanes of the batch, goal predicates and shaping evaluated on the device (tasks/predicates.py), resets drawn from
precomputed placement tables (tasks/sampler.py).  It is a tensor program without host-side control flow, so a rollout
over it can be captured in a CUDA graph, and it runs unchanged on the CPU for tests.

Drivers: ``sac_family_driver`` / ``ppo_family_driver`` train one task-conditioned policy over all tasks of a family
through the generic off-policy / on-policy loops (training/rl.py) and report per-task success rates.
Reference: noeira/tasks/family.mojo, noeira/tasks/ppo_family_driver.mojo, noeira/tasks/sac_family_driver.mojo,
noeira/tasks/lanes.mojo (task-per-lane assignment).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..envs.batched_env import BatchedEnv
from .predicates import BoundGoal, GoalState, bind_goal, evaluate, evaluate_cuda, family_tables, parse_goal, require_evaluable
from .sampler import DEFAULT_RADIUS, InitTable
from .spec import SLOT_FREE, TABLE_Z_OFFSET, FamilySpec, TaskSpec, validate_task_against_family

GRIPPER = "gripper"     # pseudo slot appended after the family's slots so that goals can name the end effector


class TabletopFamilyEnv(BatchedEnv):
    def __init__(self, family: FamilySpec, tasks: Sequence[TaskSpec], n_envs: int, sites: Optional[Dict[str, Sequence[float]]] = None,
                 device="cpu", seed: int = 0, table_k: int = 2048, move_step: float = 0.02, grasp_radius: float = 0.035,
                 workspace=((-0.4, -0.4, 0.0), (0.4, 0.4, 0.5)), shaping_scale: float = 10.0, success_bonus: float = 5.0,
                 step_cost: float = 0.01):
        import copy
        self.family = fam = copy.deepcopy(family)
        from .spec import SlotSpec
        fam.slots.append(SlotSpec(GRIPPER, SLOT_FREE, "builtin:gripper"))
        self.tasks = list(tasks)
        self.n_envs, self.device = int(n_envs), torch.device(device)
        S = self.S = len(fam.slots)
        T = self.T = len(self.tasks)
        self.act_dim = 4
        self.obs_dim = 5 + 3 * (S - 1) + T
        self.move_step, self.grasp_radius = move_step, grasp_radius
        self.shaping_scale, self.success_bonus, self.step_cost = shaping_scale, success_bonus, step_cost
        dev = self.device
        self.ws_lo = torch.tensor(workspace[0], device=dev)
        self.ws_hi = torch.tensor(workspace[1], device=dev)
        self.rect, self.geom = family_tables(fam, dev)
        self.radius = torch.tensor([s.h_radius if s.has_geom else DEFAULT_RADIUS for s in fam.slots], device=dev)
        self.free = torch.tensor([s.kind == SLOT_FREE and s.name != GRIPPER for s in fam.slots], device=dev)
        # a region's site: the origin of the slot of that name (it then moves with the slot), else a fixed world point
        sites = sites or {}
        self.site_slot = torch.tensor([fam.slot_index(r.site) if fam.has_slot(r.site) else -1 for r in fam.regions] or [-1],
                                      device=dev)
        self.site_fixed = torch.tensor([list(sites.get(r.site, (0.0, 0.0, 0.0))) for r in fam.regions] or [[0.0, 0.0, 0.0]],
                                       device=dev)
        for r in fam.regions:
            if not fam.has_slot(r.site) and r.site not in sites:
                raise KeyError(f"tasks: region {r.name}: site {r.site!r} is neither a slot nor one of the given world sites")
        # per task: bound goal, active mask, placement table
        self.bound: List[BoundGoal] = []
        self.tables: List[InitTable] = []
        self.active = torch.zeros(T, S, dtype=torch.bool, device=dev)
        self.horizon = torch.empty(T, device=dev)
        for ti, t in enumerate(self.tasks):
            validate_task_against_family(t, family)
            bg = bind_goal(parse_goal(t.goal), fam)
            require_evaluable(bg)
            self.bound.append(bg)
            static_sites = {r.name: self._site_world_static(r) for r in fam.regions}
            self.tables.append(InitTable(t, family, static_sites, k=table_k, seed=seed + 17 * ti, device=dev))
            for a in t.active:
                self.active[ti, fam.slot_index(a)] = True
            self.horizon[ti] = float(t.horizon or family.horizon)
        self.tapes = [bg.tensors(dev) for bg in self.bound]
        self.pos = torch.zeros(self.n_envs, S, 3, device=dev)
        self.quat = torch.zeros(self.n_envs, S, 4, device=dev)
        self.quat[..., 0] = 1.0
        self.closed = torch.zeros(self.n_envs, device=dev)
        self.holding = torch.full((self.n_envs,), -1, dtype=torch.long, device=dev)
        self.lane_task = (torch.arange(self.n_envs, device=dev) % T)            # lanes are dealt round-robin to tasks
        self.task_onehot = torch.nn.functional.one_hot(self.lane_task, T).float()
        self.t = torch.zeros(self.n_envs, device=dev)
        self.episode = torch.zeros(self.n_envs, dtype=torch.long, device=dev)
        self.prev_dist = torch.zeros(self.n_envs, device=dev)
        self.succeeded = torch.zeros(self.n_envs, dtype=torch.bool, device=dev)
        self.ep_return = torch.zeros(self.n_envs, device=dev)
        self.success_count = torch.zeros(T, device=dev)
        self.episode_count = torch.zeros(T, device=dev)
        self.seed = seed
        self._alloc_io(dev)

    # ------------------------------------------------------------------ geometry helpers
    def _site_world_static(self, r):
        fam = self.family
        if fam.has_slot(r.site):
            s = fam.slots[fam.slot_index(r.site)]
            base = s.pose if s.pose is not None else [0.0, 0.0, 0.0]
            return torch.tensor([base[0], base[1], base[2] + (s.top_z if s.has_geom else 0.0)], device=self.device)
        return self.site_fixed[fam.region_index(r.name)].clone()

    def _sites(self):
        """[N, R, 3] region site positions now (a site on a slot sits at that slot's top)."""
        idx = self.site_slot.clamp(min=0)
        on_slot = self.pos[:, idx] + torch.stack([torch.zeros_like(self.geom[idx, 1]), torch.zeros_like(self.geom[idx, 1]),
                                                 self.geom[idx, 1]], dim=-1)
        return torch.where((self.site_slot >= 0)[None, :, None], on_slot, self.site_fixed[None].expand(self.n_envs, -1, -1))

    def _goal_state(self):
        return GoalState(self.pos, self.quat, self._sites(), self.rect, self.geom, None)

    def _goal(self):
        """(success [N] bool, distance [N]) of every lane's own task."""
        st = self._goal_state()
        ok = torch.zeros(self.n_envs, dtype=torch.bool, device=self.device)
        dist = torch.zeros(self.n_envs, device=self.device)
        for ti, bg in enumerate(self.bound):
            o, d = (evaluate_cuda(bg, st, self.tapes[ti]) if self.device.type == "cuda" else evaluate(bg, st))
            sel = self.lane_task == ti
            ok = torch.where(sel, o, ok)
            dist = torch.where(sel, d, dist)
        return ok, dist

    # ------------------------------------------------------------------ reset / observe
    def _reset_where(self, mask):
        for ti, tab in enumerate(self.tables):
            # counter-hash draw: no generator state, so the reset can sit inside a captured graph
            lane = torch.arange(self.n_envs, device=self.device)
            h = (lane * 2654435761 + self.episode * 40503 + self.seed * 97 + ti * 7919) & 0x7FFFFFFF
            idx = ((h >> 7) ^ h) % len(tab)
            sel = mask & (self.lane_task == ti)
            S0 = self.S - 1
            self.pos[:, :S0] = torch.where(sel[:, None, None], tab.pos[idx], self.pos[:, :S0])
            self.quat[:, :S0] = torch.where(sel[:, None, None], tab.quat[idx], self.quat[:, :S0])
        home = torch.tensor([0.0, 0.0, 0.25], device=self.device)
        self.pos[:, -1] = torch.where(mask[:, None], home, self.pos[:, -1])
        self.closed = torch.where(mask, torch.zeros_like(self.closed), self.closed)
        self.holding = torch.where(mask, torch.full_like(self.holding, -1), self.holding)
        self.t = torch.where(mask, torch.zeros_like(self.t), self.t)
        self.episode = self.episode + mask.long()
        _, d = self._goal()
        self.prev_dist = torch.where(mask, d, self.prev_dist)
        self.succeeded = self.succeeded & ~mask
        self.ep_return = torch.where(mask, torch.zeros_like(self.ep_return), self.ep_return)

    def _observe(self, out, out_bf16):
        g = self.pos[:, -1]
        rel = (self.pos[:, :-1] - g[:, None]).reshape(self.n_envs, -1)
        act = self.active[self.lane_task][:, :-1].float().repeat_interleave(3, dim=1)
        o = torch.cat([g, self.closed[:, None], (self.holding >= 0).float()[:, None], rel * act, self.task_onehot], dim=1)
        out.copy_(o)
        out_bf16[:, : self.obs_dim].copy_(o)

    def reset_batch(self):
        self._reset_where(torch.ones(self.n_envs, dtype=torch.bool, device=self.device))
        self._observe(self.obs, self.obs_bf16)
        return self.obs

    # ------------------------------------------------------------------ step
    def step_batch(self, action, auto_reset: bool = True):
        N, S = self.n_envs, self.S
        a = action[:, :4].float().clamp(-1.0, 1.0)
        g = torch.minimum(torch.maximum(self.pos[:, -1] + self.move_step * a[:, :3], self.ws_lo), self.ws_hi)
        close = a[:, 3] > 0
        lane_active = self.active[self.lane_task] & self.free[None]                        # [N, S] graspable now
        # grasp: nearest graspable object inside the grasp radius, when the hand closes empty
        d = torch.linalg.vector_norm(self.pos - g[:, None], dim=-1)
        d = torch.where(lane_active, d, torch.full_like(d, 1e9))
        near_d, near_i = d.min(dim=1)
        take = close & (self.holding < 0) & (near_d < self.grasp_radius)
        holding = torch.where(take, near_i, self.holding)
        # release: the object settles on what is below it
        drop = (~close) & (holding >= 0)
        hi = holding.clamp(min=0)
        ar = torch.arange(N, device=self.device)
        obj = self.pos[ar, hi]
        sites = self._sites()
        dxy = obj[:, None, :2] - sites[:, :, :2]
        inside = (dxy[..., 0] >= self.rect[:, 0]) & (dxy[..., 0] <= self.rect[:, 2]) & (dxy[..., 1] >= self.rect[:, 1]) & \
                 (dxy[..., 1] <= self.rect[:, 3]) & (sites[..., 2] <= obj[:, None, 2] + 1e-4)
        own_site = self.site_slot[None, :] == hi[:, None]                                  # never rest on a region of itself
        sup_r = torch.where(inside & ~own_site, sites[..., 2] + TABLE_Z_OFFSET, torch.zeros_like(sites[..., 2])).amax(dim=1)
        oxy = torch.linalg.vector_norm(self.pos[:, :, :2] - obj[:, None, :2], dim=-1)
        others = lane_active | (self.active[self.lane_task] & ~self.free[None])
        others = others & (torch.arange(S, device=self.device)[None] != hi[:, None]) & (oxy < 0.03) & \
                 (self.pos[:, :, 2] <= obj[:, None, 2] + 1e-4)
        sup_o = torch.where(others, self.pos[:, :, 2] + self.geom[None, :, 1] + 0.01, torch.zeros_like(oxy)).amax(dim=1)
        bottom = self.geom[hi, 0]
        rest_z = torch.maximum(sup_r, sup_o) - torch.where(bottom != 0, bottom, -self.radius[hi])
        # carried object follows the hand; a released one settles
        carried = torch.where(drop[:, None], torch.cat([obj[:, :2], rest_z[:, None]], dim=1), g)
        moved = (holding >= 0)
        newpos = self.pos.clone()
        newpos[:, -1] = g
        upd = torch.where(moved[:, None], carried, newpos[ar, hi])
        newpos[ar, hi] = torch.where(moved[:, None], upd, newpos[ar, hi])
        newpos[:, -1] = g
        self.pos = newpos
        self.holding = torch.where(drop, torch.full_like(holding, -1), holding)
        self.closed = close.float()
        self.t = self.t + 1
        ok, dist = self._goal()
        first = ok & ~self.succeeded
        r = self.shaping_scale * (self.prev_dist - dist) - self.step_cost + self.success_bonus * first.float()
        self.prev_dist = dist
        self.succeeded = self.succeeded | ok
        timeout = self.t >= self.horizon[self.lane_task]
        done = ok | timeout
        self.ep_return = self.ep_return + r
        self.reward.copy_(r)
        self.terminated.copy_(ok.float())
        self.done.copy_(done.float())
        self.finished_return.copy_(torch.where(done, self.ep_return, torch.full_like(self.ep_return, float("nan"))))
        self.ep_stats[0] += torch.where(done, self.ep_return, torch.zeros_like(r)).sum()
        self.ep_stats[1] += done.float().sum()
        self.ep_stats[2] += r.sum()
        self.ep_stats[3] += torch.where(done, self.t, torch.zeros_like(self.t)).sum()
        self.success_count += torch.zeros_like(self.success_count).index_add_(0, self.lane_task, (done & ok).float())
        self.episode_count += torch.zeros_like(self.episode_count).index_add_(0, self.lane_task, done.float())
        self._observe(self.next_obs, self.next_obs_bf16)
        if auto_reset:
            self._reset_where(done)
        self._observe(self.obs, self.obs_bf16)
        return self.obs, self.reward, self.done, self.terminated

    def success_rates(self) -> Dict[str, float]:
        s, e = self.success_count.tolist(), self.episode_count.tolist()
        return {t.name: (s[i] / e[i] if e[i] > 0 else float("nan")) for i, t in enumerate(self.tasks)}

    def clear_statistics(self):
        self.success_count.zero_()
        self.episode_count.zero_()


def sac_family_driver(family: FamilySpec, tasks: Sequence[TaskSpec], *, n_envs: int = 64, total_env_steps: int = 20000,
                      sites=None, device="cpu", seed: int = 0, hidden: int = 128, **sac_kw):
    """One task-conditioned SAC policy over every task of the family.  Returns (trainer, env, log, success rates)."""
    from ..agents.sac import SACConfig, SACTrainer
    from ..training.rl import run_offpolicy_train_batched
    env = TabletopFamilyEnv(family, tasks, n_envs, sites=sites, device=device, seed=seed)
    from ..data.replay import StoreReplay
    batch = sac_kw.pop("batch", 128)
    learning_starts = sac_kw.pop("learning_starts", min(1000, total_env_steps // 4))
    cfg = SACConfig(obs_dim=env.obs_dim, act_dim=env.act_dim, hidden=hidden, batch=batch, seed=seed, **sac_kw)
    trainer = SACTrainer(cfg, device=device)
    replay = StoreReplay(max(total_env_steps, 4096), env.obs_dim, env.act_dim, device=device)
    log = run_offpolicy_train_batched(trainer, env, replay, total_env_steps, learning_starts=learning_starts, batch_size=batch)
    return trainer, env, log, env.success_rates()


def ppo_family_driver(family: FamilySpec, tasks: Sequence[TaskSpec], *, n_envs: int = 1024, iterations: int = 50, sites=None,
                      seed: int = 0, **ppo_kw):
    """One task-conditioned PPO policy over every task of the family with the device rollout (CUDA only: the rollout,
    GAE and the minibatch updates are captured graphs).  Returns (agent, env, per-iteration metrics, success rates)."""
    from ..agents.ppo import PPOConfig, PPOTrainer
    env = TabletopFamilyEnv(family, tasks, n_envs, sites=sites, device="cuda", seed=seed)
    env.engine = _EngineAdapter(env)
    agent = PPOTrainer(env, PPOConfig(n_envs=n_envs, **ppo_kw))
    hist = [agent.train_iteration() for _ in range(iterations)]
    return agent, env, hist, env.success_rates()


class _EngineAdapter:
    """The call shape the PPO rollout uses on a physics engine (``engine.step(action, reward, done, terminated, …)``)
    over a tensor-program environment."""

    def __init__(self, env: TabletopFamilyEnv):
        self.env = env

    def step(self, action, reward, done, terminated, obs_f32=None, obs_bf16=None, next_obs_f32=None, next_obs_bf16=None,
             finished_return=None, do_reset=True, ep_stats=None, dbg=None):
        e = self.env
        e.step_batch(action, auto_reset=do_reset)
        reward.copy_(e.reward); done.copy_(e.done); terminated.copy_(e.terminated)
        if obs_f32 is not None: obs_f32.copy_(e.obs)
        if obs_bf16 is not None: obs_bf16.copy_(e.obs_bf16)
        if next_obs_f32 is not None: next_obs_f32.copy_(e.next_obs)
        if next_obs_bf16 is not None: next_obs_bf16.copy_(e.next_obs_bf16)
        if finished_return is not None: finished_return.copy_(e.finished_return)
