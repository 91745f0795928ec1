"""ACT deployment side: temporal ensembling, the normalisation file a deployed policy reads, camera preprocessing.

  TemporalEnsemble   ring of the last K predicted chunks; the action for step t is the weighted mean of every chunk that
                     covers t, weight exp(-m·(i − i_min)) for the chunk queried at step i (i_min = start of the window), so
                     the OLDEST covering query weighs most (noeira/deep_agents/act/inference.mojo:52-155).  The ensemble
                     runs in normalised units; the caller denormalises the one combined action.
  ACTNorm            ``norm.json``: qpos / action mean, std, min, max, camera slot order, image size, provenance — the few
                     numbers a deployment needs from the training store (noeira/deep_agents/act/norm_file.mojo:42-156).
                     float32 statistics are written as float64 decimals and round-trip bit-exactly.
  normalize_camera_chw / denormalize   the same arithmetic the training data path uses.
  ACTPolicy          query → chunk → ensemble → denormalised action, around an ``ACTModel``.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch

ACT_TEMPORAL_ENSEMBLE_M = 0.01
IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)
NORM_SCHEMA_VERSION = 1


class TemporalEnsemble:
    def __init__(self, adim: int, k: int, m: float = ACT_TEMPORAL_ENSEMBLE_M):
        if adim <= 0 or k <= 0:
            raise ValueError("TemporalEnsemble: K and ADIM must be > 0")
        self.adim, self.k, self.m = adim, k, m
        self.chunks = np.zeros((k, k, adim), dtype=np.float32)      # slot i % K holds the chunk queried at step i
        self.query_step = [-1] * k

    def reset(self):
        self.query_step = [-1] * self.k

    def push(self, t: int, chunk):
        """Record the ``[K, ADIM]`` chunk (normalised units) predicted AT step ``t``."""
        c = np.asarray(chunk.detach().float().cpu() if torch.is_tensor(chunk) else chunk, dtype=np.float32).reshape(self.k, self.adim)
        slot = t % self.k
        self.query_step[slot] = t
        self.chunks[slot] = c

    def _window(self, t: int):
        i_min = max(t - self.k + 1, 0)
        return i_min, [i for i in range(i_min, t + 1) if self.query_step[i % self.k] == i]

    def n_contributors(self, t: int) -> int:
        return len(self._window(t)[1])

    def action_at(self, t: int) -> np.ndarray:
        i_min, qs = self._window(t)
        if not qs:
            raise RuntimeError(f"TemporalEnsemble.action_at: no chunk covers step {t} - push() the query for this step first")
        w = np.array([math.exp(-self.m * (i - i_min)) for i in qs], dtype=np.float64)
        w /= w.sum()
        out = np.zeros(self.adim, dtype=np.float32)
        for wi, i in zip(w, qs):
            out += np.float32(wi) * self.chunks[i % self.k, t - i]
        return out


def denormalize(a, mean, std):
    """``a·std + mean``: back to the units the robot speaks (applied once, to the ensembled action)."""
    return np.asarray(a, dtype=np.float32) * np.asarray(std, dtype=np.float32) + np.asarray(mean, dtype=np.float32)


def normalize_camera_chw(img_u8: torch.Tensor) -> torch.Tensor:
    """uint8 ``[..., 3, H, W]`` → ``/255`` → ImageNet mean / std, fp32; the ONE preprocessing shared by training and
    deployment (noeira/deep_agents/act/inference.mojo:188)."""
    x = img_u8.float() / 255.0
    mean = torch.tensor(IMAGENET_MEAN, device=x.device).view(3, 1, 1)
    std = torch.tensor(IMAGENET_STD, device=x.device).view(3, 1, 1)
    return (x - mean) / std


@dataclass
class ACTNorm:
    qpos_mean: List[float] = field(default_factory=list)
    qpos_std: List[float] = field(default_factory=list)
    action_mean: List[float] = field(default_factory=list)
    action_std: List[float] = field(default_factory=list)
    qpos_min: List[float] = field(default_factory=list)
    qpos_max: List[float] = field(default_factory=list)
    action_min: List[float] = field(default_factory=list)
    action_max: List[float] = field(default_factory=list)
    cameras: List[str] = field(default_factory=list)      # slot order
    img_h: int = 0
    img_w: int = 0
    n_rows: int = 0
    n_episodes: int = 0
    store: str = ""

    @staticmethod
    def from_data(qpos: np.ndarray, action: np.ndarray, cameras=(), img_h=0, img_w=0, n_episodes=0, store="", std_floor=1e-2):
        """Statistics over the rows of the store (std clipped from below as the original ACT does)."""
        q, a = np.asarray(qpos, np.float32), np.asarray(action, np.float32).reshape(-1, np.asarray(action).shape[-1])
        f = lambda v: [float(x) for x in v]
        return ACTNorm(f(q.mean(0)), f(np.maximum(q.std(0), std_floor)), f(a.mean(0)), f(np.maximum(a.std(0), std_floor)),
                       f(q.min(0)), f(q.max(0)), f(a.min(0)), f(a.max(0)), list(cameras), img_h, img_w, int(q.shape[0]),
                       n_episodes, store)

    def save(self, path: str):
        d = {"schema_version": NORM_SCHEMA_VERSION}
        d.update({k: getattr(self, k) for k in self.__dataclass_fields__})
        # float32 statistics as float64 decimals (repr round-trips exactly)
        for k in ("qpos_mean", "qpos_std", "action_mean", "action_std"):
            d[k] = [float(np.float32(v)) for v in d[k]]
        tmp = path + ".tmp"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(tmp, "w") as f:
            json.dump(d, f, indent=1)
        os.replace(tmp, path)

    @staticmethod
    def load(path: str) -> "ACTNorm":
        d = json.load(open(path))
        if d.get("schema_version", 1) != NORM_SCHEMA_VERSION:
            raise ValueError(f"{path}: norm schema {d.get('schema_version')} is not {NORM_SCHEMA_VERSION}")
        return ACTNorm(**{k: d[k] for k in ACTNorm.__dataclass_fields__ if k in d})

    def normalize_qpos(self, q):
        return (np.asarray(q, np.float32) - np.asarray(self.qpos_mean, np.float32)) / np.asarray(self.qpos_std, np.float32)

    def action_box(self, margin: float = 0.05):
        lo, hi = np.asarray(self.action_min), np.asarray(self.action_max)
        pad = margin * (hi - lo)
        return lo - pad, hi + pad


class ACTPolicy:
    """Closed-loop inference: every ``query_every`` steps the model predicts a chunk (latent = prior mean, i.e. the CVAE
    branch multiplied by zero), chunks are ensembled, the combined action is denormalised and clamped to the action box."""

    def __init__(self, model, norm: ACTNorm, query_every: int = 1, m: float = ACT_TEMPORAL_ENSEMBLE_M):
        self.model, self.norm, self.query_every = model, norm, query_every
        cfg = model.cfg
        self.ens = TemporalEnsemble(cfg.action_dim if hasattr(cfg, "action_dim") else len(norm.action_mean), cfg.chunk, m)
        self.t = 0

    def reset(self):
        self.ens.reset()
        self.t = 0

    def act(self, qpos, images_u8: torch.Tensor) -> np.ndarray:
        """``qpos [QPOS]`` raw joint state, ``images_u8 [N_CAM, 3, H, W]`` uint8.  Returns one raw-unit action."""
        if self.t % self.query_every == 0:
            dev = next(iter(self.model.params())).storage.device
            q = torch.tensor(self.norm.normalize_qpos(qpos), device=dev)[None]
            with torch.no_grad():
                chunk = self.model.infer(q, images_u8[None].to(dev))
            self.ens.push(self.t, chunk[0])
        a = denormalize(self.ens.action_at(self.t), self.norm.action_mean, self.norm.action_std)
        lo, hi = self.norm.action_box()
        self.t += 1
        return np.clip(a, lo, hi)
