"""Resident imitation dataset for action-chunking policies.

Episodes of (camera frames uint8, joint state, action) live on the training device; ``sample(batch)`` draws random
(episode, time) pairs on the device and returns the observation at that time with the NEXT ``chunk`` actions of the same
episode, zero-padded past the episode end together with the validity mask the loss and the CVAE encoder need
(``valid [B, chunk + 2]``: class token, joint token, then one flag per action).  Joint states and actions are normalised
with the dataset statistics (mean / std per dimension), images stay uint8 until the model's own normalisation.
Reference: ``ACTDataset`` + device draw / gather / normalise kernels (noeira/deep_agents/act/data_gpu.mojo:89-322),
episode layout of the LeRobot-style stores (noeira/data/store.mojo).
"""
from __future__ import annotations

from typing import List, Sequence

import torch


class ACTDataset:
    def __init__(self, episodes: Sequence[dict], chunk: int, device="cpu", seed: int = 0):
        """``episodes``: dicts with ``images [T, cams, 3, H, W] uint8``, ``qpos [T, J]``, ``action [T, A]``."""
        self.chunk, self.device = chunk, torch.device(device)
        lens = [int(e["qpos"].shape[0]) for e in episodes]
        self.lengths = torch.tensor(lens, device=self.device)
        self.offsets = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)[:-1]), device=self.device)
        self.images = torch.cat([torch.as_tensor(e["images"], dtype=torch.uint8) for e in episodes]).to(self.device)
        self.qpos = torch.cat([torch.as_tensor(e["qpos"], dtype=torch.float32) for e in episodes]).to(self.device)
        self.action = torch.cat([torch.as_tensor(e["action"], dtype=torch.float32) for e in episodes]).to(self.device)
        self.n_steps = int(self.qpos.shape[0])
        self.episode_of = torch.repeat_interleave(torch.arange(len(lens), device=self.device), self.lengths)
        self.q_mean, self.q_std = self.qpos.mean(0), self.qpos.std(0).clamp_min(1e-2)
        self.a_mean, self.a_std = self.action.mean(0), self.action.std(0).clamp_min(1e-2)
        self.gen = torch.Generator(device=self.device).manual_seed(seed)
        self._ar = torch.arange(chunk, device=self.device)

    def stats(self) -> dict:
        return dict(qpos_mean=self.q_mean, qpos_std=self.q_std, action_mean=self.a_mean, action_std=self.a_std)

    def sample(self, batch: int):
        """→ qpos [B, J] (normalised), images [B, cams, 3, H, W] uint8, actions [B, chunk, A] (normalised, zero padded),
        valid [B, chunk + 2] float (1 = real)."""
        t = torch.randint(0, self.n_steps, (batch,), device=self.device, generator=self.gen)
        ep = self.episode_of[t]
        end = self.offsets[ep] + self.lengths[ep]                     # one past the episode's last step
        idx = t[:, None] + self._ar[None]                             # [B, chunk] global step indices
        ok = idx < end[:, None]
        idx = torch.minimum(idx, (end - 1)[:, None])
        act = (self.action[idx] - self.a_mean) / self.a_std * ok[..., None]
        valid = torch.cat([torch.ones(batch, 2, device=self.device), ok.float()], 1)
        return (self.qpos[t] - self.q_mean) / self.q_std, self.images[t], act, valid

    def denormalise_action(self, a):
        return a * self.a_std + self.a_mean


def synthetic_episodes(n: int, length: int, cams: int, height: int, width: int, joints: int = 6, seed: int = 0) -> List[dict]:
    """Seed-generated stand-in episodes of the shapes the ACT configuration names."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for e in range(n):
        T = length - (e % 3) * (length // 5)
        q = torch.cumsum(torch.randn(T, joints, generator=g) * 0.05, 0)
        out.append(dict(images=torch.randint(0, 256, (T, cams, 3, height, width), dtype=torch.uint8, generator=g),
                        qpos=q, action=q + torch.randn(T, joints, generator=g) * 0.01))
    return out


def load_aloha_episode(path: str, cameras: Sequence[str] = None) -> dict:
    """One ALOHA / ACT episode file (HDF5: ``/action [T, A]``, ``/observations/qpos [T, J]``,
    ``/observations/images/<camera> [T, H, W, 3] uint8``) as the dict ``ACTDataset`` takes (images channel-first, cameras in
    the given or the file's sorted order)."""
    from ..io.hdf5 import H5File
    with H5File(path) as f:
        cams = list(cameras) if cameras is not None else f["observations/images"].keys()
        frames = [torch.from_numpy(f[f"observations/images/{c}"].read()).permute(0, 3, 1, 2) for c in cams]
        return dict(images=torch.stack(frames, 1).contiguous(), qpos=torch.from_numpy(f["observations/qpos"].read()).float(),
                    action=torch.from_numpy(f["action"].read()).float(), cameras=cams, attrs=dict(f.attrs))


def save_aloha_episode(path: str, episode: dict, cameras: Sequence[str], compression: str = "gzip"):
    """The inverse of ``load_aloha_episode`` (episodes recorded here can be read by the usual ACT tooling)."""
    from ..io.hdf5 import write_hdf5
    img = torch.as_tensor(episode["images"])
    tree = {"action": torch.as_tensor(episode["action"]).float().numpy(),
            "observations": {"qpos": torch.as_tensor(episode["qpos"]).float().numpy(),
                             "images": {c: img[:, i].permute(0, 2, 3, 1).contiguous().numpy() for i, c in enumerate(cameras)}}}
    write_hdf5(path, tree, compression=compression, chunk_rows=max(1, min(64, img.shape[0] // 4 or 1)), attrs={"": {"sim": False}})
