"""Per-epoch input augmentation for the resident-dataset trainer.

An ``Augmenter`` rewrites the WHOLE augmentation buffer from the raw training set once per epoch (the trainer keeps the
raw data untouched and trains from the buffer); ``is_noop`` lets the trainer skip the buffer altogether.
``CropFlipAugmenter`` is the CIFAR recipe: zero-pad by ``pad``, take a random crop of the original size, flip it
horizontally with probability 1/2 — one draw per (sample, epoch) from a counter hash, so the result depends only on
(seed, epoch, sample index) and is identical on every device and under graph replay.  On CUDA it is one kernel
(``csrc/augment.cu``: thread per output element, NCHW or NHWC); the tensor program below runs anywhere and is the
oracle of the GPU test.
Reference: noeira/nn/training/augmenter.mojo:24-200 (Augmenter trait, IdentityAugmenter, CIFAR10CropFlipAugmenter{,NHWC}).
"""
from __future__ import annotations

import ctypes

import torch


class Augmenter:
    is_noop = False

    def augment(self, aug: torch.Tensor, raw: torch.Tensor, epoch: int, seed: int) -> None:
        """Fill ``aug`` (same shape as ``raw``) completely from ``raw``."""
        raise NotImplementedError


class IdentityAugmenter(Augmenter):
    is_noop = True

    def augment(self, aug, raw, epoch, seed):
        aug.copy_(raw)


def _hash_u32(x: torch.Tensor) -> torch.Tensor:
    """The mixing function of the kernel, on int64 tensors holding 32-bit values."""
    m = 0xFFFFFFFF
    x = x & m
    x = (x ^ (x >> 16)) * 0x7FEB352D & m
    x = (x ^ (x >> 15)) * 0x846CA68B & m
    return (x ^ (x >> 16)) & m


def crop_flip_draws(n: int, epoch: int, seed: int, pad: int, device):
    """(dx, dy in [0, 2·pad], flip in {0,1}) per sample, exactly as the kernel draws them."""
    i = torch.arange(n, device=device, dtype=torch.int64)
    h = _hash_u32(i * 0x9E3779B1 + (epoch & 0xFFFFFFFF) * 0x85EBCA77 + (seed & 0xFFFFFFFF) * 0xC2B2AE3D)
    span = 2 * pad + 1
    return (h % span), ((h >> 8) % span), ((h >> 20) & 1)


class CropFlipAugmenter(Augmenter):
    def __init__(self, pad: int = 4, layout: str = "nchw"):
        assert layout in ("nchw", "nhwc")
        self.pad, self.layout = pad, layout

    def augment(self, aug, raw, epoch, seed):
        assert aug.shape == raw.shape and raw.dim() == 4
        if raw.is_cuda and raw.dtype in (torch.float32, torch.bfloat16) and raw.is_contiguous() and aug.is_contiguous():
            from .._native import check, cuda_lib, ptr, stream_ptr
            N = raw.shape[0]
            C, H, W = (raw.shape[1], raw.shape[2], raw.shape[3]) if self.layout == "nchw" else (raw.shape[3], raw.shape[1], raw.shape[2])
            c = ctypes
            check(cuda_lib().nb_augment_crop_flip(ptr(raw), ptr(aug), c.c_int(N), c.c_int(C), c.c_int(H), c.c_int(W), c.c_int(self.pad),
                                                  c.c_int(1 if self.layout == "nhwc" else 0), c.c_int(1 if raw.dtype == torch.bfloat16 else 0),
                                                  c.c_uint(epoch & 0xFFFFFFFF), c.c_uint(seed & 0xFFFFFFFF), stream_ptr()), "augment_crop_flip")
            return
        aug.copy_(self.reference(raw, epoch, seed))

    def reference(self, raw, epoch, seed):
        x = raw if self.layout == "nchw" else raw.permute(0, 3, 1, 2)
        N, C, H, W = x.shape
        dx, dy, flip = crop_flip_draws(N, epoch, seed, self.pad, raw.device)
        xp = torch.nn.functional.pad(x, (self.pad,) * 4)
        ys = dy[:, None] + torch.arange(H, device=raw.device)[None]                       # [N, H]
        xs = torch.arange(W, device=raw.device)[None].expand(N, W)
        xs = torch.where(flip[:, None] > 0, W - 1 - xs, xs) + dx[:, None]                  # [N, W]
        out = xp[torch.arange(N, device=raw.device)[:, None, None, None], torch.arange(C, device=raw.device)[None, :, None, None],
                 ys[:, None, :, None], xs[:, None, None, :]]
        return out if self.layout == "nchw" else out.permute(0, 2, 3, 1)
