"""Image preprocessing shared by training and deployment: PIL-compatible bilinear resize on uint8 (separable triangle
filter with the support widened when shrinking, fixed-point accumulation as Pillow does), BGR camera frame → CHW RGB, and
aspect-preserving resize with padding.  Reference: noeira/vision/preprocess.mojo:50-260 (``pil_bilinear_u8``,
``camera_frame_to_chw_rgb``), noeira/vision/resize_pad.mojo."""
from __future__ import annotations

import numpy as np


def _coeffs(in_size: int, out_size: int):
    scale = in_size / out_size
    fscale = max(scale, 1.0)
    support = 1.0 * fscale
    ksize = int(np.ceil(support)) * 2 + 1
    bounds, ws = [], np.zeros((out_size, ksize), np.float64)
    for xx in range(out_size):
        center = (xx + 0.5) * scale
        xmin = max(int(center - support + 0.5), 0)
        xmax = min(int(center + support + 0.5), in_size)
        x = (np.arange(xmin, xmax) - center + 0.5) / fscale
        w = np.clip(1.0 - np.abs(x), 0.0, None)
        w /= w.sum()
        ws[xx, : xmax - xmin] = w
        bounds.append((xmin, xmax - xmin))
    return bounds, ws


def _resample_axis(img: np.ndarray, out_size: int, axis: int) -> np.ndarray:
    bounds, ws = _coeffs(img.shape[axis], out_size)
    PRECISION = 22                                        # Pillow's fixed-point weights for 8-bit images
    wi = np.round(ws * (1 << PRECISION)).astype(np.int64)
    src = np.moveaxis(img, axis, 0).astype(np.int64)
    out = np.empty((out_size,) + src.shape[1:], np.uint8)
    for i, (x0, n) in enumerate(bounds):
        acc = np.tensordot(wi[i, :n], src[x0:x0 + n], axes=(0, 0)) + (1 << (PRECISION - 1))
        out[i] = np.clip(acc >> PRECISION, 0, 255).astype(np.uint8)
    return np.moveaxis(out, 0, axis)


def pil_bilinear_u8(img: np.ndarray, out_h: int, out_w: int) -> np.ndarray:
    """``PIL.Image.resize((out_w, out_h), BILINEAR)`` on an ``[H, W, C]`` / ``[H, W]`` uint8 array, bit for bit
    (horizontal pass first, as Pillow does)."""
    x = img if img.shape[1] == out_w else _resample_axis(img, out_w, 1)
    return x if x.shape[0] == out_h else _resample_axis(x, out_h, 0)


def camera_frame_to_chw_rgb(frame_bgr: np.ndarray, out_h: int, out_w: int) -> np.ndarray:
    """BGR ``[H, W, 3]`` camera frame → resized RGB ``[3, out_h, out_w]`` uint8."""
    rgb = frame_bgr[:, :, ::-1]
    return np.ascontiguousarray(pil_bilinear_u8(rgb, out_h, out_w).transpose(2, 0, 1))


def resize_pad(img: np.ndarray, out_h: int, out_w: int, fill: int = 0) -> np.ndarray:
    """Aspect-preserving resize into ``out_h x out_w`` with the remainder padded (content anchored top-left, the
    convention of the VLA image path)."""
    h, w = img.shape[:2]
    r = min(out_h / h, out_w / w)
    nh, nw = max(1, int(round(h * r))), max(1, int(round(w * r)))
    small = pil_bilinear_u8(img, nh, nw)
    out = np.full((out_h, out_w) + img.shape[2:], fill, img.dtype)
    out[:nh, :nw] = small
    return out
