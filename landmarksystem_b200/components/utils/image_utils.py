"""PSNR helpers and depth visualisation (reference: landmark/nerf_components/utils/image_utils.py:17-53)."""
import numpy as np
import torch


def mse(img1, img2):
    return ((img1 - img2) ** 2).reshape(img1.shape[0], -1).mean(1, keepdim=True)


def psnr(img1, img2):
    m = ((img1 - img2) ** 2).reshape(img1.shape[0], -1).mean(1, keepdim=True)
    return 20 * torch.log10(1.0 / torch.sqrt(m))


def mse2psnr_npy(x):
    return -10.0 * np.log(x) / np.log(10.0)


def visualize_depth_numpy(depth, minmax=None):
    """Map a depth image to an 8-bit RGB jet-like ramp; returns ``(image, (lo, hi))``."""
    x = np.nan_to_num(depth)
    if minmax is None:
        pos = x[x > 0]
        lo, hi = (float(pos.min()), float(x.max())) if pos.size else (0.0, 1.0)
    else:
        lo, hi = minmax
    x = np.clip((x - lo) / (hi - lo + 1e-8), 0, 1)
    r = np.clip(1.5 - np.abs(4 * x - 3), 0, 1)
    g = np.clip(1.5 - np.abs(4 * x - 2), 0, 1)
    b = np.clip(1.5 - np.abs(4 * x - 1), 0, 1)
    return (np.stack((r, g, b), -1) * 255).astype(np.uint8), (lo, hi)
