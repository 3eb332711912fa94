"""Assorted math helpers for the Gaussian models (reference:
landmark/nerf_components/utils/general_utils.py:15-102)."""
import numpy as np
import torch


def inverse_sigmoid(x):
    return torch.log(x / (1 - x))


def get_expon_lr_func(lr_init, lr_final, lr_delay_steps=0, lr_delay_mult=1.0, max_steps=1000000):
    """Log-linear interpolation from ``lr_init`` to ``lr_final`` with an optional smooth warm-up."""

    def helper(step):
        if step < 0 or (lr_init == 0.0 and lr_final == 0.0):
            return 0.0
        if lr_delay_steps > 0:
            delay = lr_delay_mult + (1 - lr_delay_mult) * np.sin(0.5 * np.pi * np.clip(step / lr_delay_steps, 0, 1))
        else:
            delay = 1.0
        t = np.clip(step / max_steps, 0, 1)
        return delay * np.exp(np.log(lr_init) * (1 - t) + np.log(lr_final) * t)

    return helper


def strip_lowerdiag(L):
    return torch.stack((L[:, 0, 0], L[:, 0, 1], L[:, 0, 2], L[:, 1, 1], L[:, 1, 2], L[:, 2, 2]), dim=-1)


def strip_symmetric(sym):
    return strip_lowerdiag(sym)


def build_rotation(r):
    """Unit-normalise quaternions ``[N, 4]`` (w, x, y, z) and return rotation matrices ``[N, 3, 3]``."""
    q = r / r.norm(dim=1, keepdim=True)
    w, x, y, z = q.unbind(-1)
    return torch.stack((
        1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
        2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
        2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)), dim=-1).reshape(-1, 3, 3)


def build_scaling_rotation(s, r):
    return build_rotation(r) * s[:, None, :]
