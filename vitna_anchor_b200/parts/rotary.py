"""Rotary position encoding in half-split form: tables built on the host in float32.

inv_freq[j] = 1 / theta^(2j / rot_dim); angle = (float)pos * inv_freq[j];
cos and sin of the angle in float32 (engine/src/model.c:408-413, 899-904; the
reference's GPU path also uses host-built tables so that both devices share
the bits, model.c:1213-1232).  The mixer rotates pairs (j, j + rot_dim/2) of
the first rot_dim dimensions of every q and k head.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding


class Rotary(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, device, rot_dim: int = 0):
        rot_dim = rot_dim or head_dim
        if rot_dim % 2 or rot_dim > head_dim:
            raise ValueError("the rotated part of a head must be even and no larger than the head")
        self.head_dim, self.theta, self.max_positions, self.rot_dim = head_dim, float(theta), max_positions, rot_dim
        j2 = np.arange(0, rot_dim, 2, dtype=np.float32)
        inv_freq = (np.float32(1.0) / np.power(np.float32(theta), j2 / np.float32(rot_dim))).astype(np.float32)
        angle = (np.arange(max_positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
        self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(device)
        self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(device)

    def tensors(self):
        return []  # tables are read a row per token; they are not counted as weights

    def rotary_tables(self):
        return self.cos, self.sin, self.rot_dim


class NoPositionEncoding(PositionEncoding):
    """Nothing is added or rotated."""


def blended_frequencies(base: float, dims: int, scaling=None):
    """Frequencies of a rotation over `dims` values, f_i = base^(-2i/dims), i < dims/2, and the factor on cos and sin.

    With scaling = (factor, original, fast, slow) the frequencies of long wavelengths are divided by `factor` and those of
    short ones kept, with a linear ramp over i between them (the YaRN recipe): with
    at(turns) = dims * ln(original / (2 pi turns)) / (2 ln base),  lo = max(floor(at(fast)), 0),  hi = min(ceil(at(slow)), dims - 1),
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)  the frequency is  f_i / factor * ramp_i + f_i * (1 - ramp_i),  and cos
    and sin are multiplied by 0.1 ln(factor) + 1.  Worked out in float64 on the host; -> (float32 [dims/2] array, float)."""
    import math
    if dims % 2:
        raise ValueError("a rotation turns an even number of values")
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    if scaling is None:
        return f.astype(np.float32), 1.0
    factor, original, fast, slow = (float(v) for v in scaling)
    at = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
    lo, hi = max(math.floor(at(fast)), 0), min(math.ceil(at(slow)), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32), 0.1 * math.log(factor) + 1.0
