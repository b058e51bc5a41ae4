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
