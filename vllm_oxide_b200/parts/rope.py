"""Rotate-half rotary position encoding over the whole head.

The table is the reference's (vllm-oxide, crates/vllm-oxide/src/layers/rope.rs:50-88):
inv_freq[i] = 1 / theta^(2i/hd) with a float32 pow, angle = float32(p) * inv_freq[i], and
[max_pos, hd] = cos(angle) || sin(angle), all float32 on both paths.  The rotation itself
(rope.rs:129-159) happens inside the mixer's kernel, which reads this table by position.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, max_position: int, theta: float, device=None, **_):
        if head_dim % 2:
            raise ValueError(f"rotary position encoding needs an even head_dim, got {head_dim}")
        self.head_dim, self.max_position, self.theta = head_dim, max_position, float(theta)
        half = head_dim // 2
        i = torch.arange(half, dtype=torch.float32)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), (2 * i) / head_dim)
        t = torch.arange(max_position, dtype=torch.float32)
        freqs = t[:, None] * inv_freq[None, :]
        self.cos_sin = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous().to(device)


register_part("position", "rope", RotaryEmbedding)
