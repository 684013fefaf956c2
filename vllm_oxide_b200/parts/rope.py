"""Rotary position encoding: the table of angles and the rule by which a mixer's kernel applies it.

The table is the reference's (vllm-oxide, crates/vllm-oxide/src/layers/rope.rs:50-88):
inv_freq[i] = 1 / theta^(2i/d) with a float32 pow, angle = float32(p) * inv_freq[i], and
[max_pos, d] = cos(angle) || sin(angle), all float32 on both paths.  The rotation itself
(rope.rs:129-159) happens inside the mixer's kernel, which gets the table and the rule from
`rotation_rule()`.  The reference rotates the whole head in halves (d = head_dim, rope.rs asserts it);
`rotary_dim` < head_dim rotates only the first elements of a head and `interleaved` pairs neighbouring
elements instead of halves: parameters an architecture's plan may set, not used by Qwen3.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, RotationRule, register_part


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, max_position: int, theta: float, rotary_dim: Optional[int] = None,
                 interleaved: bool = False, device=None, **_):
        d = head_dim if rotary_dim is None else int(rotary_dim)
        if d % 2 or not 0 < d <= head_dim:
            raise ValueError(f"rotary position encoding needs an even rotary_dim in (0, head_dim {head_dim}], got {d}")
        self.head_dim, self.rotary_dim, self.interleaved = head_dim, d, bool(interleaved)
        self.max_position, self.theta = max_position, float(theta)
        half = d // 2
        i = torch.arange(half, dtype=torch.float32)
        inv_freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), (2 * i) / d)
        t = torch.arange(max_position, dtype=torch.float32)
        freqs = t[:, None] * inv_freq[None, :]
        self.cos_sin = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous().to(device)

    def rotation_rule(self) -> RotationRule:
        return RotationRule(self.cos_sin, self.rotary_dim, self.interleaved)


register_part("position", "rope", RotaryEmbedding)
