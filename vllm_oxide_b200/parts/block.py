"""The arrangement of parts in one layer.

"pre_norm" is the reference's decoder layer (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:247-258):
add+norm -> mixer -> add+norm -> feed-forward, carrying (hidden, residual) so that each residual
add is fused into the following norm.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights.loader import TensorSpec
from .base import Block, PartSpec, build_part, register_part


class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, input_norm: PartSpec, post_mixer_norm: PartSpec,
                 **common):
        self.input_norm = build_part("norm", input_norm, **common)
        self.mixer = build_part("mixer", mixer, **common)
        self.post_mixer_norm = build_part("norm", post_mixer_norm, **common)
        self.feed_forward = build_part("feed_forward", feed_forward, **common)
        self._parts = [self.input_norm, self.mixer, self.post_mixer_norm, self.feed_forward]
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load({s.name: tensors[s.name] for s in p.tensor_specs()})

    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        normed, residual = self.input_norm.forward(hidden, residual, ctx)
        mixed = self.mixer.forward(normed, ctx, cache, state, write_cache)
        normed, residual = self.post_mixer_norm.forward(mixed, residual, ctx)
        return self.feed_forward.forward(normed, ctx), residual


register_part("block", "pre_norm", PreNormBlock)
