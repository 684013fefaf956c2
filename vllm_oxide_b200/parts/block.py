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
from .norm import RMSNorm

# Decode-sized steps keep the residual stream inside the products of the attention and the feed-forward (see
# PreNormBlock._keeps_stream); False runs the separate add+norm kernels always.
STREAM_IN_PRODUCTS = True
# Every step the weight-streaming product takes (up to 16 tokens).  Measured at Qwen3-8B sizes against the separate
# add+norm kernels: 323 against 314 tokens/s at batch 1, 2,385 against 2,306 at batch 8 with the norm's arithmetic inside
# the loop of the product that follows the norm (at batch 16 that arithmetic cost what the two kernels saved); with
# NORM_AHEAD the step takes 3.01 against 3.12 ms at batch 1, 3.27 against 3.42 at batch 8, 3.91 against 4.09 at batch 16.
STREAM_MAX_TOKENS = 16
# The product that writes the stream also does the arithmetic of the norm that follows (stream * weight, sums of squares
# per tile), so the next product runs its plain loop and only scales by 1/rms at its end: about 2 us less for each of
# the two products a layer that follow a norm.
NORM_AHEAD = True
# Steps of more than 16 tokens: the library's output and down products add into the residual stream (the stream is their
# addend), so the add+norm kernels that follow read one tensor and write one instead of reading two and writing two.
ADD_IN_PRODUCTS = True


class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, input_norm: PartSpec, post_mixer_norm: PartSpec,
                 **common):
        self.input_norm = build_part("norm", input_norm, **common)
        self.mixer = build_part("mixer", mixer, **common)
        self.post_mixer_norm = build_part("norm", post_mixer_norm, **common)
        self.feed_forward = build_part("feed_forward", feed_forward, **common)
        self._parts = [self.input_norm, self.mixer, self.post_mixer_norm, self.feed_forward]
        self.graph_safe = all(p.graph_safe for p in self._parts)

    def parts(self):
        return list(self._parts)

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load({s.name: tensors[s.name] for s in p.tensor_specs()})

    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        """(hidden, residual) in and out.  hidden None means that the part before has already added its output into
        `residual` (the stream); this block leaves it so too when its parts can keep the stream inside their products."""
        if (hidden is None or residual is None) and self._keeps_stream(hidden if residual is None else residual, ctx):
            stream = hidden if residual is None else residual
            # the half of this block's first norm that the block before may have left; what this block leaves for the next
            ahead = getattr(ctx, "prenormed", None)
            ahead = ahead if NORM_AHEAD and ahead is not None and ahead.norm is self.input_norm else None
            after = self.mixer.forward_on_stream(stream, self.input_norm, ctx, cache, state, write_cache, prenormed=ahead,
                                                 emit_norm=self.post_mixer_norm if NORM_AHEAD else None)
            nxt = getattr(ctx, "next_norm", None) if NORM_AHEAD else None
            ctx.prenormed = self.feed_forward.forward_on_stream(stream, self.post_mixer_norm, ctx, prenormed=after,
                                                                emit_norm=nxt if isinstance(nxt, RMSNorm) else None)
            return None, stream
        ctx.prenormed = None
        normed, residual = self.input_norm.forward(hidden, residual, ctx)
        if self._adds_in_products(residual):
            # larger bfloat16 steps: the library's output and down products take the stream as their addend
            self.mixer.forward(normed, ctx, cache, state, write_cache, add_into=residual)
            normed, residual = self.post_mixer_norm.forward(None, residual, ctx)
            self.feed_forward.forward(normed, ctx, add_into=residual)
            return None, residual
        mixed = self.mixer.forward(normed, ctx, cache, state, write_cache)
        normed, residual = self.post_mixer_norm.forward(mixed, residual, ctx)
        return self.feed_forward.forward(normed, ctx), residual

    def _adds_in_products(self, stream) -> bool:
        """bfloat16 steps too large for the weight-streaming kernel, with a mixer and a feed-forward that can add their
        result into the stream themselves (`adds_into_stream`, `forward(..., add_into=stream)`)."""
        return (ADD_IN_PRODUCTS and stream.dtype == torch.bfloat16 and stream.shape[0] > STREAM_MAX_TOKENS
                and getattr(self.mixer, "adds_into_stream", False) and getattr(self.feed_forward, "adds_into_stream", False))

    def _keeps_stream(self, stream, ctx) -> bool:
        """Decode-sized bfloat16 steps whose norms are RMSNorm and whose mixer and feed-forward offer
        forward_on_stream(stream, norm, ...): stream += part(norm(stream)), with the norm applied inside the part's
        first product and the sum made by its last one (two kernels less a layer)."""
        if not STREAM_IN_PRODUCTS or stream.dtype != torch.bfloat16 or stream.shape[0] > STREAM_MAX_TOKENS:
            return False
        if not (isinstance(self.input_norm, RMSNorm) and isinstance(self.post_mixer_norm, RMSNorm)):
            return False
        can_m = getattr(self.mixer, "can_forward_on_stream", None)
        can_f = getattr(self.feed_forward, "can_forward_on_stream", None)
        return bool(can_m and can_f and can_m(stream, ctx) and can_f(stream, ctx))


register_part("block", "pre_norm", PreNormBlock)
