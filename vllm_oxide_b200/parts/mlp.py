"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ) with gate and up merged into one product
(vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:60-87, crates/vllm-oxide/src/layers/activation.rs:17-21)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part
from .linear import linear, linear_into_stream, tc5_product


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str, **_):
        self.H, self.I, self.prefix = hidden_size, intermediate_size, prefix
        self.wgu = self.wdown = None
        self.interleaved = False

    def tensor_specs(self) -> List[TensorSpec]:
        p = self.prefix
        return [TensorSpec(p + "gate_proj.weight", (self.I, self.H), "matrix", self.H),
                TensorSpec(p + "up_proj.weight", (self.I, self.H), "matrix", self.H),
                TensorSpec(p + "down_proj.weight", (self.H, self.I), "matrix", self.I)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        self.interleaved = self.I % 8 == 0
        if self.interleaved:
            # groups of eight gate rows followed by the eight up rows of the same outputs: one 16-row tile of the
            # product then holds both halves of eight outputs, and the activation becomes the product's epilogue
            self.wgu = torch.stack([gate.reshape(self.I // 8, 8, self.H), up.reshape(self.I // 8, 8, self.H)],
                                   dim=1).reshape(2 * self.I, self.H).contiguous()
        else:
            # rows of gate, then up (crates/vllm-oxide/src/layers/linear.rs:132-138)
            self.wgu = torch.cat([gate, up], dim=0).contiguous()
        self.wdown = tensors[p + "down_proj.weight"].contiguous()

    adds_into_stream = True

    def forward(self, x, ctx, add_into=None):
        """`add_into`: the residual stream; the down product then adds its result there and nothing is returned."""
        T = x.shape[0]
        act = ctx.ws.get("act", T, self.I, x.dtype)
        if self.interleaved and kernels.gemm_skinny_supported(x, self.wgu):
            # decode-sized steps: the activation is the epilogue of the gate|up product
            kernels.gemm_skinny(x, self.wgu, act, kernels.EPI_SWIGLU, ctx.err)
        elif self.interleaved and tc5_product(x, self.wgu, act, kernels.EPI_SWIGLU, ctx):
            pass
        else:
            gu = linear(x, self.wgu, ctx.ws.get("gate_up", T, 2 * self.I, x.dtype), ctx)
            kernels.silu_mul(gu, act, T, self.interleaved)
        if add_into is not None:
            linear_into_stream(act, self.wdown, add_into)
            return None
        return linear(act, self.wdown, ctx.ws.get("mlp_out", T, self.H, x.dtype), ctx)

    # ---- the same with the residual stream kept inside the products (decode-sized steps)
    def can_forward_on_stream(self, stream, ctx) -> bool:
        act = ctx.ws.get("act", stream.shape[0], self.I, stream.dtype)
        return (self.interleaved and kernels.gemm_skinny_supported(stream, self.wgu)
                and kernels.gemm_skinny_supported(act, self.wdown))

    def forward_on_stream(self, stream, norm, ctx, prenormed=None, emit_norm=None):
        """stream += down(SiLU(gate) * up) of RMSNorm(stream): the norm inside the gate|up product, the sum made by
        the down product.  `prenormed` / `emit_norm` as in the attention part: the norm's arithmetic done by the product
        before, and left behind for the part after."""
        from .attention import leave_prenormed
        act = ctx.ws.get("act", stream.shape[0], self.I, stream.dtype)
        if prenormed is not None:
            kernels.gemm_skinny(prenormed.scaled, self.wgu, act, kernels.EPI_SWIGLU, ctx.err, eps=norm.eps,
                                prenormed=prenormed.parts)
        else:
            kernels.gemm_skinny(stream, self.wgu, act, kernels.EPI_SWIGLU, ctx.err, norm_weight=norm.weight, eps=norm.eps)
        left = leave_prenormed(emit_norm, "after_feed_forward", stream, ctx)
        kernels.gemm_skinny(act, self.wdown, stream, kernels.EPI_ADD, ctx.err,
                            emit=(emit_norm.weight, left.scaled, left.parts) if left else None)
        return left


register_part("feed_forward", "swiglu", SwiGLU)
