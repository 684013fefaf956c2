"""A causal language model built from a `ModelPlan`: embedding, blocks in plan order, last norm,
output product.

The engine-facing contract is the reference's `CausalLM` (vllm-oxide,
crates/vllm-oxide/src/causal_lm.rs:13-18: forward(input_ids, positions) -> hidden,
compute_logits(hidden) -> logits), with the step's batch descriptor as an explicit argument
instead of a shared mutex (crates/vllm-oxide/src/attention/mod.rs:34-38): `forward(ctx)` returns
the residual stream before the last norm, `compute_logits(hidden, residual, ctx)` applies the last
norm and the output product on the wanted rows only and returns float32 logits.

What surrounds the blocks is data of the plan too: a scale on the embedded tokens, position parts that add
to the embedding (`PositionEncoding.embed`), a soft cap on the logits.  Qwen3 uses none of the three.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..parts.base import CachePlane, CacheSpec, StateSpec, build_part
from ..parts.linear import linear, tc5_product
from ..weights.loader import TensorSpec
from .plan import ModelPlan


class CausalLM:
    def __init__(self, plan: ModelPlan, dtype: torch.dtype, device):
        plan.validate()
        self.plan, self.dtype, self.device = plan, dtype, device
        self.positions = {name: build_part("position", spec, device=device) for name, spec in plan.positions.items()}
        common = dict(positions=self.positions, dtype=dtype, device=device)
        self.blocks = [build_part("block", spec, **common) for spec in plan.layers]
        self.final_norm = build_part("norm", plan.final_norm, **common)
        self.graph_safe = (all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
                           and all(p.graph_safe for p in self.positions.values()))
        self.embedding = None
        self.lm_head = None
        self.planes: List[Optional[CachePlane]] = [None] * plan.num_planes()
        self.states: List[Optional[torch.Tensor]] = [None] * plan.num_planes()

    # ---- what the model needs
    @property
    def vocab_size(self) -> int:
        return self.plan.vocab_size

    def tensor_specs(self) -> List[TensorSpec]:
        p = self.plan
        specs = [TensorSpec(p.embedding_name, (p.vocab_size, p.hidden_size), "embedding")]
        if p.lm_head_name:
            specs.append(TensorSpec(p.lm_head_name, (p.vocab_size, p.hidden_size), "matrix", p.hidden_size))
        for part in self.positions.values():
            specs += part.tensor_specs()
        for b in self.blocks:
            specs += b.tensor_specs()
        specs += self.final_norm.tensor_specs()
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        p = self.plan
        self.embedding = tensors[p.embedding_name].contiguous()
        self.lm_head = tensors[p.lm_head_name].contiguous() if p.lm_head_name else self.embedding
        for part in self.positions.values():
            part.load({s.name: tensors[s.name] for s in part.tensor_specs()})
        for b in self.blocks:
            b.load({s.name: tensors[s.name] for s in b.tensor_specs()})
        self.final_norm.load({s.name: tensors[s.name] for s in self.final_norm.tensor_specs()})

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        """Per plane: what its writer's mixer keeps in pages (None: nothing)."""
        out: List[Optional[CacheSpec]] = [None] * self.plan.num_planes()
        for s in self.plan.order:
            if s.plane is not None and s.write_cache:
                out[s.plane] = self.blocks[s.layer].mixer.cache_spec()
        return out

    def state_specs(self) -> List[Optional[StateSpec]]:
        """Per plane: the fixed-size per-request state of its writer's mixer (None: none)."""
        out: List[Optional[StateSpec]] = [None] * self.plan.num_planes()
        for s in self.plan.order:
            if s.plane is not None and s.write_cache:
                out[s.plane] = self.blocks[s.layer].mixer.state_spec()
        return out

    def bind(self, planes: List[Optional[CachePlane]], states: List[Optional[torch.Tensor]]) -> None:
        self.planes, self.states = list(planes), list(states)

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor (a tied output matrix counts once)."""
        seen, total = set(), 0
        tensors = [self.embedding, self.lm_head] + self.final_norm.device_tensors()
        for part in self.positions.values():
            tensors += part.device_tensors()
        for b in self.blocks:
            tensors += b.device_tensors()
        for t in tensors:
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # ---- one step
    def forward(self, ctx):
        T = ctx.launch_tokens
        hidden = ctx.ws.get("embedded", T, self.plan.hidden_size, self.dtype)
        kernels.embedding(self.embedding, ctx.token_ids, hidden, T, ctx.err, self.plan.embedding_scale)
        for part in self.positions.values():
            part.embed(hidden, ctx)
        residual = None
        order = self.plan.order
        ctx.prenormed = None
        for i, s in enumerate(order):
            plane = self.planes[s.plane] if s.plane is not None else None
            state = self.states[s.plane] if s.plane is not None else None
            # a hint for blocks that can use it: the first norm of the block that runs next (its arithmetic may be done
            # by the product that writes the residual stream); the last block has none
            ctx.next_norm = getattr(self.blocks[order[i + 1].layer], "input_norm", None) if i + 1 < len(order) else None
            hidden, residual = self.blocks[s.layer].forward(hidden, residual, ctx, plane, state, s.write_cache)
        ctx.next_norm = ctx.prenormed = None
        return hidden, residual

    def compute_logits(self, hidden, residual, ctx) -> torch.Tensor:
        R = ctx.launch_rows
        normed, _ = self.final_norm.forward(hidden, residual, ctx, rows=ctx.logit_rows, n_rows=R, name="final_normed")
        out = self._logits(normed, R, ctx)
        if self.plan.logit_softcap > 0.0:
            kernels.softcap(out, R, self.plan.logit_softcap)
        return out

    def _logits(self, normed, R: int, ctx) -> torch.Tensor:
        V = self.plan.vocab_size
        if self.dtype == torch.float32:
            return linear(normed, self.lm_head, ctx.ws.get_rows("logits", R, V, self.dtype), ctx)
        out = ctx.ws.get_rows("logits_f32", R, V, torch.float32)
        if kernels.gemm_skinny_supported(normed, self.lm_head):
            kernels.gemm_skinny(normed, self.lm_head, out, kernels.EPI_F32, ctx.err)   # rounds to bfloat16, stores float
        elif tc5_product(normed, self.lm_head, out, kernels.EPI_F32, ctx):
            pass
        else:
            out.copy_(linear(normed, self.lm_head, ctx.ws.get_rows("logits", R, V, self.dtype), ctx))
        return out
