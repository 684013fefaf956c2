"""Grouped-query attention over the paged cache, with optional per-head q/k norm, bias and window.

The order is the reference's (vllm-oxide, crates/vllm-oxide/src/models/qwen3.rs:160-213):
merged q|k|v product, split, RMSNorm over head_dim of q and of k, rotation of q and k, keys
(after norm and rotation) and values written to the cache, attention with scale
1/sqrt(head_dim), output product.  Unlike the reference's prefill, which reads only the keys of
the current step (crates/vllm-oxide/src/attention/flash_attn.rs:15-37), every query here reads
its keys from the pages, so portions, cache hits, recomputation and decoding are one case.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import NO_ROTATION, CacheSpec, Mixer, Prenormed, register_part
from .linear import linear, linear_into_stream


class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                 qkv_bias: bool, qk_norm: bool, window: Optional[int], position: Optional[str], prefix: str,
                 positions: dict, dtype, device, **_):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if head_dim % 16 or head_dim > 512:
            raise ValueError(f"head_dim {head_dim} is not supported by the attention kernels "
                             f"(a multiple of 16 up to 512)")
        self.H, self.nh, self.kvh, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.eps, self.qkv_bias, self.qk_norm = float(eps), qkv_bias, qk_norm
        self.window = int(window or 0)
        # the position encoding is named by the plan; None (or a part that rotates nothing) leaves q and k as they are
        if position is not None and position not in positions:
            raise KeyError(f"the plan names position encoding {position!r}, but has only {sorted(positions)}")
        encoding = positions[position] if position is not None else None
        self.rotation = encoding.rotation_rule() if encoding is not None else NO_ROTATION
        self.prefix, self.dtype, self.device = prefix, dtype, device
        self.scale = 1.0 / math.sqrt(head_dim)   # qwen3.rs:204
        self.wqkv = self.wo = self.bqkv = self.wq_norm = self.wk_norm = None
        self._pairs = None      # this layer's counter for decode attention of many requests (made with the weights)

    # ---- tensors
    def _names(self):
        p = self.prefix
        return {k: f"{p}{k}" for k in ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                                       "q_proj.bias", "k_proj.bias", "v_proj.bias", "q_norm.weight", "k_norm.weight")}

    def tensor_specs(self) -> List[TensorSpec]:
        n, q, kv = self._names(), self.nh * self.hd, self.kvh * self.hd
        specs = [TensorSpec(n["q_proj.weight"], (q, self.H), "matrix", self.H),
                 TensorSpec(n["k_proj.weight"], (kv, self.H), "matrix", self.H),
                 TensorSpec(n["v_proj.weight"], (kv, self.H), "matrix", self.H),
                 TensorSpec(n["o_proj.weight"], (self.H, q), "matrix", q)]
        if self.qkv_bias:
            specs += [TensorSpec(n["q_proj.bias"], (q,), "bias"), TensorSpec(n["k_proj.bias"], (kv,), "bias"),
                      TensorSpec(n["v_proj.bias"], (kv,), "bias")]
        if self.qk_norm:
            specs += [TensorSpec(n["q_norm.weight"], (self.hd,), "norm"),
                      TensorSpec(n["k_norm.weight"], (self.hd,), "norm")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self._names()
        # rows of q, then k, then v (crates/vllm-oxide/src/layers/linear.rs:109-119)
        self.wqkv = torch.cat([tensors[n["q_proj.weight"]], tensors[n["k_proj.weight"]],
                               tensors[n["v_proj.weight"]]], dim=0).contiguous()
        self.wo = tensors[n["o_proj.weight"]].contiguous()
        if self.qkv_bias:
            self.bqkv = torch.cat([tensors[n["q_proj.bias"]], tensors[n["k_proj.bias"]],
                                   tensors[n["v_proj.bias"]]], dim=0).contiguous()
        if self.qk_norm:
            self.wq_norm = tensors[n["q_norm.weight"]].contiguous()
            self.wk_norm = tensors[n["k_norm.weight"]].contiguous()
        if self.wo.is_cuda:
            # a counter of this layer's own, so that no two launches that could overlap ever share one
            self._pairs = kernels.decode_pairs_counter(self.wo.device)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kvh, self.hd, self.window)

    # ---- one step
    adds_into_stream = True

    def forward(self, x, ctx, cache, state=None, write_cache: bool = True, add_into=None):
        """`add_into`: the residual stream; the output product then adds its result there and nothing is returned."""
        T = x.shape[0]
        width = (self.nh + 2 * self.kvh) * self.hd
        qkv = linear(x, self.wqkv, ctx.ws.get("qkv", T, width, x.dtype), ctx)
        g = cache.group
        kernels.qk_norm_rope_kv_write(qkv, self.bqkv, ctx.positions, ctx.slot_mapping[g], self.wq_norm, self.wk_norm,
                                      self.rotation, cache.k, cache.v, T, self.nh, self.kvh, self.hd, self.eps,
                                      write_cache, ctx.err)
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, x.dtype)
        self.attend(qkv, width, attn, cache, ctx, T)
        if add_into is not None:
            linear_into_stream(attn, self.wo, add_into)
            return None
        return linear(attn, self.wo, ctx.ws.get("attn_proj", T, self.H, x.dtype), ctx)

    # ---- the same with the residual stream kept inside the products (decode-sized steps)
    def can_forward_on_stream(self, stream, ctx) -> bool:
        T = stream.shape[0]
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, stream.dtype)
        return (kernels.gemm_skinny_supported(stream, self.wqkv) and kernels.gemm_skinny_supported(attn, self.wo))

    def forward_on_stream(self, stream, norm, ctx, cache, state=None, write_cache: bool = True, prenormed=None,
                          emit_norm=None):
        """stream += attention(RMSNorm(stream)): the norm is applied inside the q|k|v product, the sum made by the
        output product.  `prenormed` (a `Prenormed` of `norm`, left by the product that wrote the stream) spares the
        q|k|v product the norm's arithmetic; with `emit_norm` the output product leaves such a half-done norm behind
        for the part that follows, and it is returned."""
        T = stream.shape[0]
        width = (self.nh + 2 * self.kvh) * self.hd
        qkv = ctx.ws.get("qkv", T, width, stream.dtype)
        if prenormed is not None:
            kernels.gemm_skinny(prenormed.scaled, self.wqkv, qkv, kernels.EPI_BF16, ctx.err, eps=norm.eps,
                                prenormed=prenormed.parts)
        else:
            kernels.gemm_skinny(stream, self.wqkv, qkv, kernels.EPI_BF16, ctx.err, norm_weight=norm.weight, eps=norm.eps)
        g = cache.group
        kernels.qk_norm_rope_kv_write(qkv, self.bqkv, ctx.positions, ctx.slot_mapping[g], self.wq_norm, self.wk_norm,
                                      self.rotation, cache.k, cache.v, T, self.nh, self.kvh, self.hd, self.eps,
                                      write_cache, ctx.err)
        attn = ctx.ws.get("attn_out", T, self.nh * self.hd, stream.dtype)
        self.attend(qkv, width, attn, cache, ctx, T)
        left = leave_prenormed(emit_norm, "after_mixer", stream, ctx)
        kernels.gemm_skinny(attn, self.wo, stream, kernels.EPI_ADD, ctx.err,
                            emit=(emit_norm.weight, left.scaled, left.parts) if left else None)
        return left

    def attend(self, qkv, q_stride, out, cache, ctx, T):
        """bfloat16: decoding requests (one token) go to the split-key tensor-core kernel, requests with a
        portion to the tensor-core kernel for portions.  The 32-bit path, and sizes those kernels refuse,
        go to the plain kernel."""
        tables = ctx.block_tables[cache.group]
        if not kernels.has_fast_attention(qkv.dtype, self.hd, self.nh // self.kvh):
            kernels.paged_attention_generic(qkv, q_stride, out, cache.k, cache.v, tables, ctx.token_req, ctx.positions, T,
                                            self.nh, self.kvh, self.hd, self.window, self.scale, ctx.err)
            return
        B = ctx.launch_requests
        if ctx.num_decode > 0:
            keys = ctx.max_context if self.window == 0 else min(ctx.max_context, self.window)
            splits = decode_splits(B, self.kvh, keys, kernels.sm_count())
            n = kernels.attention_decode_scratch_floats(self.hd, B, self.nh, splits)
            scratch = ctx.ws.get_flat("attention_decode_scratch", n, torch.float32) if n else None
            kernels.attention_decode(qkv, q_stride, out, cache.k, cache.v, tables, ctx.cu_q, ctx.context_lens, B, self.nh,
                                     self.kvh, self.hd, self.window, self.scale, splits, scratch, ctx.err, pairs=self._pairs)
        if ctx.max_q > 1:
            kernels.attention_prefill(qkv, q_stride, out, cache.k, cache.v, tables, ctx.cu_q, ctx.context_lens, B,
                                      ctx.max_q, self.nh, self.kvh, self.hd, self.window, self.scale, ctx.err)


DECODE_BLOCKS_PER_SM = 2   # blocks of the decode attention kernel that fit an SM (its shared memory decides)


def leave_prenormed(norm, name: str, stream, ctx) -> Optional[Prenormed]:
    """Buffers for the half-done norm that a product adding into `stream` leaves for `norm` (None: nothing to leave)."""
    if norm is None or getattr(norm, "weight", None) is None:
        return None
    T, H = stream.shape
    scaled = ctx.ws.get("stream_scaled_" + name, T, H, stream.dtype)
    parts = ctx.ws.get_flat("stream_squares_" + name, kernels.gemm_skinny_weight_tiles(H) * 16, torch.float32)
    return Prenormed(norm, scaled, parts)


def decode_splits(num_requests: int, kv_heads: int, max_keys: int, num_sms: int) -> int:
    """Splits of the key range per (request, kv head): as many as keep every block resident at once
    (DECODE_BLOCKS_PER_SM blocks on each of the device's SMs), but at least two 64-key tiles per split.  Up to 8 the blocks of a
    (request, kv head) merge their results as a thread-block cluster, without a second kernel; beyond that a second
    kernel merges them, which pays only for few requests with long contexts (one request of 32,000 keys: 56 us with
    8 splits, 44 us with 16, 37 us with 32), so more than 8 are taken only from 8,192 keys on and only if at least 12
    fit, and 32 only from 16,384 keys on and only if all 32 fit (with 18 of them two requests were slower than with 16)."""
    tiles = -(-max_keys // 64)
    fit = (DECODE_BLOCKS_PER_SM * num_sms) // max(1, num_requests * kv_heads)
    most = 8 if tiles < 128 else (32 if tiles >= 256 and fit >= 32 else 16)
    splits = max(1, min(fit, tiles // 2, most))
    return splits if splits <= 8 or splits >= 12 else 8


register_part("mixer", "attention", Attention)
