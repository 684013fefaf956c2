"""Interfaces of the parts a model is put together from, and the registries that name them.

A model is a list of blocks; a block arranges a token mixer, a feed-forward and norms; a
mixer may use a position encoding.  Every part takes its sizes and constants as
constructor parameters and is chosen by kind name, layer by layer, from a `PartSpec`.  No
part knows which model it is in: it sees its own tensors (by the checkpoint names it is
given), the step's batch, its cache plane or state, and a workspace for activations.

Interfaces (duck-typed; the base classes document them):

  Norm.forward(x, residual, ctx, rows=None)   -> (y, residual)   fused add + norm
  PositionEncoding                              a table plus what the mixer's kernel needs of it
  Mixer.forward(x, ctx, cache, state)          -> [T, hidden]
  FeedForward.forward(x, ctx)                  -> [T, hidden]
  Block.forward(hidden, residual, ctx, cache, state) -> (hidden, residual)

and, for every part that owns tensors:

  tensor_specs() -> [TensorSpec]      what it needs from the checkpoint
  load(tensors: {name: tensor})       called once with exactly those tensors
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class PartSpec:
    """Which part, and its parameters: the configuration's choice for one place in one layer."""
    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps in pages, a token: `tensors` tensors (2: keys and values; 1: a single tensor, e.g. a latent that
    stands for both) of `kv_heads * head_dim` elements each, for all positions (window 0) or the last `window`; in pages
    of `block_size` tokens (None: the engine's page size) and in `dtype` (None: the model's).  A plane is stored as
    [tensors, pages, kv_heads, block_size, head_dim].  Planes with equal windows and page sizes share a group: one page
    pool and one block table per request, whatever their widths, tensors and dtypes."""
    kv_heads: int
    head_dim: int
    window: int = 0
    tensors: int = 2
    block_size: Optional[int] = None
    dtype: Optional[torch.dtype] = None

    def elements_per_token(self) -> int:
        return self.tensors * self.kv_heads * self.head_dim


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size that a mixer keeps beside (or instead of) the paged cache."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CachePlane:
    """One layer's pages: `k` (the first, or only, tensor) and `v` (the second, None for a one-tensor plane), each
    [num_pages, kv_heads, block_size, head_dim]; `data` is both as one tensor [tensors, num_pages, ...]."""
    k: torch.Tensor
    v: Optional[torch.Tensor]
    group: int
    block_size: int
    data: Optional[torch.Tensor] = None


@dataclass
class Prenormed:
    """One half of an RMSNorm, done ahead by the product that wrote the residual stream: `scaled` = bfloat16(stream *
    norm.weight) and `parts`, sums of squares of the stream that add up to each token's (see kernels.gemm_skinny).  The
    product that follows `norm` takes `scaled` as its tokens and applies 1/rms itself."""
    norm: "Norm"
    scaled: torch.Tensor
    parts: torch.Tensor


class Workspace:
    """Activation buffers with fixed addresses: allocated once for the largest step and handed out
    by name, so that a step captured in a CUDA graph finds them where they were."""

    def __init__(self, max_rows: int, device, dtype: torch.dtype):
        self.max_rows, self.device, self.dtype = max_rows, device, dtype
        self._buffers: Dict[tuple, torch.Tensor] = {}

    def get(self, name: str, rows: int, cols: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        dtype = dtype or self.dtype
        key = (name, cols, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, self.max_rows)
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def get_rows(self, name: str, rows: int, cols: int, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A buffer whose row count follows demand (wanted rows, not tokens): it grows when asked for
        more rows than it has, and never shrinks."""
        dtype = dtype or self.dtype
        key = (name, cols, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            buf = torch.empty((max(rows, 1), cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def get_flat(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """Scratch memory of a kernel: a flat buffer that grows on demand (`zero`: filled with zeros when made)."""
        key = (name, 0, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            make = torch.zeros if zero else torch.empty
            buf = make(max(numel, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:numel]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


class Part:
    # True when forward() launches the same kernels, with the same arguments, whatever the step's batch
    # holds (everything that varies is read on the device): such a part can be captured in a CUDA graph.
    graph_safe = False

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def parts(self) -> List["Part"]:
        """The parts this part is made of (a block: its norms, mixer and feed-forward)."""
        return []

    def device_tensors(self) -> List[torch.Tensor]:
        """Every tensor this part and its parts hold (weights as loaded or merged, tables): what a step may read."""
        own = [v for v in vars(self).values() if isinstance(v, torch.Tensor)]
        for v in vars(self).values():
            if isinstance(v, (list, tuple)):
                own += [t for t in v if isinstance(t, torch.Tensor)]
        return own + [t for p in self.parts() for t in p.device_tensors()]


class Norm(Part):
    def forward(self, x, residual, ctx, rows=None, n_rows=None):
        """(norm(x + residual), x + residual).  x may be None: the block before has already added its output into
        `residual`, and the norm is of `residual` itself."""
        raise NotImplementedError


@dataclass(frozen=True)
class RotationRule:
    """What a mixer's kernel needs of a rotary position encoding: the first `rotary_dim` elements of every query and key
    head are rotated (0: none), in pairs (i, i + rotary_dim/2) or, `interleaved`, in pairs (2i, 2i + 1), by the angles of
    the token's position in `table`: float32 [max_position, rotary_dim], cos of rotary_dim/2 angles, then their sin."""
    table: Optional[torch.Tensor]
    rotary_dim: int
    interleaved: bool = False


NO_ROTATION = RotationRule(None, 0, False)


class PositionEncoding(Part):
    graph_safe = True      # the default embed() launches nothing

    def embed(self, hidden: torch.Tensor, ctx) -> None:
        """Adds what this encoding contributes to the embedded tokens, in place (absolute or learned positions: a table
        row per `ctx.positions`); the default adds nothing.  Called once a step, after the embedding."""

    def rotation_rule(self) -> RotationRule:
        """The rule a mixer hands to its rotation kernel; a position encoding that rotates nothing (absolute positions
        added elsewhere, or none at all) keeps this default."""
        return NO_ROTATION


class Mixer(Part):
    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x, ctx, cache: Optional[CachePlane], state: Optional[torch.Tensor], write_cache: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    def forward(self, hidden, residual, ctx, cache, state, write_cache=True):
        raise NotImplementedError


# ------------------------------------------------------------------ registries
_REGISTRIES: Dict[str, Dict[str, Callable]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}}


def register_part(family: str, kind: str, factory: Callable) -> None:
    """Makes `factory(**params, **common)` available under (family, kind).  Families: norm, position,
    mixer, feed_forward, block.  Registering a kind twice replaces it (tests register toy parts)."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; families are {sorted(_REGISTRIES)}")
    _REGISTRIES[family][kind] = factory


def build_part(family: str, spec: PartSpec, **common):
    try:
        factory = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} part of kind {spec.kind!r}; known: {sorted(_REGISTRIES[family])}") from None
    return factory(**spec.params, **common)


def known_parts(family: str) -> List[str]:
    return sorted(_REGISTRIES[family])
