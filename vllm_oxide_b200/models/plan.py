"""The plan of a model: which parts, with which parameters, in which order.

An architecture turns its typed configuration into a `ModelPlan`; `CausalLM` builds the
plan.  Everything here is data: the layers are a list of block specs (each may choose a
different mixer, feed-forward or norm), and the order in which they run is a list too.
An `ExecStep` names a layer and the cache plane it uses; the same layer may be named twice
(each run with a plane of its own), and a step with `write_cache=False` reads the plane
that another step wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..parts.base import PartSpec


@dataclass(frozen=True)
class ExecStep:
    layer: int
    plane: Optional[int]        # cache plane / state index this run uses; None: the mixer keeps nothing
    write_cache: bool = True    # False: read what another run wrote into `plane`


@dataclass
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding_name: str
    lm_head_name: Optional[str]            # None: logits use the embedding table (tied)
    final_norm: PartSpec
    positions: Dict[str, PartSpec]
    layers: List[PartSpec]                 # block specs
    order: List[ExecStep]
    eos_token_id: Optional[int] = None
    default_dtype: str = "bfloat16"
    embedding_scale: float = 1.0           # the embedded tokens are multiplied by it
    logit_softcap: float = 0.0             # > 0: logits = cap * tanh(logits / cap)

    def num_planes(self) -> int:
        return 1 + max((s.plane for s in self.order if s.plane is not None), default=-1)

    def validate(self) -> None:
        writers = {}
        for s in self.order:
            if not 0 <= s.layer < len(self.layers):
                raise ValueError(f"order names layer {s.layer}, but the plan has {len(self.layers)} layers")
            if s.plane is not None and s.write_cache:
                if s.plane in writers:
                    raise ValueError(f"cache plane {s.plane} is written by two runs")
                writers[s.plane] = s.layer
        seen = set()
        for s in self.order:
            if s.plane is not None and s.write_cache:
                seen.add(s.plane)
            if s.plane is not None and not s.write_cache and s.plane not in seen:
                raise ValueError(f"a run reads cache plane {s.plane} before any run has written it")
