"""Per-request sampling options, with the reference's names, meanings and defaults
(vllm-oxide, crates/vllm-oxide/src/sampler.rs:35-90)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0: greedy argmax
    top_k: Optional[int] = None       # keep tokens whose logit is >= the k-th largest (ties kept); 1: greedy
    top_p: Optional[float] = None     # nucleus; applied for 0 < p < 1
    max_tokens: int = 16
    ignore_eos: bool = False
    presence_penalty: float = 0.0     # 0 = off for all three
    frequency_penalty: float = 0.0
    repetition_penalty: float = 0.0
    # None: the engine's seed, and the random numbers are keyed by (seed, request id, token index).  Given: they are
    # keyed by (seed, token index) only, so the same prompt and seed give the same tokens in any call and any batch.
    seed: Optional[int] = None

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.top_k is not None and self.top_k < 1:
            raise ValueError(f"top_k must be >= 1, got {self.top_k}")
        if self.top_p is not None and not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1
