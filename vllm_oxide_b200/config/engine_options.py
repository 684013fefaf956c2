"""Options of one engine instance, with the reference's names and defaults.

`EngineOptions` of the reference (vllm-oxide, crates/vllm-oxide/src/llm.rs:28-55) has
max_num_batched_tokens 16384, max_num_seqs 512, max_model_len 4096,
gpu_memory_utilization 0.9, enforce_eager and dtype.  Added here: the page size (fixed at
256 in the reference, crates/vllm-oxide/src/engine/sequence.rs:20), an explicit pool size,
the sampling seed and the prefix-cache switch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineOptions:
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    enforce_eager: bool = False      # False: decode steps are replayed from CUDA graphs
    dtype: Optional[str] = None      # None: bfloat16; "bfloat16" or "float32" (true 32-bit)
    block_size: int = 256            # tokens per cache page
    num_kv_blocks: Optional[int] = None   # pages per cache group; None: sized from free memory
    seed: int = 0
    enable_prefix_caching: bool = True

    def validate(self) -> None:
        if self.block_size <= 0 or self.block_size % 16:
            raise ValueError(f"block_size must be a positive multiple of 16, got {self.block_size}")
        if self.max_num_batched_tokens <= 0 or self.max_num_seqs <= 0 or self.max_model_len <= 0:
            raise ValueError("max_num_batched_tokens, max_num_seqs and max_model_len must be positive")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.dtype not in (None, "bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        if self.num_kv_blocks is not None and self.num_kv_blocks <= 0:
            raise ValueError("num_kv_blocks must be positive")
