"""Device memory of the cache: pages per plane, state slots per plane.

Every plane (a layer's cache) says through its `CacheSpec` what it stores a token: keys and values, or one
tensor; how wide; for all positions or a window; in pages of how many tokens; in which dtype.  Planes with the
same window and page size form a cache group: one page pool and one block table per request, managed on the
host by `KvCacheManager` (C++).  The reference keeps one buffer [2, layers, num_blocks, block_size, kv_heads,
head_dim] (vllm-oxide, crates/vllm-oxide/src/attention/mod.rs:42-85); here every plane has a [tensors, num_pages,
kv_heads, block_size, head_dim] buffer: planes of different widths can share a group, and the keys of one head
within a page are contiguous in memory (a decoding block reads one head's keys, and HBM serves long runs far
better than 256-byte pieces).  The pool is sized like the reference's (crates/vllm-oxide/src/llm.rs:485-537):
free memory times `gpu_memory_utilization`, divided by the bytes that one token takes in every plane, unless a
page count is given (in pages of the engine's page size; a group with pages of its own size gets as many pages
as hold the same number of tokens).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import host
from ..parts.base import CachePlane, CacheSpec, StateSpec


@dataclass
class CacheGroup:
    window: int
    block_size: int
    num_blocks: int
    planes: List[int]


class PagedCache:
    def __init__(self, cache_specs: List[Optional[CacheSpec]], state_specs: List[Optional[StateSpec]],
                 dtype: torch.dtype, device, block_size: int, num_blocks: Optional[int], num_state_slots: int,
                 gpu_memory_utilization: float = 0.9, prefix_caching: bool = False, reserve_bytes: int = 0):
        self.dtype, self.device, self.block_size = dtype, device, block_size
        for s in cache_specs:
            if s is not None and (s.tensors not in (1, 2) or s.kv_heads <= 0 or s.head_dim <= 0 or s.window < 0
                                  or (s.block_size is not None and s.block_size <= 0)):
                raise ValueError(f"unusable cache spec {s}")
        page_size = lambda s: s.block_size or block_size
        keys = sorted({(s.window, page_size(s)) for s in cache_specs if s is not None})
        if not keys:
            keys = [(0, block_size)]   # a model without paged keys still gets block tables (of a pool nobody reads)
        self.groups: List[CacheGroup] = [CacheGroup(w, bs, 0, []) for w, bs in keys]
        for plane, s in enumerate(cache_specs):
            if s is not None:
                self.groups[keys.index((s.window, page_size(s)))].planes.append(plane)
        width = lambda s: torch.empty((), dtype=s.dtype or dtype).element_size() * s.elements_per_token()
        token_bytes = sum(width(s) for s in cache_specs if s is not None)
        if num_blocks is None:
            if torch.device(device).type != "cuda":
                raise ValueError("num_kv_blocks must be given when the cache is not on a CUDA device")
            free, _ = torch.cuda.mem_get_info(device)
            budget = int(free * gpu_memory_utilization) - reserve_bytes
            num_blocks = budget // max(token_bytes * block_size, 1)
            if num_blocks < 1:
                raise RuntimeError(f"no memory for the cache: {free >> 20} MiB free, a page takes "
                                   f"{token_bytes * block_size} bytes")
        self.num_blocks = int(num_blocks)            # in pages of the engine's size
        for g in self.groups:
            g.num_blocks = max(1, self.num_blocks * block_size // g.block_size)
        self.planes: List[Optional[CachePlane]] = []
        for plane, s in enumerate(cache_specs):
            if s is None:
                self.planes.append(None)
                continue
            gi = keys.index((s.window, page_size(s)))
            g = self.groups[gi]
            buf = torch.zeros((s.tensors, g.num_blocks, s.kv_heads, g.block_size, s.head_dim), dtype=s.dtype or dtype,
                              device=device)
            self.planes.append(CachePlane(buf[0], buf[1] if s.tensors == 2 else None, gi, g.block_size, buf))
        self.num_state_slots = num_state_slots
        self.states: List[Optional[torch.Tensor]] = [
            None if s is None else torch.zeros((num_state_slots, *s.shape), dtype=s.dtype, device=device)
            for s in state_specs]
        self.manager = host.KvCacheManager(
            [host.GroupSpec(g.block_size, g.num_blocks, g.window) for g in self.groups], num_state_slots,
            # state of fixed size is not snapshotted at page boundaries: with such a layer nothing is skipped on a hit
            prefix_caching and not any(s is not None for s in state_specs))

    def bytes(self) -> int:
        total = sum(p.data.numel() * p.data.element_size() for p in self.planes if p is not None)
        return total + sum(s.numel() * s.element_size() for s in self.states if s is not None)

    @property
    def has_states(self) -> bool:
        return any(s is not None for s in self.states)

    def zero_states(self, slots: List[int]) -> None:
        if not slots:
            return
        idx = torch.as_tensor(slots, dtype=torch.long, device=self.device)
        for s in self.states:
            if s is not None:
                s.index_fill_(0, idx, 0)
