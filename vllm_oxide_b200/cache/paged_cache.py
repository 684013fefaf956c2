"""Device memory of the cache: pages of keys and values per plane, state slots per plane.

Planes whose mixers have the same needs (the same window) form a cache group: one page pool and
one block table per request, managed on the host by `KvCacheManager` (C++).  The reference keeps
one buffer [2, layers, num_blocks, block_size, kv_heads, head_dim] (vllm-oxide,
crates/vllm-oxide/src/attention/mod.rs:42-85); here every plane has a [2, num_pages, kv_heads,
block_size, head_dim] buffer: planes of different widths can share a group, and the keys of one head
within a page are contiguous in memory (a decoding block reads one head's keys, and HBM serves long
runs far better than 256-byte pieces).  The pool is sized
like the reference's (crates/vllm-oxide/src/llm.rs:485-537): free memory times
`gpu_memory_utilization`, divided by the bytes of one page in every plane, unless a page count
is given.
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
        windows = sorted({s.window for s in cache_specs if s is not None})
        if not windows:
            windows = [0]   # a model without paged keys still gets block tables (of a pool nobody reads)
        self.groups: List[CacheGroup] = [CacheGroup(w, block_size, 0, []) for w in windows]
        for plane, s in enumerate(cache_specs):
            if s is not None:
                self.groups[windows.index(s.window)].planes.append(plane)
        elt = torch.empty((), dtype=dtype).element_size()
        page_bytes = sum(2 * block_size * s.kv_heads * s.head_dim * elt for s in cache_specs if s is not None)
        if num_blocks is None:
            if torch.device(device).type != "cuda":
                raise ValueError("num_kv_blocks must be given when the cache is not on a CUDA device")
            free, _ = torch.cuda.mem_get_info(device)
            budget = int(free * gpu_memory_utilization) - reserve_bytes
            num_blocks = budget // max(page_bytes, 1)
            if num_blocks < 1:
                raise RuntimeError(f"no memory for the cache: {free >> 20} MiB free, a page takes {page_bytes} bytes")
        for g in self.groups:
            g.num_blocks = int(num_blocks)
        self.num_blocks = int(num_blocks)
        self.planes: List[Optional[CachePlane]] = []
        for plane, s in enumerate(cache_specs):
            if s is None:
                self.planes.append(None)
                continue
            gi = windows.index(s.window)
            buf = torch.zeros((2, self.num_blocks, s.kv_heads, block_size, s.head_dim), dtype=dtype, device=device)
            self.planes.append(CachePlane(buf[0], buf[1], gi, block_size))
        self.num_state_slots = num_state_slots
        self.states: List[Optional[torch.Tensor]] = [
            None if s is None else torch.zeros((num_state_slots, *s.shape), dtype=s.dtype, device=device)
            for s in state_specs]
        self.manager = host.KvCacheManager(
            [host.GroupSpec(g.block_size, g.num_blocks, g.window) for g in self.groups], num_state_slots,
            # state of fixed size is not snapshotted at page boundaries: with such a layer nothing is skipped on a hit
            prefix_caching and not any(s is not None for s in state_specs))

    def bytes(self) -> int:
        total = sum(2 * p.k.numel() * p.k.element_size() for p in self.planes if p is not None)
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
