"""The host runtime (C++): block pool, cache manager, scheduler, batch builder.

Built in-tree at first import; the names are re-exported from the compiled module `_host`.
"""
from __future__ import annotations

import importlib

from .csrc import build as _build

_build.build_host()
_mod = importlib.import_module(__package__ + "._host")

BlockPool = _mod.BlockPool
GroupSpec = _mod.GroupSpec
KvCacheManager = _mod.KvCacheManager
Scheduler = _mod.Scheduler
SchedSamplingParams = _mod.SchedSamplingParams
BatchLayout = _mod.BatchLayout
BatchEntry = _mod.BatchEntry
PoolError = _mod.PoolError
fill_step_batch = _mod.fill_step_batch
chain_hash = _mod.chain_hash
xxh64 = _mod.xxh64
