"""The host runtime (C++): block pool, cache manager, scheduler, batch builder.

Built in-tree at first import; the names are re-exported from the compiled module `_host`.
"""
from __future__ import annotations

import importlib
import importlib.util
import sys

from .csrc import build as _build

_path = _build.build_host()
if _build.host_sanitized():
    # the sanitizer build lives in a folder of its own: load it under the module's usual name
    _spec = importlib.util.spec_from_file_location(__package__ + "._host", _path)
    _mod = importlib.util.module_from_spec(_spec)
    sys.modules[__package__ + "._host"] = _mod
    _spec.loader.exec_module(_mod)
else:
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
