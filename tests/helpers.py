"""Test helpers: a step context built by hand, so that one part can be run alone."""
import numpy as np
import torch

from vllm_oxide_b200 import host
from vllm_oxide_b200.engine.core import StepContext
from vllm_oxide_b200.parts import Workspace


def make_context(manager, entries, dtype, device="cuda:0"):
    """entries: [(request id, start, tokens, want)]; pages must have been ensured."""
    be = [host.BatchEntry(rid, start, list(toks), list(want)) for rid, start, toks, want in entries]
    T = sum(len(e.tokens) for e in be)
    R = max(1, sum(len(e.want) for e in be))
    pages = max(len(manager.block_table(e.id, g)) for e in be for g in range(manager.num_groups))
    layout = host.BatchLayout(T, len(be), R, manager.num_groups, max(pages, 1))
    buf = np.zeros(layout.total, dtype=np.int32)
    counts = host.fill_step_batch(manager, be, layout, buf)
    dev = torch.from_numpy(buf).to(device)
    err = torch.zeros(1, dtype=torch.int32, device=device)
    return StepContext(layout, dev, buf, counts, Workspace(T, device, dtype), err)
