"""The step function: one batch of (request, its next tokens) through the model, from the cache.

`EngineCore.run(entries)` takes portions of prompts beside single decoded tokens, cut anywhere,
runs exactly the tokens it is given as ONE batch and returns float32 logits at the wanted places.
The reference's step (vllm-oxide, crates/vllm-oxide/src/engine/mod.rs:83-151) runs either prompt
portions or decode tokens, with two builders (:156-227, :232-278); here there is one builder and
one path, and prefill reads earlier portions from the pages.

All integer arrays of a step are built on the host by the C++ batch builder in one pinned
buffer and reach the device in one copy.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import host, kernels
from ..cache.paged_cache import PagedCache
from ..parts.base import Workspace


class StepContext:
    """What the parts see of a step: device arrays of the batch, the workspace, the error word."""

    def __init__(self, layout, dev: torch.Tensor, host_array: np.ndarray, counts, ws: Workspace, err: torch.Tensor,
                 launch_tokens: Optional[int] = None, launch_rows: Optional[int] = None):
        L = layout
        self.layout, self.counts, self.ws, self.err = L, counts, ws, err
        self.host = host_array
        self.num_tokens, self.num_requests, self.num_rows = counts.num_tokens, counts.num_requests, counts.num_rows
        self.num_decode, self.max_q, self.max_context = counts.num_decode, counts.max_q, counts.max_context
        self.launch_tokens = self.num_tokens if launch_tokens is None else launch_tokens
        self.launch_rows = self.num_rows if launch_rows is None else launch_rows
        self.launch_requests = L.B
        self.token_ids = dev[L.token_ids:L.token_ids + L.T]
        self.positions = dev[L.positions:L.positions + L.T]
        self.token_req = dev[L.token_req:L.token_req + L.T]
        self.slot_mapping = [dev[L.slot_mapping + g * L.T:L.slot_mapping + (g + 1) * L.T] for g in range(L.G)]
        self.cu_q = dev[L.cu_q:L.cu_q + L.B + 1]
        self.context_lens = dev[L.context_lens:L.context_lens + L.B]
        self.state_slots = dev[L.state_slots:L.state_slots + L.B]
        self.state_fresh = dev[L.state_fresh:L.state_fresh + L.B]
        self.logit_rows = dev[L.logit_rows:L.logit_rows + L.R]
        self.block_tables = [dev[L.block_tables + g * L.B * L.P:L.block_tables + (g + 1) * L.B * L.P].view(L.B, L.P)
                             for g in range(L.G)]

    def host_view(self, name: str) -> np.ndarray:
        """The host copy of one array (for parts that loop over requests on the host, and for tests)."""
        L = self.layout
        sizes = dict(token_ids=L.T, positions=L.T, token_req=L.T, cu_q=L.B + 1, context_lens=L.B, state_slots=L.B,
                     state_fresh=L.B, logit_rows=L.R)
        off = getattr(L, name)
        return self.host[off:off + sizes[name]]


class EngineCore:
    def __init__(self, model, cache: PagedCache, max_num_batched_tokens: int, max_num_seqs: int, max_model_len: int):
        self.model, self.cache = model, cache
        self.device = model.device
        self.manager = cache.manager
        self.max_tokens, self.max_seqs, self.max_model_len = max_num_batched_tokens, max_num_seqs, max_model_len
        self.num_groups = len(cache.groups)
        self.max_pages = (max_model_len + cache.block_size - 1) // cache.block_size
        cap = host.BatchLayout(self.max_tokens, self.max_seqs, self.max_tokens, self.num_groups, self.max_pages).total
        self._host_buf = torch.empty(cap, dtype=torch.int32, pin_memory=torch.device(self.device).type == "cuda")
        self._host_np = self._host_buf.numpy()
        self._dev_buf = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ws = Workspace(min(self.max_tokens, 8192), self.device, model.dtype)
        model.bind(cache.planes, cache.states)
        self._copied = torch.cuda.Event() if torch.device(self.device).type == "cuda" else None
        self.h2d_bytes_last = 0

    # ---- building a step
    def build_context(self, entries: Sequence["host.BatchEntry"]) -> StepContext:
        n_tok = sum(len(e.tokens) for e in entries)
        n_rows = sum(len(e.want) for e in entries)
        if n_tok > self.max_tokens:
            raise ValueError(f"a step of {n_tok} tokens exceeds max_num_batched_tokens {self.max_tokens}")
        if len(entries) > self.max_seqs:
            raise ValueError(f"a step of {len(entries)} requests exceeds max_num_seqs {self.max_seqs}")
        pages = max((len(self.manager.block_table(e.id, g)) for e in entries for g in range(self.num_groups)), default=1)
        layout = host.BatchLayout(max(n_tok, 1), max(len(entries), 1), max(n_rows, 1), self.num_groups, max(pages, 1))
        if self._copied is not None:
            self._copied.synchronize()   # the previous step's copy has left the pinned buffer
        counts = host.fill_step_batch(self.manager, list(entries), layout, self._host_np)
        fresh = [int(s) for s, f in zip(self._host_np[layout.state_slots:layout.state_slots + counts.num_requests],
                                        self._host_np[layout.state_fresh:layout.state_fresh + counts.num_requests]) if f]
        self.cache.zero_states(fresh)
        self._dev_buf[:layout.total].copy_(self._host_buf[:layout.total], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        self.h2d_bytes_last = layout.total * 4
        return StepContext(layout, self._dev_buf, self._host_np, counts, self.ws, self.err)

    # ---- one step
    def run(self, entries: Sequence["host.BatchEntry"]) -> torch.Tensor:
        """Float32 logits [wanted rows, vocab] in the order of the entries and of their `want`."""
        if not entries:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        ctx = self.build_context(entries)
        hidden, residual = self.model.forward(ctx)
        if ctx.num_rows == 0:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.compute_logits(hidden, residual, ctx)

    def check_errors(self) -> None:
        """Raises if a kernel met a bad index since the last check (synchronises)."""
        word = int(self.err.item())
        if word:
            self.err.zero_()
            raise kernels.KernelError("a kernel refused an access: " + kernels.describe_error_word(word))
