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
        self.next_norm = None      # hints between blocks within a step (models/causal_lm.py sets them, parts/block.py reads them)
        self.prenormed = None
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


GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)


class _DecodeGraph:
    """One captured decode step for a padded batch size: its layout, buffers, graph and logits."""

    def __init__(self, layout, ws, dev):
        self.layout, self.ws, self.dev = layout, ws, dev
        self.graph = None
        self.logits = None
        self.host_view = self.dev_view = None     # the step's arrays in the pinned buffer and on the device
        self.launches = 0     # this package's kernel launches inside the graph


class EngineCore:
    def __init__(self, model, cache: PagedCache, max_num_batched_tokens: int, max_num_seqs: int, max_model_len: int,
                 use_graphs: bool = True):
        self.model, self.cache = model, cache
        self.device = model.device
        self.manager = cache.manager
        self.max_tokens, self.max_seqs, self.max_model_len = max_num_batched_tokens, max_num_seqs, max_model_len
        self.num_groups = len(cache.groups)
        # width of the block tables: the pages of a request of max_model_len in the group with the smallest pages
        self.max_pages = max((max_model_len + g.block_size - 1) // g.block_size for g in cache.groups)
        cap = host.BatchLayout(self.max_tokens, self.max_seqs, self.max_tokens, self.num_groups, self.max_pages).total
        # a decode step replayed from a graph is padded to the next batch size that has one, which may be more
        # requests (and tokens) than a step may hold: the staging buffers take that layout too
        padded = next((b for b in GRAPH_BUCKETS if b >= self.max_seqs), GRAPH_BUCKETS[-1])
        cap = max(cap, host.BatchLayout(padded, padded, padded, self.num_groups, self.max_pages).total)
        self._host_buf = torch.empty(cap, dtype=torch.int32, pin_memory=torch.device(self.device).type == "cuda")
        self._host_np = self._host_buf.numpy()
        self._dev_buf = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        # activation buffers for the largest step the scheduler may form, so that no step re-allocates them
        self.ws = Workspace(max(1, min(self.max_tokens, self.max_seqs * self.max_model_len)), self.device, model.dtype)
        model.bind(cache.planes, cache.states)
        self._copied = torch.cuda.Event() if torch.device(self.device).type == "cuda" else None
        self.h2d_bytes_last = 0
        # Steps in which every request brings one token are replayed from CUDA graphs, one per padded
        # batch size, when every part of the model launches the same kernels whatever the batch holds.
        self.use_graphs = bool(use_graphs and getattr(model, "graph_safe", False))
        self._graphs = {}
        self.graph_replays = 0

    # ---- building a step
    def build_context(self, entries: Sequence["host.BatchEntry"]) -> StepContext:
        n_tok = sum(len(e.tokens) for e in entries)
        n_rows = sum(len(e.want) for e in entries)
        pages = max((len(self.manager.block_table(e.id, g)) for e in entries for g in range(self.num_groups)), default=1)
        entries = list(entries)
        return self._build_context(len(entries), n_tok, n_rows, pages,
                                   lambda layout: host.fill_step_batch(self.manager, entries, layout, self._host_np))

    def _build_context(self, n_req: int, n_tok: int, n_rows: int, pages: int, fill) -> StepContext:
        """`fill(layout)` writes the step's arrays into the pinned buffer and returns its counts."""
        if n_tok > self.max_tokens:
            raise ValueError(f"a step of {n_tok} tokens exceeds max_num_batched_tokens {self.max_tokens}")
        if n_req > self.max_seqs:
            raise ValueError(f"a step of {n_req} requests exceeds max_num_seqs {self.max_seqs}")
        layout = host.BatchLayout(max(n_tok, 1), max(n_req, 1), max(n_rows, 1), self.num_groups, max(pages, 1))
        if self._copied is not None:
            self._copied.synchronize()   # the previous step's copy has left the pinned buffer
        counts = fill(layout)
        fresh = [int(s) for s, f in zip(self._host_np[layout.state_slots:layout.state_slots + counts.num_requests],
                                        self._host_np[layout.state_fresh:layout.state_fresh + counts.num_requests]) if f]
        self.cache.zero_states(fresh)
        self._dev_buf[:layout.total].copy_(self._host_buf[:layout.total], non_blocking=True)
        if self._copied is not None:
            self._copied.record()
        self.h2d_bytes_last = layout.total * 4
        return StepContext(layout, self._dev_buf, self._host_np, counts, self.ws, self.err)

    # ---- decode steps from CUDA graphs
    def _graph_bucket(self, entries) -> Optional[int]:
        if not self.use_graphs or any(len(e.tokens) != 1 for e in entries):
            return None
        return self._bucket_for(len(entries))

    def _bucket_for(self, num_requests: int) -> Optional[int]:
        for b in GRAPH_BUCKETS:
            if b >= num_requests:
                return b if b <= max(self.max_seqs, 1) * 2 else None
        return None

    def _fill_fixed(self, g: _DecodeGraph, fill) -> "host.BatchCounts":
        if self._copied is not None:
            self._copied.synchronize()
        counts = fill(g.layout)
        L = g.layout
        if self.cache.has_states:
            fresh = [int(s) for s, f in zip(self._host_np[L.state_slots:L.state_slots + counts.num_requests],
                                            self._host_np[L.state_fresh:L.state_fresh + counts.num_requests]) if f]
            self.cache.zero_states(fresh)
        if g.host_view is None:
            g.host_view, g.dev_view = self._host_buf[:L.total], g.dev[:L.total]
        g.dev_view.copy_(g.host_view, non_blocking=True)
        self.h2d_bytes_last = L.total * 4
        return counts

    def _graph_context(self, g: _DecodeGraph, counts) -> StepContext:
        ctx = StepContext(g.layout, g.dev, self._host_np, counts, g.ws, self.err,
                          launch_tokens=g.layout.T, launch_rows=g.layout.R)
        # what the host knows of a decode step must not depend on the step, or the capture would bake it in
        ctx.num_decode = ctx.num_requests = g.layout.B
        ctx.max_q, ctx.max_context = 1, self.max_model_len
        return ctx

    def _run_graph(self, bucket: int, fill) -> torch.Tensor:
        g = self._graphs.get(bucket)
        if g is None:
            layout = host.BatchLayout(bucket, bucket, bucket, self.num_groups, self.max_pages)
            g = _DecodeGraph(layout, Workspace(bucket, self.device, self.model.dtype),
                             torch.empty(layout.total, dtype=torch.int32, device=self.device))
            counts = self._fill_fixed(g, fill)
            ctx = self._graph_context(g, counts)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):          # once outside capture: buffers, library handles, attributes
                hidden, residual = self.model.forward(ctx)
                self.model.compute_logits(hidden, residual, ctx)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g.graph = torch.cuda.CUDAGraph()
            before = kernels.launch_count
            with torch.cuda.graph(g.graph):
                hidden, residual = self.model.forward(ctx)
                g.logits = self.model.compute_logits(hidden, residual, ctx)
            g.launches = kernels.launch_count - before
            self._graphs[bucket] = g
        else:
            counts = self._fill_fixed(g, fill)
        g.graph.replay()
        if self._copied is not None:
            self._copied.record()     # after the launch: it guards the pinned buffer, and recording it is not free
        kernels.launch_count += g.launches
        self.graph_replays += 1
        return g.logits[:counts.num_rows]

    # ---- one step
    def run(self, entries: Sequence["host.BatchEntry"]) -> torch.Tensor:
        """Float32 logits [wanted rows, vocab] in the order of the entries and of their `want`."""
        if not entries:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        bucket = self._graph_bucket(entries)
        if bucket is not None:
            entries = entries if isinstance(entries, list) else list(entries)
            return self._run_graph(bucket, lambda layout: host.fill_step_batch(self.manager, entries, layout, self._host_np))
        return self._forward(self.build_context(entries))

    def run_scheduled(self, scheduler: "host.Scheduler") -> torch.Tensor:
        """The step that `scheduler.schedule()` has just decided, without building entries on the way: the scheduler
        writes the step's arrays from its sequences straight into the pinned buffer.  Same logits as
        `run(scheduler.batch_entries())`."""
        s = scheduler.summary()
        if s.num_requests == 0:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        fill = lambda layout: scheduler.fill_batch(layout, self._host_np)
        bucket = self._bucket_for(s.num_requests) if self.use_graphs and s.all_single else None
        if bucket is not None:
            return self._run_graph(bucket, fill)
        return self._forward(self._build_context(s.num_requests, s.num_tokens, s.num_rows, s.max_pages, fill))

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        hidden, residual = self.model.forward(ctx)
        if ctx.num_rows == 0:
            return torch.empty((0, self.model.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.compute_logits(hidden, residual, ctx)

    def check_errors(self) -> None:
        """Raises if a kernel met a bad index since the last check (synchronises)."""
        self.raise_for(int(self.err.item()))

    def raise_for(self, word: int) -> None:
        """Raises for a non-zero value of the error word (read by the caller, e.g. together with the sampled tokens)."""
        if word:
            self.err.zero_()
            raise kernels.KernelError("a kernel refused an access: " + kernels.describe_error_word(word))
