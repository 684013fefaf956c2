"""The sampler: float32 logits on the device in, one token per row out.

The pipeline and its order are the reference's (vllm-oxide, crates/vllm-oxide/src/sampler.rs:207-261):
penalties, greedy short-circuit, temperature, top-k, top-p, Gumbel-max.  It runs in one kernel
per step over all rows; the uniform numbers of a row come from a counter-based generator keyed
by (seed, request, index of the token in the request's output), so a request samples the same
tokens alone, in any batch, after any cut of its prompt and after preemption.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels

_M = (1 << 64) - 1


def row_key(seed: int, request: int, index: int) -> int:
    """64-bit key of one sampled token (splitmix64 finaliser over the three numbers)."""
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + index * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


class Sampler:
    def __init__(self, device, max_rows: int = 512):
        self.device = device
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self._cap:
            return
        rows = (rows + 1) // 2 * 2          # the 64-bit keys start on an 8-byte boundary of the staging block
        self._cap = rows
        pin = torch.device(self.device).type == "cuda"
        # one pinned staging block: temperature f32 | top_p f32 | top_k i32 | keys u64 (as 2 x i32)
        self._host = torch.empty(5 * rows, dtype=torch.int32, pin_memory=pin)
        self._dev = torch.empty(5 * rows, dtype=torch.int32, device=self.device)
        self._out = torch.empty(rows, dtype=torch.int32, device=self.device)
        h, n = self._host.numpy(), rows
        # the four arrays of the staging block, for callers that fill them in place (the scheduler does, in C++)
        self.host_temperature, self.host_top_p = h[0:n].view(np.float32), h[n:2 * n].view(np.float32)
        self.host_top_k, self.host_keys = h[2 * n:3 * n], h[3 * n:5 * n].view(np.uint64)

    def reserve(self, rows: int) -> None:
        """Makes room for `rows` rows (the staging arrays are replaced when it has to grow)."""
        self._grow(rows)

    def forward_staged(self, logits: torch.Tensor, rows: int) -> torch.Tensor:
        """As forward(), with the settings of the first `rows` rows already written to the host_* arrays."""
        n = self._cap
        self._dev.copy_(self._host, non_blocking=True)
        d = self._dev
        kernels.sample(logits, d[0:n].view(torch.float32), d[2 * n:3 * n], d[n:2 * n].view(torch.float32),
                       d[3 * n:5 * n], self._out, rows)
        return self._out[:rows]

    def forward(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
                top_p: Sequence[float], keys: Sequence[int]) -> torch.Tensor:
        """Token ids [R] (int32, on the device).  top_k 0 and top_p >= 1 mean off."""
        R = logits.shape[0]
        self._grow(R)
        n = self._cap
        h = self._host.numpy()
        h[0:R].view(np.float32)[:] = np.asarray(temperature, dtype=np.float32)
        h[n:n + R].view(np.float32)[:] = np.asarray(top_p, dtype=np.float32)
        h[2 * n:2 * n + R] = np.asarray(top_k, dtype=np.int32)
        h[3 * n:3 * n + 2 * R].view(np.uint64)[:] = np.asarray(keys, dtype=np.uint64)
        self._dev.copy_(self._host, non_blocking=True)
        d = self._dev
        kernels.sample(logits, d[0:n].view(torch.float32), d[2 * n:3 * n], d[n:2 * n].view(torch.float32),
                       d[3 * n:5 * n], self._out, R)
        return self._out[:R]

    def apply_penalties(self, logits: torch.Tensor, histories: List[Optional[Sequence[int]]], presence: Sequence[float],
                        frequency: Sequence[float], repetition: Sequence[float]) -> None:
        """In place, once per distinct token of a row's history (sampler.rs:320-345)."""
        rows, toks, counts = [], [], []
        for r, hist in enumerate(histories):
            if hist is None:
                continue
            for tok, c in Counter(hist).items():
                rows.append(r)
                toks.append(tok)
                counts.append(c)
        if not rows:
            return
        dev = self.device
        f = lambda x, dt: torch.as_tensor(np.asarray(x), dtype=dt).to(dev)
        kernels.apply_penalties(logits, f(rows, torch.int32), f(toks, torch.int32), f(counts, torch.int32),
                                f(presence, torch.float32), f(frequency, torch.float32), f(repetition, torch.float32),
                                len(rows))
