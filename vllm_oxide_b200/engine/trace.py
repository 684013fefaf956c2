"""Trace replay: given token ids through the engine's own step function, logits to disk.

It samples nothing and owns no forward pass, cache or loader: requests are registered with the
cache manager, pages are ensured for each portion, the portion runs through `EngineCore.run`
(the function generation uses), pages that a window has passed are given back, and a finished
request frees what it holds.  Its ancestor in the reference is `LLM::generate_logits`
(vllm-oxide, crates/vllm-oxide/src/llm.rs:279-313).

With `prefix_caching` the runner does what the scheduler does with the prefix cache (the reference's
`can_allocate` / `allocate` / `hash_blocks`, crates/vllm-oxide/src/engine/block_pool.rs:198-285,337-358):
when a request first appears, the full pages at the start of its first entry that an earlier request has
computed (live or ended, as long as the pages have not been handed out again) are taken into its block table
and their tokens are not run; after every step the pages that became full are published.  Only pages before
the entry's first wanted place are taken, so every wanted row is still computed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, List

import numpy as np
import torch

from .. import host
from ..cache.paged_cache import PagedCache
from .core import EngineCore
from .loading import load_model, resolve_dtype


class TraceRunner:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, block_size: int = 64, device: str = "cuda:0",
                 max_live: int = 64, prefix_caching: bool = False, _model=None):
        if not torch.cuda.is_available():
            raise RuntimeError("trace replay needs a CUDA device: the engine has no CPU path")
        self.dtype = resolve_dtype(dtype)
        # `_model`: a (config, model) pair that is already on the device (tests at the layer sizes of large models,
        # which write no folder); otherwise the folder is loaded like everywhere in the engine
        self.cfg, self.model = _model if _model is not None else load_model(model_dir, self.dtype, device)
        if self.model.dtype != self.dtype:
            raise ValueError(f"the model is in {self.model.dtype}, the replay was asked for {self.dtype}")
        pool_tokens = (max(max_tokens, 1) + block_size - 1) // block_size * block_size
        self.cache = PagedCache(self.model.cache_specs(), self.model.state_specs(), self.dtype, device, block_size,
                                pool_tokens // block_size, num_state_slots=max_live, prefix_caching=prefix_caching)
        self.core = EngineCore(self.model, self.cache, max_num_batched_tokens=pool_tokens, max_num_seqs=max_live,
                               max_model_len=min(pool_tokens, self.model.plan.max_position))
        self.manager = self.cache.manager
        self._ids: Dict[str, int] = {}
        self._pos: Dict[str, int] = {}
        self._tokens: Dict[str, List[int]] = {}
        self._next = 0
        self.prefix_hit_tokens = 0      # tokens that were taken from pages of earlier requests instead of being run

    def step(self, entries: List[dict], end: List[str]) -> np.ndarray:
        """Runs one step; returns float32 logits [wanted, vocab] (possibly zero rows)."""
        batch = []
        for e in entries:
            name, tokens, want = str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]
            if not tokens:
                raise ValueError(f"request {name}: an entry without tokens")
            if name not in self._ids:
                self._ids[name], self._pos[name] = self._next, 0
                self._next += 1
                if not self.manager.add_request(self._ids[name]):
                    raise RuntimeError(f"request {name}: more live requests than the runner was made for")
                self._tokens[name] = []
                if self.manager.prefix_caching:
                    # the page that holds the last token given to lookup_prefix is never taken: pass the tokens up to
                    # the first wanted place, so that place (and the entry's last token) is computed in any case
                    upto = min(min(want) + 1, len(tokens)) if want else len(tokens)
                    hit = self.manager.lookup_prefix(self._ids[name], tokens[:upto])
                    self._pos[name] = hit
                    self._tokens[name] = tokens[:hit]
                    self.prefix_hit_tokens += hit
                    tokens, want = tokens[hit:], [w - hit for w in want]
            rid, pos = self._ids[name], self._pos[name]
            if pos + len(tokens) > self.model.plan.max_position:
                raise ValueError(f"request {name}: position {pos + len(tokens)} exceeds max_position_embeddings")
            if not self.manager.ensure(rid, pos, len(tokens)):
                raise RuntimeError(f"request {name}: the cache pool (--max-tokens) has no pages left for "
                                   f"{len(tokens)} more tokens at position {pos}")
            batch.append(host.BatchEntry(rid, pos, tokens, want))
            self._tokens[name].extend(tokens)
        logits = self.core.run(batch)
        out = logits.cpu().numpy() if logits.shape[0] else np.zeros((0, self.model.vocab_size), np.float32)
        self.core.check_errors()
        for e in entries:
            name = str(e["id"])
            self._pos[name] = len(self._tokens[name])
            self.manager.commit(self._ids[name], self._tokens[name], self._pos[name])
            self.manager.advance(self._ids[name], self._pos[name])
        for name in end:
            name = str(name)
            if name in self._ids:
                self.manager.free_request(self._ids.pop(name))
                self._pos.pop(name)
                self._tokens.pop(name)
        return out


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="feed token ids through the engine step by step "
                                 "and write the logits at the wanted places")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool is made for")
    ap.add_argument("--block-size", type=int, default=64, help="tokens per cache page (default 64)")
    ap.add_argument("--prefix-caching", action="store_true",
                    help="a request's first entry starts on the full pages that an earlier request computed for the same tokens")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    runner = TraceRunner(args.model, args.dtype, args.max_tokens, args.block_size, prefix_caching=args.prefix_caching)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        logits = runner.step(rec.get("entries", []), rec.get("end", []))
        if logits.shape[0]:
            logits.astype("<f4").tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        print(f"done {rec['step']}", flush=True)
    return 0
