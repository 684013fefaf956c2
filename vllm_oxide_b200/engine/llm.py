"""The Python entry point, in the manner of the reference's `LLM::new` / `LLM::generate`
(vllm-oxide, crates/vllm-oxide/src/llm.rs:82-178,188-268,279-313).

    llm = LLM("/path/to/model", EngineOptions(max_model_len=4096))
    outs = llm.generate([[1, 2, 3], "some text"], [SamplingParams(), SamplingParams(temperature=0.8)])

Prompts are token id lists or text (text needs tokenizer.json in the model folder); one
`SamplingParams` per prompt; outputs come back in prompt order.  Unlike the reference, whose
outputs are indexed by a counter that never resets (llm.rs:221-231), results are mapped by
request, so `generate` can be called again and again.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from .. import host
from ..cache.paged_cache import PagedCache
from ..config.engine_options import EngineOptions
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .core import EngineCore
from .loading import load_model, random_model, resolve_dtype

Prompt = Union[str, Sequence[int]]


@dataclass
class RequestOutput:
    seq_id: int
    token_ids: List[int]
    text: str = ""
    finished: bool = True
    finish_reason: str = ""


@dataclass
class GenerateStats:
    total_tokens: int = 0
    elapsed_s: float = 0.0
    steps: int = 0
    preemptions: int = 0
    prefix_hit_tokens: int = 0

    @property
    def tok_per_sec(self) -> float:
        return self.total_tokens / self.elapsed_s if self.elapsed_s > 0 else 0.0


class LLM:
    def __init__(self, source: str, options: Optional[EngineOptions] = None, *, device: str = "cuda:0",
                 _model=None):
        if not torch.cuda.is_available():
            raise RuntimeError("vllm_oxide_b200 runs on a CUDA device (sm_100a); none is visible and there is no CPU path")
        self.options = options or EngineOptions()
        self.options.validate()
        self.device = device
        self.dtype = resolve_dtype(self.options.dtype)
        if _model is not None:
            self.config, self.model = _model
        else:
            if not os.path.isdir(source):
                raise FileNotFoundError(f"model folder {source!r} does not exist (only local folders are supported)")
            self.config, self.model = load_model(source, self.dtype, device)
        self.source = source
        plan = self.model.plan
        if self.options.max_model_len > plan.max_position:   # llm.rs:97-105
            raise ValueError(f"max_model_len {self.options.max_model_len} exceeds the model's "
                             f"max_position_embeddings {plan.max_position}")
        o = self.options
        self.cache = self._make_cache()
        self.core = EngineCore(self.model, self.cache, o.max_num_batched_tokens, o.max_num_seqs, o.max_model_len,
                               use_graphs=not o.enforce_eager)
        eos = plan.eos_token_id if plan.eos_token_id is not None else -1
        self.scheduler = host.Scheduler(self.cache.manager, o.max_num_batched_tokens, o.max_num_seqs, o.max_model_len, eos)
        self.sampler = Sampler(device, min(o.max_num_seqs, 512))
        self.tokenizer = self._load_tokenizer(source) if isinstance(source, str) else None
        self.last_stats = GenerateStats()
        self.last_sampled_ids: List[int] = []

    @classmethod
    def from_config(cls, config_dict: dict, options: Optional[EngineOptions] = None, *, seed: int = 0,
                    init_scheme: str = "fan_in", device: str = "cuda:0", draw_on: Optional[str] = None) -> "LLM":
        """An engine over seeded random weights (no files): drawn on the device, or with `draw_on="cpu"` by the host's
        generator, which gives the values a written random model folder holds for the same seed."""
        options = options or EngineOptions()
        model = random_model(config_dict, seed, resolve_dtype(options.dtype), device, init_scheme, draw_on)
        return cls("<random weights>", options, device=device, _model=model)

    # ---- construction helpers
    def _make_cache(self) -> PagedCache:
        o = self.options
        specs, states = self.model.cache_specs(), self.model.state_specs()
        reserve = 0
        if o.num_kv_blocks is None:
            reserve = self._activation_reserve()
        return PagedCache(specs, states, self.dtype, self.device, o.block_size, o.num_kv_blocks, o.max_num_seqs,
                          o.gpu_memory_utilization, o.enable_prefix_caching, reserve)

    def _activation_reserve(self) -> int:
        """Bytes to leave for the activations of the largest step: measured by running one such step
        over a throw-away cache (the reference sizes its pool without running anything, llm.rs:485-537)."""
        o = self.options
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        n_tok = max(1, min(o.max_num_batched_tokens, o.max_num_seqs * o.max_model_len))   # the largest step there can be
        per_req = min(o.max_model_len, n_tok)
        n_req = max(1, min(n_tok // per_req, o.max_num_seqs))
        pages = n_req * ((per_req + o.block_size - 1) // o.block_size)
        cache = PagedCache(self.model.cache_specs(), self.model.state_specs(), self.dtype, self.device, o.block_size,
                           pages, max(n_req, 1), prefix_caching=False)
        core = EngineCore(self.model, cache, n_req * per_req, max(n_req, 1), o.max_model_len, use_graphs=False)
        entries = []
        for r in range(n_req):
            cache.manager.add_request(r)
            cache.manager.ensure(r, 0, per_req)
            entries.append(host.BatchEntry(r, 0, [0] * per_req, [per_req - 1]))
        core.run(entries)
        torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated(self.device)
        del core, cache
        torch.cuda.empty_cache()
        logits_rows = o.max_num_seqs * self.model.vocab_size * 8
        return max(0, peak - before) + logits_rows + (256 << 20)

    @staticmethod
    def _load_tokenizer(source: str):
        path = os.path.join(source, "tokenizer.json")
        if not os.path.isfile(path):
            return None
        try:
            from tokenizers import Tokenizer
        except ImportError:
            return None
        return Tokenizer.from_file(path)

    def _tokenize(self, prompt: Prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs tokenizer.json in the model folder (and the `tokenizers` "
                                 "package); pass token ids instead")
            return list(self.tokenizer.encode(prompt).ids)
        ids = [int(t) for t in prompt]
        V = self.model.vocab_size
        bad = [t for t in ids if t < 0 or t >= V]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary of {V}")
        return ids

    # ---- requests
    def add_request(self, token_ids: Sequence[int], params: SamplingParams) -> int:
        params.validate()
        p = host.SchedSamplingParams()
        p.temperature = float(params.temperature)
        p.top_k = int(params.top_k or 0)
        p.top_p = float(params.top_p if params.top_p is not None else 1.0)
        p.max_tokens = int(params.max_tokens)
        p.ignore_eos = bool(params.ignore_eos)
        p.presence_penalty = float(params.presence_penalty)
        p.frequency_penalty = float(params.frequency_penalty)
        p.repetition_penalty = float(params.repetition_penalty)
        p.seed = int(params.seed if params.seed is not None else self.options.seed) & ((1 << 64) - 1)
        p.own_seed = params.seed is not None
        return self.scheduler.add_request([int(t) for t in token_ids], p)

    def is_running(self) -> bool:
        return self.scheduler.has_unfinished()

    def step(self, want_logits: bool = False):
        """One engine step: schedule, run, sample, book.  Returns the finished requests' outputs
        (and, with `want_logits`, the float32 logits of the rows that were sampled from)."""
        sched, sampler = self.scheduler, self.sampler
        if not sched.schedule_step():
            if sched.has_unfinished():
                raise RuntimeError("the scheduler produced an empty step while requests are unfinished")
            return ([], None) if want_logits else []
        logits = self.core.run_scheduled(sched)        # the step's arrays go from the sequences into the pinned buffer
        sampler.reserve(logits.shape[0])
        rows, penalties = sched.fill_sampling(sampler.host_temperature, sampler.host_top_p, sampler.host_top_k,
                                              sampler.host_keys)
        sampled: List[int] = []
        if rows:
            if penalties or want_logits:
                reqs = sched.sample_requests()
                self.last_sampled_ids = [r[0] for r in reqs]     # the requests of the logits' rows, in row order
                if penalties:
                    self._penalties(logits, reqs)
            sampled = self._read_back(sampler.forward_staged(logits, rows))
        else:
            self.last_sampled_ids = []
            self.core.check_errors()
        outs = [RequestOutput(o.id, list(o.token_ids), "", o.finished, o.finish_reason)
                for o in sched.postprocess(sampled)]
        if want_logits:
            return outs, (logits.float().cpu().numpy().copy() if rows else None)
        return outs

    def _read_back(self, toks: torch.Tensor) -> List[int]:
        """The sampled tokens and the kernels' error word in one wait: two copies into one pinned buffer."""
        n = toks.shape[0]
        buf = getattr(self, "_readback", None)
        if buf is None or buf.numel() < n + 1:
            buf = self._readback = torch.empty(max(n + 1, 1025), dtype=torch.int32,
                                               pin_memory=torch.device(self.core.device).type == "cuda")
        buf[:n].copy_(toks, non_blocking=True)
        buf[n:n + 1].copy_(self.core.err, non_blocking=True)
        if torch.device(self.core.device).type == "cuda":
            torch.cuda.current_stream(torch.cuda.current_device()).synchronize()
        vals = buf[:n + 1].tolist()
        self.core.raise_for(vals[n])
        return vals[:n]

    def _penalties(self, logits, reqs) -> None:
        hist, pres, freq, rep = [], [], [], []
        for r in reqs:
            seq = self.scheduler.sequence(r[0])
            hist.append(list(seq.tokens) if r[6] else None)
            pres.append(seq.params.presence_penalty)
            freq.append(seq.params.frequency_penalty)
            rep.append(seq.params.repetition_penalty)
        self.sampler.apply_penalties(logits, hist, pres, freq, rep)

    # ---- the public calls
    def generate(self, prompts: Sequence[Prompt], sampling_params: Union[SamplingParams, Sequence[SamplingParams]]
                 ) -> List[RequestOutput]:
        if len(prompts) == 0:
            return []
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):   # llm.rs:196-202
            raise ValueError(f"generate: expected {len(prompts)} sampling_params, got {len(sampling_params)}")
        token_lists = [self._tokenize(p) for p in prompts]
        ids = [self.add_request(t, sp) for t, sp in zip(token_lists, sampling_params)]
        index = {rid: i for i, rid in enumerate(ids)}
        results: List[Optional[RequestOutput]] = [None] * len(prompts)
        t0 = time.perf_counter()
        steps = 0
        s0 = self.scheduler.stats
        pre0, hit0 = s0.preemptions, s0.prefix_hit_tokens
        while self.scheduler.has_unfinished():
            for out in self.step():
                i = index.get(out.seq_id)
                if i is None:
                    continue
                if self.tokenizer is not None:
                    out.text = self.tokenizer.decode(out.token_ids, skip_special_tokens=True)
                out.seq_id = i
                results[i] = out
            steps += 1
        s1 = self.scheduler.stats
        total = sum(len(t) for t in token_lists) + sum(len(r.token_ids) for r in results if r)
        self.last_stats = GenerateStats(total, time.perf_counter() - t0, steps, s1.preemptions - pre0,
                                        s1.prefix_hit_tokens - hit0)
        return [r if r is not None else RequestOutput(i, [], "", False) for i, r in enumerate(results)]

    def generate_logits(self, prompt: Prompt, max_tokens: int) -> np.ndarray:
        """Greedy generation of one prompt; float32 logits [steps, vocab] before every sampled token."""
        self.add_request(self._tokenize(prompt), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
        rows = []
        while self.scheduler.has_unfinished():
            _, logits = self.step(want_logits=True)
            if logits is not None:
                rows.append(logits)
        return np.concatenate(rows, 0) if rows else np.zeros((0, self.model.vocab_size), np.float32)
