"""Decode and prefill throughput of the engine at Qwen3-8B sizes (bf16, random weights, one B200).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The default run has the layer sizes of the 8B configuration, a batch
of 8 requests whose context starts at 2,048 tokens, and prints ONE JSON line:
  value     decoded tokens per second, timed on the device with CUDA events around K steps;
  e2e       the same through the Python entry point (LLM.add_request / LLM.step): pinned host
            buffers in, sampled tokens out, every step;
  prefill   one 2,048-token prompt in one step; frac = flops / time / peak;
  roofline  the decode step's bytes (every weight once + the cache of the live requests) / time
            against the measured copy bandwidth;
  points    decode at batch 1, 16, 32 and 64 with their fractions of the copy bandwidth; the end-to-end rate at batch 1
            and 64 and the host's time per step (end-to-end minus device) at batch 1, 8 and 64; decode at contexts of
            8,192 and 32,768 tokens (batch 1 and 8);
  workloads serving_0_6b: 256 whole requests at Qwen3-0.6B sizes through LLM.generate (continuous batching), with the
            bytes its steps had to move against the copy bandwidth.
The cache that the decode steps read was written by a real prefill of random prompts.  Every timed step reads 15 GB of weights, far more than the 126 MB L2, so nothing stays cached
between iterations.  Peaks come from MEASURED_PEAKS.json beside this file when present.

    python bench.py --workload serving-0.6b | mixed-32b

runs one of the two other workloads instead (whole requests through LLM.generate, wall clock, a JSON line of its
own): 256 requests with prompts of 16 to 1,024 tokens and 128 new tokens each at Qwen3-0.6B sizes (continuous
batching), or 32 requests with prompts of 512 to 8,192 tokens and 256 new tokens at Qwen3-32B sizes under an
8,192-token step budget and a cache pool too small for all of them (portions, recompute preemption).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=40960, tie_word_embeddings=False, hidden_act="silu",
                attention_bias=False, torch_dtype="bfloat16")
PROMPT_LEN, NEW_TOKENS, CONTEXT, BLOCK = 2048, 256, 4096, 256
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            flat = {}
            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return dict(hbm_gbs=flat["hbm_gbs"], bf16_tflops=flat["bf16_tflops"],
                            bf16_tflops_sustained=flat.get("bf16_tflops_sustained"), source="measured")
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        self.result = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons))


def model_numbers(c):
    H, L, nh, kvh, hd, I, V = (c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"],
                               c["head_dim"], c["intermediate_size"], c["vocab_size"])
    per_layer = (nh + 2 * kvh) * hd * H + nh * hd * H + 3 * I * H
    linear_params = L * per_layer
    weight_bytes = 2 * (linear_params + V * H) + 4 * (L * (2 * H + 2 * hd) + H)   # bf16 matrices + lm_head, f32 norms
    kv_bytes_per_token = 2 * L * kvh * hd * 2
    return dict(linear_params=linear_params, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                lm_head_params=V * H, L=L, nh=nh, hd=hd)


def prefill_flops(c, T):
    n = model_numbers(c)
    linear = 2 * T * n["linear_params"] + 2 * n["lm_head_params"]          # lm_head on one row
    attention = n["L"] * 4 * n["nh"] * n["hd"] * (T * (T + 1) // 2)         # causal QK^T and PV
    return linear + attention


def fill_cache(llm, ids, ctx_len, seed):
    """Prompts of `ctx_len` random tokens for the requests `ids`, run through the step function in steps of at most the
    token budget, so that the pages the decode steps will read hold real keys and values."""
    import torch
    from vllm_oxide_b200 import host
    mgr, core = llm.cache.manager, llm.core
    g = torch.Generator().manual_seed(seed)
    budget = llm.options.max_num_batched_tokens
    for rid in ids:
        toks = torch.randint(0, llm.model.vocab_size, (ctx_len,), generator=g).tolist()
        for start in range(0, ctx_len, budget):
            core.run([host.BatchEntry(rid, start, toks[start:start + budget], [])])
    torch.cuda.synchronize()
    core.check_errors()


def decode_run(llm, batch, steps, warmup, start_ctx):
    """K decode steps of `batch` requests whose context starts at `start_ctx` (prefilled), timed on the device."""
    import torch
    from vllm_oxide_b200 import host, kernels
    mgr, core, sampler = llm.cache.manager, llm.core, llm.sampler
    ids = list(range(10_000, 10_000 + batch))
    for rid in ids:
        assert mgr.add_request(rid) and mgr.ensure(rid, 0, start_ctx)
    fill_cache(llm, ids, start_ctx, seed=batch)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, llm.model.vocab_size, (batch, steps + warmup), generator=g).tolist()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    temp, topk, topp, keys = [0.0] * batch, [0] * batch, [1.0] * batch, [0] * batch
    pos = start_ctx
    launches0 = 0
    for i in range(steps + warmup):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = kernels.launch_count
            ev0.record()
        entries = []
        for b, rid in enumerate(ids):
            assert mgr.ensure(rid, pos, 1)
            entries.append(host.BatchEntry(rid, pos, [toks[b][i]], [0]))
        logits = core.run(entries)
        sampler.forward(logits, temp, topk, topp, keys)
        pos += 1
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    launches = kernels.launch_count - launches0
    core.check_errors()
    for rid in ids:
        mgr.free_request(rid)
    mean_ctx = start_ctx + warmup + (steps + 1) / 2
    return ms, launches, mean_ctx


def e2e_run(llm, batch, steps, warmup):
    """The same metric through the public calls: prompts of 2,048 host token ids in, tokens out each step.
    Returns (tokens a second, host-to-device bytes a step, device-to-host bytes a step, milliseconds a step)."""
    import torch
    from vllm_oxide_b200 import SamplingParams
    g = torch.Generator().manual_seed(100 + batch)       # other prompts in every run: nothing comes from the prefix cache
    prompts = torch.randint(0, llm.model.vocab_size, (batch, PROMPT_LEN), generator=g).tolist()
    entered = lambda: llm.scheduler.stats.prefill_tokens + llm.scheduler.stats.prefix_hit_tokens
    before = entered()
    # the first requests decode while the later prompts are still being computed: room for those tokens too
    room = steps + warmup + 16 + batch * PROMPT_LEN // llm.options.max_num_batched_tokens
    for p in prompts:
        llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=room, ignore_eos=True))
    while llm.is_running() and entered() - before < batch * PROMPT_LEN:
        llm.step()                            # prompts, in portions under the token budget
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = d2h = 0
    for _ in range(steps):
        llm.step()                            # pinned batch arrays in, sampled tokens out
        h2d += llm.core.h2d_bytes_last + 20 * batch
        d2h += 4 * batch + 4
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert llm.scheduler.num_running == batch, "a request finished inside the timed region"
    while llm.is_running():
        llm.step()
    return batch * steps / dt, h2d // steps, d2h // steps, dt / steps * 1e3


def prefill_run(llm, T, reps=3, warmup=2):
    import torch
    from vllm_oxide_b200 import host
    mgr, core = llm.cache.manager, llm.core
    g = torch.Generator().manual_seed(2)
    best = None
    for i in range(reps + warmup):
        toks = torch.randint(0, llm.model.vocab_size, (T,), generator=g).tolist()
        rid = 20_000 + i
        assert mgr.add_request(rid) and mgr.ensure(rid, 0, T)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        core.run([host.BatchEntry(rid, 0, toks, [T - 1])])
        ev1.record()
        torch.cuda.synchronize()
        mgr.free_request(rid)
        if i >= warmup:
            ms = ev0.elapsed_time(ev1)
            best = ms if best is None else min(best, ms)
    core.check_errors()
    return best


WORKLOADS = {
    "serving-0.6b": dict(
        config=dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                    intermediate_size=3072, tie_word_embeddings=True),
        requests=256, prompt=(16, 1024), new=128, seed=2,
        options=dict(max_model_len=2048, block_size=256, max_num_seqs=256, max_num_batched_tokens=8192, num_kv_blocks=2048)),
    "mixed-32b": dict(
        config=dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                    intermediate_size=25600, tie_word_embeddings=False),
        requests=32, prompt=(512, 8192), new=256, seed=3,
        # all 32 contexts together would need about 580 pages of 256 tokens: the pool holds 400
        options=dict(max_model_len=8192 + 256, block_size=256, max_num_seqs=32, max_num_batched_tokens=8192, num_kv_blocks=400)),
}


def workload_run(name: str, pk=None) -> dict:
    """Whole requests through the public entry point (LLM.generate, wall clock).  Returns the record of the run: rates,
    steps, mean number of requests in a step, and the bytes its steps had to move (every weight once a step, the cache
    of every scheduled request's context, and the float logits of every sampled row written by the output product and
    read by the sampler) against the copy bandwidth."""
    import random
    import torch
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    w = WORKLOADS[name]
    pk = pk or peaks()
    cfg = dict(QWEN3_8B)
    cfg.update(w["config"])
    llm = LLM.from_config(cfg, EngineOptions(dtype="bfloat16", **w["options"]), seed=w["seed"], init_scheme="0.02")
    rng = random.Random(0)
    lo, hi = w["prompt"]
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(lo, hi))] for _ in range(w["requests"])]
    sp = SamplingParams(temperature=0.0, max_tokens=w["new"], ignore_eos=True)
    # warm-up: the same shape of work once with other prompts (libraries, a CUDA graph per batch size met; nothing of the
    # timed prompts may lie in the prefix cache)
    wrng = random.Random(1)
    warm = [[wrng.randrange(cfg["vocab_size"]) for _ in range(len(p))] for p in prompts]
    llm.generate(warm, [sp] * len(warm))
    torch.cuda.synchronize()
    s0 = llm.scheduler.stats
    before = (s0.steps, s0.scheduled_requests, s0.context_tokens, s0.sampled_rows)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, [sp] * len(prompts))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert all(o.finished and len(o.token_ids) == w["new"] for o in outs)
    st, s1 = llm.last_stats, llm.scheduler.stats
    steps, scheduled, context, rows = (b - a for a, b in zip(before, (s1.steps, s1.scheduled_requests, s1.context_tokens,
                                                                      s1.sampled_rows)))
    n = model_numbers(cfg)
    weight_bytes = n["weight_bytes"]       # the layers and the output matrix (tied or not, it is read once a step)
    moved = steps * weight_bytes + context * n["kv_bytes_per_token"] + rows * cfg["vocab_size"] * 8
    achieved = moved / dt / 1e9
    flops = 2 * st.total_tokens * n["linear_params"] + 2 * rows * n["lm_head_params"]
    return {
        "metric": f"tokens/s over whole requests ({name})", "value": round(st.total_tokens / dt, 1), "unit": "tokens/s",
        "generated_tokens_per_s": round(w["requests"] * w["new"] / dt, 1), "seconds": round(dt, 3), "steps": steps,
        "mean_requests_per_step": round(scheduled / max(steps, 1), 1), "preemptions": st.preemptions,
        "bytes_per_step_gb": round(moved / max(steps, 1) / 1e9, 3),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "linear_tflops": round(flops / dt / 1e12, 1),
        "n_gpus": 1, "dtype": "bf16", "impl": "ours", "data": "synthetic token ids, seeded random weights",
        "config": {"model": name, "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "requests": w["requests"],
                   "prompt_min": lo, "prompt_max": hi, "new_tokens": w["new"], "step_budget": w["options"]["max_num_batched_tokens"],
                   "pool_pages": w["options"]["num_kv_blocks"], "block_size": w["options"]["block_size"]}}


def attention_kernels_run(pk) -> dict:
    """The attention kernels alone.  Prefill: Qwen3-8B head shapes, one prompt of 2,048 and of 8,192 tokens, the device
    time of a launch (CUDA events around a graph of 20 launches, so the host's share of a launch is not in it).
    Decode: hundreds of requests with one key split each, 50 launches in a row (caches larger than L2)."""
    import math
    import torch
    from vllm_oxide_b200 import kernels
    dev = "cuda:0"
    nh, kvh, hd = QWEN3_8B["num_attention_heads"], QWEN3_8B["num_key_value_heads"], QWEN3_8B["head_dim"]
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"only": "attention", "heads": nh, "kv_heads": kvh, "head_dim": hd, "block_size": BLOCK, "launches_per_graph": 20}
    for T in (2048, 8192):
        pages = (T + BLOCK - 1) // BLOCK
        kc = torch.randn(pages, kvh, BLOCK, hd, device=dev).bfloat16()
        vc = torch.randn(pages, kvh, BLOCK, hd, device=dev).bfloat16()
        bt = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
        q = torch.randn(T, nh * hd, device=dev).bfloat16()
        o = torch.empty_like(q)
        cu_q = torch.tensor([0, T], dtype=torch.int32, device=dev)
        ctx = torch.tensor([T], dtype=torch.int32, device=dev)

        def launch():
            kernels.attention_prefill(q, nh * hd, o, kc, vc, bt, cu_q, ctx, 1, T, nh, kvh, hd, 0, 1 / math.sqrt(hd), err)
        for _ in range(3):
            launch()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(20):
                launch()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 20)
        ms = sorted(times)[len(times) // 2]
        flops = 4 * nh * hd * T * (T + 1) / 2
        tf = flops / ms / 1e9
        out[f"prefill_{T}"] = {"us": round(ms * 1e3, 1), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}
        assert err.item() == 0
        del kc, vc, q, o
    # Decode attention of many requests with one key split each (the serving workload's shape: 16 heads over 8 kv heads,
    # contexts of 300 to 1,000 keys): persistent blocks against one block per (request, kv head).
    nh, g = 16, torch.Generator().manual_seed(1)
    for name, B, lo, hi in (("decode_228x650", 228, 650, 650), ("decode_228x300_1000", 228, 300, 1000), ("decode_512x100_400", 512, 100, 400)):
        ctx_host = torch.randint(lo, hi + 1, (B,), generator=g).int()
        per = (hi + BLOCK - 1) // BLOCK
        kc = torch.randn(B * per, kvh, BLOCK, hd, device=dev).bfloat16()
        vc = torch.randn(B * per, kvh, BLOCK, hd, device=dev).bfloat16()
        bt = torch.randperm(B * per, generator=g).int().view(B, per).to(dev)
        q = torch.randn(B, nh * hd, device=dev).bfloat16()
        o = torch.empty_like(q)
        cu_q = torch.arange(B + 1, dtype=torch.int32, device=dev)
        ctx = ctx_host.to(dev)
        nbytes = float(ctx_host.sum()) * kvh * hd * 2 * 2
        row = {}
        for mode, pairs in (("persistent", kernels.decode_pairs_counter(dev)), ("block_per_pair", None)):

            def launch():
                kernels.attention_decode(q, nh * hd, o, kc, vc, bt, cu_q, ctx, B, nh, kvh, hd, 0, 1 / math.sqrt(hd), 1, None, err,
                                         pairs=pairs)
            for _ in range(5):
                launch()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                launch()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 50 * 1e3
            row[mode] = {"us": round(us, 1), "gbs": round(nbytes / us / 1e3), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        out[name] = row
        assert err.item() == 0
        del kc, vc
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (reported)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None, help="another workload instead of the default run")
    ap.add_argument("--only", choices=["decode", "prefill", "attention"], default=None,
                    help="run one phase and print its time only (for short profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust crate on candle: no Rust toolchain or "
                          "network here, and pip finds neither setup.py nor pyproject.toml in it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.workload:
        print(json.dumps(workload_run(args.workload)))
        return 0
    if args.only == "attention":
        print(json.dumps(attention_kernels_run(peaks())))
        return 0
    import torch
    from vllm_oxide_b200 import LLM, EngineOptions

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    cfg = dict(QWEN3_8B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    n = model_numbers(cfg)
    max_batch = 64 if not args.skip_points else args.batch
    pages_per_req = (PROMPT_LEN + NEW_TOKENS + BLOCK - 1) // BLOCK + 1
    opts = EngineOptions(max_model_len=CONTEXT, block_size=BLOCK, num_kv_blocks=max_batch * pages_per_req + 16,
                         max_num_seqs=max(max_batch, 8), max_num_batched_tokens=8192, dtype="bfloat16")
    llm = LLM.from_config(cfg, opts, seed=0, init_scheme="0.02")

    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "ms": prefill_run(llm, PROMPT_LEN, reps=1, warmup=1)}))
        return 0
    if args.only == "decode":
        ms, launches, _ = decode_run(llm, args.batch, steps, warmup, PROMPT_LEN)
        print(json.dumps({"only": "decode", "ms_per_step": ms, "gpu_launches": launches}))
        return 0
    prefill_ms = prefill_run(llm, PROMPT_LEN)
    with ClockSampler() as clocks:
        ms, launches, mean_ctx = decode_run(llm, args.batch, steps, warmup, PROMPT_LEN)
    value = args.batch * 1000.0 / ms

    def hbm_frac(batch, ctx, step_ms):
        return (n["weight_bytes"] + batch * ctx * n["kv_bytes_per_token"]) / (step_ms * 1e-3) / 1e9 / pk["hbm_gbs"]
    achieved = hbm_frac(args.batch, mean_ctx, ms) * pk["hbm_gbs"]
    e2e, h2d, d2h, e2e_ms = e2e_run(llm, args.batch, steps, warmup)
    points, workloads = {}, {}
    if not args.skip_points:
        short = min(steps, 32)
        points[f"host_ms_b{args.batch}"] = round(e2e_ms - ms, 4)
        for b in (1, 16, 32, 64):
            pms, _, ctx = decode_run(llm, b, short, warmup, PROMPT_LEN)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            points[f"frac_b{b}"] = round(hbm_frac(b, ctx, pms), 4)
            if b in (1, 64):
                rate, _, _, step_ms = e2e_run(llm, b, short, warmup)
                points[f"e2e_b{b}"] = round(rate, 1)
                points[f"host_ms_b{b}"] = round(step_ms - pms, 4)
        # longer contexts: another engine over the same model (its decode steps are shaped for up to 32,768 keys)
        config, model = llm.config, llm.model
        del llm
        torch.cuda.empty_cache()
        long_ctx = 32768
        pages = 8 * (long_ctx // BLOCK + 2) + 8
        opts = EngineOptions(max_model_len=long_ctx + 2 * BLOCK, block_size=BLOCK, num_kv_blocks=pages, max_num_seqs=8,
                             max_num_batched_tokens=8192, dtype="bfloat16")
        llm = LLM("<random weights>", opts, _model=(config, model))
        # a longer prompt in one step (attention is a larger share of it)
        p_ms = prefill_run(llm, 8192, reps=2, warmup=1)
        points["prefill_8192"] = round(8192 * 1000.0 / p_ms, 1)
        points["frac_prefill_8192"] = round(prefill_flops(cfg, 8192) / (p_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        for ctx0 in (8192, long_ctx):
            for b in (1, 8):
                pms, _, ctx = decode_run(llm, b, 16, warmup, ctx0)
                points[f"decode_b{b}_ctx{ctx0}"] = round(b * 1000.0 / pms, 1)
                points[f"frac_b{b}_ctx{ctx0}"] = round(hbm_frac(b, ctx, pms), 4)
        del llm, model
        torch.cuda.empty_cache()
        w = workload_run("serving-0.6b", pk)
        workloads["serving_0_6b"] = {k: w[k] for k in ("value", "generated_tokens_per_s", "seconds", "steps",
                                                       "mean_requests_per_step", "bytes_per_step_gb", "roofline")}
    flops = prefill_flops(cfg, PROMPT_LEN)
    line = {
        "metric": "decode tok/s (Qwen3-8B sizes, bf16, batch 8, context 2048+)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, seeded random weights",
        "impl": "ours",
        "config": {"model": "Qwen3-8B sizes", "layers": cfg["num_hidden_layers"], "layers_of_config": 36,
                   "hidden": 4096, "heads": 32, "kv_heads": 8, "head_dim": 128, "intermediate": 12288, "vocab": 151936,
                   "global_batch": args.batch, "seq_len": PROMPT_LEN, "new_tokens": NEW_TOKENS, "context": CONTEXT,
                   "block_size": BLOCK, "parallelism": "single GPU", "l2": "every step reads 15 GB of weights (inputs larger than L2)",
                   "peaks": pk["source"]},
        "clocks": clocks.result,
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT_LEN * 1000.0 / prefill_ms, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
