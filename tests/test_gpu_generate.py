"""Generation through the Python entry point and the command line: greedy tokens against the plain
implementation, sampling that does not depend on the batch, small pools, the prefix cache."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TINY, tokens_for
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu


def make_llm(model_folders, name, dtype="float32", **kw):
    from vllm_oxide_b200 import LLM, EngineOptions
    opts = dict(max_model_len=256, block_size=TINY[name]["block_size"], num_kv_blocks=64, dtype=dtype, max_num_seqs=16)
    opts.update(kw)
    return LLM(model_folders[name], EngineOptions(**opts))


@pytest.mark.parametrize("name,lengths,new", [("A", [7, 33, 1, 64], 16), ("B", [1, 5, 31, 32, 33, 100], 20), ("C", [40, 3], 30),
                                              ("D", [70, 2, 130], 24)])
def test_greedy_generation_matches_the_plain_implementation(model_folders, plain_models, name, lengths, new):
    from vllm_oxide_b200 import SamplingParams
    cfg, w = plain_models[name]
    prompts = [tokens_for(name, n, salt=200 + i) for i, n in enumerate(lengths)]
    llm = make_llm(model_folders, name)
    outs = llm.generate(prompts, [SamplingParams(max_tokens=new, ignore_eos=True)] * len(prompts))
    assert [o.seq_id for o in outs] == list(range(len(prompts))) and all(o.finished for o in outs)
    for p, o in zip(prompts, outs):
        assert o.token_ids == P.greedy_generate(cfg, w, p, new, torch.float32)
    again = llm.generate(prompts[:2], SamplingParams(max_tokens=4, ignore_eos=True))   # a second call works
    assert [o.token_ids for o in again] == [o.token_ids[:4] for o in outs[:2]]
    assert llm.cache.manager.num_requests == 0 and llm.cache.manager.check_invariants() == ""


@pytest.mark.parametrize("name", ["B", "D"])
def test_greedy_bfloat16_agrees_with_the_plain_bfloat16_run_where_it_is_sure(model_folders, plain_models, name):
    """B runs on the plain kernels, D on the tensor-core and weight-streaming ones, decoding from CUDA graphs."""
    from vllm_oxide_b200 import SamplingParams
    cfg, w = plain_models[name]
    prompt = tokens_for(name, 25, salt=5)
    llm = make_llm(model_folders, name, "bfloat16")
    got = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True))[0].token_ids
    ids = list(prompt)
    sure = 0
    for tok in got:       # follow the engine's tokens; wherever the plain top-2 gap is clear they must agree
        logits = P.forward_logits(cfg, w, ids, torch.bfloat16)[-1]
        top = torch.topk(logits, 2)
        if top.values[0] - top.values[1] > 0.05 * logits.abs().max():
            assert tok == int(top.indices[0])
            sure += 1
        ids.append(tok)
    assert sure >= 4, f"only {sure} of 12 steps had a clear winner: the comparison shows nothing"


def test_chunked_prefill_small_budget_and_tiny_pool_do_not_change_the_tokens(model_folders):
    from vllm_oxide_b200 import SamplingParams
    name = "B"
    prompts = [tokens_for(name, n, salt=300 + i) for i, n in enumerate([1, 5, 31, 32, 33, 100])]
    sp = [SamplingParams(max_tokens=20, ignore_eos=True)] * len(prompts)
    base = [o.token_ids for o in make_llm(model_folders, name).generate(prompts, sp)]
    chunked = make_llm(model_folders, name, max_num_batched_tokens=24)
    assert [o.token_ids for o in chunked.generate(prompts, sp)] == base
    assert chunked.last_stats.steps > 20
    tiny = make_llm(model_folders, name, num_kv_blocks=6, max_num_batched_tokens=40)    # 6 pages of 32: forces preemption
    assert [o.token_ids for o in tiny.generate(prompts, sp)] == base
    assert tiny.last_stats.preemptions > 0
    assert tiny.cache.manager.num_free_blocks(0) == 6 and tiny.cache.manager.check_invariants() == ""


def test_prefix_cache_hits_do_not_change_the_tokens(model_folders):
    from vllm_oxide_b200 import SamplingParams
    name = "B"
    shared = tokens_for(name, 64, salt=1)
    prompts = [shared + tokens_for(name, 9, salt=2), shared + tokens_for(name, 30, salt=3)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    off = make_llm(model_folders, name, enable_prefix_caching=False)
    base = [off.generate([p], sp)[0].token_ids for p in prompts]
    on = make_llm(model_folders, name)
    first = on.generate([prompts[0]], sp)[0].token_ids
    second = on.generate([prompts[1]], sp)[0].token_ids
    assert on.last_stats.prefix_hit_tokens == 64 and [first, second] == base


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "E"])
def test_scheduled_steps_with_hits_and_preemption_give_the_plain_logits(model_folders, plain_models, name, dtype):
    """The scheduler's own steps (a 24-token budget, prompts of 1 to 100 tokens, two requests that share their first two
    pages, so few pages that requests are preempted and recomputed): the logits of EVERY row a token was sampled from
    against the plain implementation of that request's own tokens up to there.  A row computed over another request's
    pages, over pages that were recomputed after a preemption, or over stale pages would show as a wrong number."""
    import numpy as np
    from test_gpu_replay import check, plain_logits
    from vllm_oxide_b200 import SamplingParams
    bs = TINY[name]["block_size"]
    shared = tokens_for(name, 2 * bs, salt=800)
    lengths = [1, 5, 31, 32, 33]
    prompts = [tokens_for(name, n, salt=801 + i) for i, n in enumerate(lengths)]
    prompts += [shared + tokens_for(name, 100 - 2 * bs, salt=810), shared + tokens_for(name, 17, salt=811)]
    pages = 6 if bs == 32 else 12                      # the pool holds 192 tokens; the requests need far more
    llm = make_llm(model_folders, name, dtype, num_kv_blocks=pages, max_num_batched_tokens=24, max_num_seqs=8)
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    ids = [llm.add_request(p, sp) for p in prompts]
    prompt_of = dict(zip(ids, prompts))
    rows = {i: [] for i in ids}                        # per request: (number of tokens the row stands after, logits)
    finished = {}
    while llm.is_running():
        outs, logits = llm.step(want_logits=True)
        for o in outs:
            finished[o.seq_id] = o.token_ids
        for row, rid in enumerate(llm.last_sampled_ids):
            toks = prompt_of[rid] + finished[rid] if rid in finished else list(llm.scheduler.sequence(rid).tokens)
            rows[rid].append((len(toks) - 1, logits[row]))          # toks ends with the token sampled from this row
        assert llm.cache.manager.check_invariants() == ""
    stats = llm.scheduler.stats
    assert stats.prefix_hit_tokens > 0 and stats.preemptions > 0
    assert llm.cache.manager.num_free_blocks(0) == pages
    for rid in ids:
        full = prompt_of[rid] + finished[rid]
        assert len(finished[rid]) == 20 and [n for n, _ in rows[rid]] == list(range(len(prompt_of[rid]), len(full)))
        want = plain_logits(plain_models, name, full[:-1], dtype)
        places = [n - 1 for n, _ in rows[rid]]
        check(np.stack([l for _, l in rows[rid]]), want[places], dtype, f"{name} scheduled request {rid}")
        if dtype == "float32":
            assert finished[rid] == [int(l.argmax()) for _, l in rows[rid]]


def test_sampled_generation_is_seeded_and_independent_of_the_batch(model_folders):
    from vllm_oxide_b200 import SamplingParams
    name = "B"      # its logits are flat enough for sampling to matter (A's tied output is sharply peaked)
    prompts = [tokens_for(name, n, salt=400 + i) for i, n in enumerate([7, 33, 1, 64])]
    sp = SamplingParams(temperature=0.8, max_tokens=16, ignore_eos=True, seed=123)
    llm = make_llm(model_folders, name)
    together = [o.token_ids for o in llm.generate(prompts, [sp] * 4)]
    llm2 = make_llm(model_folders, name)
    assert [o.token_ids for o in llm2.generate(prompts, [sp] * 4)] == together          # same seed, same tokens
    other = SamplingParams(temperature=0.8, max_tokens=16, ignore_eos=True, seed=124)
    assert [o.token_ids for o in make_llm(model_folders, name).generate(prompts, [other] * 4)] != together
    # a request that brings its seed draws the same numbers alone, later in the same engine, or in another order
    assert make_llm(model_folders, name).generate(prompts[:1], [sp])[0].token_ids == together[0]
    assert llm.generate(prompts[2:3], [sp])[0].token_ids == together[2]
    assert [o.token_ids for o in llm2.generate(prompts[::-1], [sp] * 4)] == together[::-1]
    # without a seed of its own a request's numbers are keyed by the engine's seed and its id: two copies of one
    # prompt in one call differ, and a fresh engine with the same seed repeats the call
    free = SamplingParams(temperature=0.8, max_tokens=16, ignore_eos=True)
    a = [o.token_ids for o in make_llm(model_folders, name, seed=9).generate([prompts[1]] * 2, [free] * 2)]
    assert a[0] != a[1]
    assert [o.token_ids for o in make_llm(model_folders, name, seed=9).generate([prompts[1]] * 2, [free] * 2)] == a
    greedy = [o.token_ids for o in make_llm(model_folders, name).generate(prompts, SamplingParams(max_tokens=16, ignore_eos=True))]
    assert greedy != together
    topk = SamplingParams(temperature=1.0, top_k=8, top_p=0.9, max_tokens=20, ignore_eos=True, seed=5)
    toks = make_llm(model_folders, "B").generate([tokens_for("B", 31, salt=1)], [topk])[0].token_ids
    assert len(toks) == 20


def test_eos_and_max_tokens_and_errors(model_folders, plain_models):
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    name = "A"
    cfg, w = plain_models[name]
    prompt = tokens_for(name, 12, salt=9)
    ref = P.greedy_generate(cfg, w, prompt, 8, torch.float32)
    import json, shutil, tempfile
    folder = tempfile.mkdtemp()
    for f in os.listdir(model_folders[name]):
        shutil.copy(os.path.join(model_folders[name], f), folder)
    c = json.load(open(os.path.join(folder, "config.json")))
    c["eos_token_id"] = ref[3]
    json.dump(c, open(os.path.join(folder, "config.json"), "w"))
    llm = LLM(folder, EngineOptions(max_model_len=128, block_size=16, num_kv_blocks=16, dtype="float32"))
    out = llm.generate([prompt], [SamplingParams(max_tokens=8)])[0]
    stop = ref.index(ref[3]) + 1
    assert out.token_ids == ref[:stop] and out.finish_reason == "stop"
    assert llm.generate([prompt], [SamplingParams(max_tokens=8, ignore_eos=True)])[0].token_ids == ref
    assert llm.generate([], []) == []
    with pytest.raises(ValueError, match="expected 2 sampling_params"):
        llm.generate([prompt, prompt], [SamplingParams()])
    with pytest.raises(RuntimeError, match="max_model_len"):
        llm.generate([prompt], [SamplingParams(max_tokens=500)])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        llm.generate([[1, 99999]], [SamplingParams()])
    with pytest.raises(ValueError, match="tokenizer"):
        llm.generate(["some text"], [SamplingParams()])
    with pytest.raises(ValueError, match="max_position_embeddings"):
        LLM(folder, EngineOptions(max_model_len=4096, num_kv_blocks=4, block_size=16))
    logits = llm.generate_logits(prompt, 5)
    assert logits.shape == (5, 256) and logits.argmax(-1).tolist() == ref[:5]
    shutil.rmtree(folder)


def test_command_line(model_folders, plain_models):
    cfg, w = plain_models["A"]
    prompt = tokens_for("A", 9, salt=3)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "vllm-oxide"), "-m", model_folders["A"], "--token-ids",
                           "--max-tokens", "6", "--dtype", "float32", "--max-model-len", "128", "--block-size", "16",
                           "--num-kv-blocks", "8", "--ignore-eos", " ".join(map(str, prompt))],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == P.greedy_generate(cfg, w, prompt, 6, torch.float32)


def test_command_line_with_random_weights_and_no_model_folder(model_folders, plain_models, tmp_path):
    """`--random-weights --config <config.json> --seed N` builds the model from the configuration and the seed alone and
    generates the tokens that the plain implementation generates from the folder written with the same seed."""
    name = "B"
    cfg, w = plain_models[name]                         # the folder the fixtures wrote with TINY[name]["seed"]
    prompt = tokens_for(name, 11, salt=4)
    config = tmp_path / "config.json"
    config.write_text(open(os.path.join(model_folders[name], "config.json")).read())
    base = [sys.executable, os.path.join(ROOT, "bin", "vllm-oxide"), "--token-ids", "--max-tokens", "7", "--dtype", "float32",
            "--max-model-len", "128", "--block-size", "32", "--num-kv-blocks", "8", "--ignore-eos"]
    proc = subprocess.run(base + ["--random-weights", "--config", str(config), "--seed", str(TINY[name]["seed"]),
                                  " ".join(map(str, prompt))], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == P.greedy_generate(cfg, w, prompt, 7, torch.float32)
    other = subprocess.run(base + ["--random-weights", "--config", str(config), "--seed", "99", " ".join(map(str, prompt))],
                           capture_output=True, text=True, timeout=600)
    assert other.returncode == 0 and other.stdout != proc.stdout                 # another seed, another model
    for bad in (["--random-weights"], ["--random-weights", "--config", str(config), "-m", model_folders[name]], []):
        refused = subprocess.run(base + bad + ["1 2 3"], capture_output=True, text=True, timeout=600)
        assert refused.returncode == 2 and "--" in refused.stderr


def test_a_folder_with_tensors_the_model_does_not_use_loads_and_generates(model_folders, plain_models, tmp_path):
    """A checkpoint with tied output that also stores lm_head.weight (as published small checkpoints do) and rotary
    buffers: the extra tensors are reported and ignored, and the tokens are the plain implementation's."""
    import shutil
    import warnings
    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
    from vllm_oxide_b200.weights import SafetensorsFile, write_safetensors
    from vllm_oxide_b200.weights.loader import UnexpectedTensorsWarning
    name = "A"                                          # tied output
    cfg, w = plain_models[name]
    folder = str(tmp_path / "m")
    shutil.copytree(model_folders[name], folder)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["lm_head.weight"] = torch.randn(256, 64)    # not the embedding: it must not be read
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    del f
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        llm = LLM(folder, EngineOptions(max_model_len=128, block_size=16, num_kv_blocks=16, dtype="float32"))
    assert any(issubclass(c.category, UnexpectedTensorsWarning) for c in caught)
    assert llm.model.unexpected_tensors == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    prompt = tokens_for(name, 12, salt=9)
    assert llm.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids == \
        P.greedy_generate(cfg, w, prompt, 8, torch.float32)


def greedy_tokens_agree_with_32_bit_logits(runner, prompt, tokens, what):
    """The tokens a bfloat16 engine chose greedily, fed to the 32-bit engine (`runner`, a float32 TraceRunner over the same
    weights): wherever the 32-bit logits have a clear winner (a gap of 5 % of the largest logit) it is the token that
    was chosen.  Returns how many places were that clear."""
    import numpy as np
    toks = list(prompt) + list(tokens)
    first = len(prompt) - 1
    logits = runner.step([dict(id=what, tokens=toks[:-1], want=list(range(first, len(toks) - 1)))], [what])
    sure = 0
    for row, tok in zip(logits, tokens):
        order = np.argsort(row)
        if row[order[-1]] - row[order[-2]] > 0.05 * np.abs(row).max():
            assert tok == int(order[-1]), f"{what}: chose {tok} where the 32-bit path has {int(order[-1])} by a clear margin"
            sure += 1
    return sure


def test_the_same_work_twice_gives_the_same_tokens_bit_for_bit(model_folders):
    """bfloat16 on the fast kernels, decoding from CUDA graphs: a second run in the same engine lands on other pages
    and replays the graphs the first run captured; without prefix hits (which change how prompts are cut, and with
    that the rounding) every token must repeat exactly.  A kernel that read another kernel's output too early, or
    whose result depended on where its pages lie, would show here."""
    from vllm_oxide_b200 import SamplingParams
    llm = make_llm(model_folders, "D", "bfloat16", enable_prefix_caching=False, max_num_batched_tokens=96)
    prompts = [tokens_for("D", n, salt=600 + i) for i, n in enumerate([70, 2, 130, 64, 33])]
    sps = [SamplingParams(temperature=0.0 if i % 2 == 0 else 0.9, top_k=20 if i == 3 else None, max_tokens=60,
                          ignore_eos=True, seed=i) for i in range(len(prompts))]
    first = [o.token_ids for o in llm.generate(prompts, sps)]
    assert llm.core.graph_replays > 0
    llm.generate(prompts[:2], sps[:2])                 # other work in between: the free list is in another order now
    assert [o.token_ids for o in llm.generate(prompts, sps)] == first
    # and they are the right tokens, not only the same ones: the greedy requests against the 32-bit path
    from vllm_oxide_b200.engine.trace import TraceRunner
    full = TraceRunner(model_folders["D"], "float32", 256, TINY["D"]["block_size"])
    sure = sum(greedy_tokens_agree_with_32_bit_logits(full, p, t, f"request {i}")
               for i, (p, t) in enumerate(zip(prompts, first)) if sps[i].temperature == 0.0)
    assert sure >= 60, f"only {sure} of 180 greedy steps had a clear winner"


def test_hundreds_of_requests_decode_through_the_persistent_attention_blocks(model_folders):
    """160 live requests with two key/value heads are more (request, kv head) pairs than blocks fit the GPU, so decode
    attention runs as persistent blocks that draw their pairs from a counter: the greedy tokens are the ones the 32-bit
    path is sure of, and they are the same, bit for bit, with one block per pair."""
    from vllm_oxide_b200 import SamplingParams, kernels
    from vllm_oxide_b200.engine.trace import TraceRunner
    n, new = 160, 6
    prompts = [tokens_for("D", 3 + (7 * i) % 58, salt=900 + i) for i in range(n)]
    sp = SamplingParams(max_tokens=new, ignore_eos=True)
    assert n * TINY["D"]["config"]["num_key_value_heads"] > 2 * kernels.sm_count()
    runs = []
    for persistent in (True, False):
        llm = make_llm(model_folders, "D", "bfloat16", max_num_seqs=n, num_kv_blocks=2 * n + 8, max_num_batched_tokens=8192,
                       enable_prefix_caching=False)
        mixers = [p for b in llm.model.blocks for p in b.parts() if hasattr(p, "_pairs")]
        assert mixers and all(m._pairs is not None for m in mixers)
        if not persistent:
            for m in mixers:
                m._pairs = None                    # without its counter a layer runs one block per pair
        runs.append([o.token_ids for o in llm.generate(prompts, [sp] * n)])
        assert llm.core.graph_replays > 0
        assert all(m._pairs is None or m._pairs.tolist() == [0, 0] for m in mixers)
        del llm
    assert runs[0] == runs[1]
    full = TraceRunner(model_folders["D"], "float32", 256, TINY["D"]["block_size"])
    sure = sum(greedy_tokens_agree_with_32_bit_logits(full, prompts[i], runs[0][i], f"request {i}") for i in range(0, n, 8))
    assert sure >= 30, f"only {sure} of {new * n // 8} greedy steps had a clear winner"


def test_a_decode_graph_padded_beyond_the_step_limits(model_folders):
    """Five requests with max_num_seqs 5 and a budget of 6 tokens decode from the graph for 8 requests: a layout larger
    than any step the limits allow (the staging buffers must hold it), with the same tokens as without graphs."""
    from vllm_oxide_b200 import SamplingParams
    name = "D"
    prompts = [tokens_for(name, n, salt=700 + i) for i, n in enumerate([3, 9, 2, 11, 5])]
    sp = [SamplingParams(max_tokens=12, ignore_eos=True)] * len(prompts)
    eager = make_llm(model_folders, name, max_num_seqs=5, max_num_batched_tokens=6, enforce_eager=True)
    want = [o.token_ids for o in eager.generate(prompts, sp)]
    llm = make_llm(model_folders, name, max_num_seqs=5, max_num_batched_tokens=6)
    assert [o.token_ids for o in llm.generate(prompts, sp)] == want
    assert llm.core.graph_replays > 0 and 8 in llm.core._graphs


def test_kernel_class_timers_behind_a_flag(model_folders):
    """With the timers on, every launch of the package's kernels is bracketed by events and the report adds the device
    time up by entry point; off (the default), nothing is recorded."""
    import time
    from vllm_oxide_b200 import SamplingParams, kernels
    llm = make_llm(model_folders, "D", "bfloat16", enforce_eager=True)
    prompt = tokens_for("D", 70, salt=11)
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    want = llm.generate([prompt], sp)[0].token_ids
    with pytest.raises(kernels.KernelError, match="timers are off"):
        kernels.kernel_timer_report()
    kernels.enable_kernel_timers()
    try:
        before = kernels.launch_count
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert llm.generate([prompt], sp)[0].token_ids == want          # timing changes no result
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        report = kernels.kernel_timer_report()
    finally:
        kernels.enable_kernel_timers(False)
    assert sum(n for n, _ in report.values()) == kernels.launch_count - before
    for name in ("embedding", "gemm_skinny", "qk_norm_rope_kv_write", "attention_decode_tma", "attention_prefill_tc5", "sample"):
        assert report[name][0] > 0 and report[name][1] > 0.0, (name, report)
    assert 0.0 < sum(ms for _, ms in report.values()) < wall_ms
