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
    for tok in got:       # follow the engine's tokens; wherever the plain top-2 gap is clear they must agree
        logits = P.forward_logits(cfg, w, ids, torch.bfloat16)[-1]
        top = torch.topk(logits, 2)
        if top.values[0] - top.values[1] > 0.1 * logits.abs().max():
            assert tok == int(top.indices[0])
        ids.append(tok)


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
