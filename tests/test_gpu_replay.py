"""Trace replay against the plain implementation: the same requests whole, with the last 32 tokens
decoded one by one, in portions of changing size, and mixed with other requests over so few pages
that pages are used again; in 32-bit and in bfloat16."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, TINY, tokens_for
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
NAMES = ["A", "B", "C", "D", "E"]
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [7, 33, 1, 64, 150, 260], "B": [1, 5, 31, 32, 33, 100, 300], "C": [3, 70, 41, 129, 16], "D": [2, 65, 130, 257, 64], "E": [1, 17, 64, 129, 200]}

_plain_cache = {}


def plain_logits(plain_models, name, tokens, dtype):
    """Plain logits at every position.  For float32 the float64 run (the truth a 32-bit path is held to);
    for bfloat16 the pair (float64 run, plain bfloat16 run): the second measures what rounding to
    bfloat16 at every operation costs on this very sequence."""
    key = (name, tuple(tokens), dtype)
    if key not in _plain_cache:
        cfg, w = plain_models[name]
        truth = P.forward_logits(cfg, w, tokens, torch.float64).numpy()
        if dtype == "float32":
            _plain_cache[key] = truth
        else:
            _plain_cache[key] = Both(truth, P.forward_logits(cfg, w, tokens, torch.bfloat16).double().numpy())
    return _plain_cache[key]


class Both:
    """Truth and the plain bfloat16 run; slicing slices both."""

    def __init__(self, truth, rounded):
        self.truth, self.rounded = truth, rounded

    def __getitem__(self, idx):
        return Both(self.truth[idx], self.rounded[idx])

    def __len__(self):
        return len(self.truth)


def check(got, want, dtype, what):
    """Against the float64 run alone (32-bit path, small models): within 2e-5 of the logits' scale.
    Against a `Both` (the float64 run and a plain run in the engine's own precision over the same weights): the engine
    must be as close to the float64 run as that plain run is: at most 1.5 times its root-mean-square error and 2.5
    times its worst error (two runs that round at every operation, in different orders, differ from each other by
    about 1.4 times that error).  That is the bound for bfloat16 everywhere, and for the 32-bit path of a model of
    many layers, where rounding alone exceeds any fixed small bound."""
    got = np.asarray(got, np.float64)
    if not isinstance(want, Both):
        assert dtype == "float32", what
        want = np.asarray(want, np.float64)
        assert got.shape == want.shape, what
        worst = np.abs(got - want).max() / np.abs(want).max()
        assert worst < 2e-5, f"{what}: {worst:.3e} of scale"
        return
    truth, rounded = np.asarray(want.truth, np.float64), np.asarray(want.rounded, np.float64)
    assert got.shape == truth.shape, what
    rms = lambda d: np.sqrt((d ** 2).mean())
    floor_rms, floor_worst = rms(rounded - truth), np.abs(rounded - truth).max()
    got_rms, got_worst = rms(got - truth), np.abs(got - truth).max()
    assert got_rms <= 1.5 * floor_rms and got_worst <= 2.5 * floor_worst, \
        f"{what}: rms {got_rms:.3e} vs the plain run in {dtype} {floor_rms:.3e}; worst {got_worst:.3e} vs {floor_worst:.3e}"


def check_same(a, b, dtype, what):
    """Two cuts of the same work: the 32-bit kernels give the same bits (every output element has one chain of operations
    whatever the batch); the bfloat16 kernels differ for one-token and many-token requests and agree beyond rounding."""
    if dtype == "float32":
        a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
        assert a.shape == b.shape and np.array_equal(a, b), \
            f"{what}: {int((a != b).sum())} of {a.size} logits differ, by up to {np.abs(a - b).max():.3e}"
        return
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = np.abs(a).max()
    worst = np.abs(a - b).max() / scale
    assert worst < 0.03, f"{what}: {worst:.3e} of scale"


def runner(model_folders, name, dtype, max_tokens):
    from vllm_oxide_b200.engine.trace import TraceRunner
    return TraceRunner(model_folders[name], dtype, max_tokens, TINY[name]["block_size"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_and_decode_and_portions(model_folders, plain_models, name, dtype):
    bs = TINY[name]["block_size"]
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_for(name, n, salt=i)
        want = plain_logits(plain_models, name, toks, dtype)
        pool = (n + bs - 1) // bs * bs
        # whole, every position wanted
        r = runner(model_folders, name, dtype, pool)
        whole = r.step([dict(id="w", tokens=toks, want=list(range(n)))], ["w"])
        check(whole, want, dtype, f"{name} len {n} whole")
        assert r.manager.num_free_blocks(0) == pool // bs and r.manager.check_invariants() == ""
        # most of it in one step, the last 32 one by one
        cut = max(1, n - 32)
        r = runner(model_folders, name, dtype, pool)
        rows = [r.step([dict(id="d", tokens=toks[:cut], want=[cut - 1])], [])[0]]
        for t in range(cut, n):
            rows.append(r.step([dict(id="d", tokens=[toks[t]], want=[0])], ["d"] if t == n - 1 else [])[0])
        check(np.stack(rows), want[cut - 1:], dtype, f"{name} len {n} decode")
        check_same(np.stack(rows), whole[cut - 1:], dtype, f"{name} len {n} decode vs whole")
        # portions of changing size, down to two tokens
        rng = random.Random(n)
        r = runner(model_folders, name, dtype, pool)
        got, pos = [], 0
        sizes = [2, 3, 17, 2, bs, bs + 1, 5, 2, 64]
        while pos < n:
            m = min(sizes[len(got) % len(sizes)] if rng.random() < 0.7 else rng.randrange(2, 40), n - pos)
            got.append(r.step([dict(id="p", tokens=toks[pos:pos + m], want=list(range(m)))], []))
            pos += m
        check(np.concatenate(got), want, dtype, f"{name} len {n} portions")
        check_same(np.concatenate(got), whole, dtype, f"{name} len {n} portions vs whole")


def mixed_schedule(name, lengths, seed):
    """Steps for up to four live requests: portions of some beside decoded tokens of others; a request
    may sit out a step. Returns (steps, requests, peak of live tokens rounded up to pages)."""
    reqs = {f"r{i}": tokens_for(name, n, salt=50 + i) for i, n in enumerate(lengths)}
    return mixed_schedule_of(reqs, TINY[name]["block_size"], seed)


def mixed_schedule_of(reqs, bs, seed, portions=None):
    """The same for given requests {id: tokens} and page size; `portions`: the sizes a portion is drawn from."""
    rng = random.Random(seed)
    portions = portions or [2, 2, 3, 5, bs - 1, bs, bs + 1, 40]
    waiting = list(reqs)
    live, pos, steps, peak = [], {}, [], 0
    while waiting or live:
        while waiting and len(live) < 4 and (not live or rng.random() < 0.6):
            rid = waiting.pop(0)
            live.append(rid); pos[rid] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue                                          # left out of this step
            n, p = len(reqs[rid]), pos[rid]
            left = n - p
            if left <= 32 or rng.random() < 0.3:
                m = 1                                             # decoding
            else:
                m = min(left, rng.choice(portions))
            entries.append(dict(id=rid, tokens=reqs[rid][p:p + m], want=list(range(m)), _at=p))
            pos[rid] += m
        peak = max(peak, sum((pos[r] + bs - 1) // bs * bs for r in live))
        for e in entries:
            if pos[e["id"]] == len(reqs[e["id"]]):
                end.append(e["id"]); live.remove(e["id"])
        if entries:
            steps.append(dict(step=len(steps), entries=entries, end=end))
    return steps, reqs, peak


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_used_again(model_folders, plain_models, name, dtype):
    lengths = [90, 40, 66, 35, 120, 50, 77, 34, 45]
    steps, reqs, peak = mixed_schedule(name, lengths, seed=3)
    bs = TINY[name]["block_size"]
    total_pages = sum((len(t) + bs - 1) // bs for t in reqs.values())
    assert peak // bs < 0.7 * total_pages                         # the pool is far smaller than all requests
    r = runner(model_folders, name, dtype, peak)
    got = {rid: [None] * len(t) for rid, t in reqs.items()}
    assert any(len(s["entries"]) >= 3 for s in steps)
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps)   # portions beside decodes
    for s in steps:
        out = r.step([{k: v for k, v in e.items() if k != "_at"} for e in s["entries"]], s["end"])
        row = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[e["id"]][e["_at"] + w] = out[row]
                row += 1
        assert row == out.shape[0]
        assert r.manager.check_invariants() == ""
    assert r.manager.num_free_blocks(0) == peak // bs             # everything was given back
    for rid, toks in reqs.items():
        check(np.stack(got[rid]), plain_logits(plain_models, name, toks, dtype), dtype, f"{name} mixed {rid}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_folders, plain_models, dtype):
    """300 tokens decoded one by one across many pages (and, in C and D, far past the window)."""
    for name in ["A", "C", "D"]:
        toks = tokens_for(name, 320, salt=9)
        want = plain_logits(plain_models, name, toks, dtype)
        r = runner(model_folders, name, dtype, 320)
        rows = [r.step([dict(id="x", tokens=toks[:20], want=[19])], [])[0]]
        for t in range(20, 320):
            rows.append(r.step([dict(id="x", tokens=[toks[t]], want=[0])], [])[0])
        check(np.stack(rows), want[19:], dtype, f"{name} long decode")
        if name == "C":     # the window group holds only what the window needs
            held = [b for b in r.manager.block_table(0, 1) if b >= 0]
            assert len(held) <= (24 + 16) // 16 + 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(model_folders, plain_models, name, dtype):
    toks = tokens_for(name, 4, salt=77)
    want = plain_logits(plain_models, name, toks, dtype)
    r = runner(model_folders, name, dtype, 64)
    rows = [r.step([dict(id="f", tokens=[t], want=[0])], [])[0] for t in toks]
    check(np.stack(rows), want, dtype, f"{name} first tokens one by one")
    r = runner(model_folders, name, dtype, 64)
    rows = r.step([dict(id="f", tokens=toks[:2], want=[0, 1])], [])
    rows = np.concatenate([rows, r.step([dict(id="f", tokens=toks[2:], want=[0, 1])], ["f"])])
    check(rows, want, dtype, f"{name} first tokens two by two")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_prefix_hits_start_on_another_requests_pages(model_folders, plain_models, name, dtype):
    """With the prefix cache on, a request whose first tokens another request has computed starts on that request's
    pages: while the other is live (shared pages, counted twice), after it has ended (pages taken back out of the free
    list), and not at all once the pages have been handed out again (stale hashes must not be found).  Every wanted
    row against the plain implementation of the request's own tokens.  C and D have layers with a window beside layers
    that keep all keys: their window group supplies the pages that a query after the hit still reads, some of which
    the first request has already given back."""
    from vllm_oxide_b200.engine.trace import TraceRunner
    bs = TINY[name]["block_size"]
    shared = tokens_for(name, 3 * bs + 5, salt=31)
    a = shared + tokens_for(name, 11, salt=32)
    b = shared[:3 * bs] + tokens_for(name, 2 * bs + 3, salt=33)
    c = shared[:2 * bs] + tokens_for(name, bs + 7, salt=34)
    d = tokens_for(name, 8 * bs, salt=35)                    # fills the whole pool: every page is handed out again
    pool = 8 * bs
    r = TraceRunner(model_folders[name], dtype, pool, bs, prefix_caching=True)
    assert r.manager.prefix_caching
    got = {}

    def step(entries, end, at):
        out = r.step(entries, end)
        row = 0
        for e, start in zip(entries, at):
            for w in e["want"]:
                got.setdefault(e["id"], {})[start + w] = out[row]
                row += 1
        assert row == out.shape[0] and r.manager.check_invariants() == ""

    step([dict(id="a", tokens=a[:-2], want=list(range(len(a) - 2)))], [], [0])
    assert r.prefix_hit_tokens == 0
    # b starts on a's first three pages while a is live
    step([dict(id="b", tokens=b[:-1], want=list(range(3 * bs, len(b) - 1)))], [], [0])
    assert r.prefix_hit_tokens == 3 * bs
    assert r.manager.block_table(r._ids["b"], 0)[:3] == r.manager.block_table(r._ids["a"], 0)[:3]
    assert all(r.manager.ref_count(0, p) == 2 for p in r.manager.block_table(r._ids["a"], 0)[:3])
    # both decode side by side over the shared pages
    step([dict(id="a", tokens=a[-2:-1], want=[0]), dict(id="b", tokens=b[-1:], want=[0])], ["a"], [len(a) - 2, len(b) - 1])
    step([dict(id="b", tokens=[a[-1]], want=[0])], ["b"], [len(b)])           # b goes on alone after a has ended
    b_full = b + [a[-1]]
    assert r.manager.num_free_blocks(0) == 8
    # c arrives after both have ended: two pages come back out of the free list
    step([dict(id="c", tokens=c, want=list(range(2 * bs, len(c))))], ["c"], [0])
    assert r.prefix_hit_tokens == 5 * bs
    # d takes every page of the pool; then the same tokens as a must be computed again, on pages that held d
    step([dict(id="d", tokens=d[:4 * bs], want=[]), ], [], [0])
    step([dict(id="d", tokens=d[4 * bs:], want=[4 * bs - 1])], ["d"], [4 * bs])
    hits = r.prefix_hit_tokens
    step([dict(id="a2", tokens=a, want=list(range(3 * bs, len(a))))], ["a2"], [0])
    assert r.prefix_hit_tokens == hits, "pages that were handed out again must not be found by their old hashes"
    assert r.manager.num_free_blocks(0) == 8
    for rid, toks in (("a", a[:-1]), ("b", b_full), ("c", c), ("d", d), ("a2", a)):
        want = plain_logits(plain_models, name, toks, dtype)
        places = sorted(got[rid])
        check(np.stack([got[rid][p] for p in places]), want[places], dtype, f"{name} prefix {rid}")
    assert sorted(got["b"]) == list(range(3 * bs, len(b_full)))


def test_the_program_itself(model_folders, plain_models, tmp_path):
    """bin/trace_run as a user calls it: steps on stdin, `done <step>` lines, <step>.f32 files."""
    name, dtype = "B", "float32"
    a, b = tokens_for(name, 40, salt=1), tokens_for(name, 21, salt=2)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:30], want=[29])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[30:31], want=[0]), dict(id="b", tokens=b[:20], want=[])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=b[20:], want=[0])], end=["b"]),
        dict(step=3, entries=[dict(id="a", tokens=a[31:], want=[0, 8])], end=["a"]),
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders[name],
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "128", "--block-size", "32"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    V = TINY[name]["config"]["vocab_size"]
    pa, pb = plain_logits(plain_models, name, a, dtype), plain_logits(plain_models, name, b, dtype)
    read = lambda i: np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
    check(read(0), pa[29:30], dtype, "step 0")
    check(read(1), pa[30:31], dtype, "step 1")
    check(read(2), pb[20:21], dtype, "step 2")
    check(read(3), pa[[31, 39]], dtype, "step 3")
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32", "3.f32"]


def test_the_program_step_by_step(model_folders, plain_models, tmp_path):
    """The next step is written only after `done <step>` of the one before has been read (a pipe, no end of input in
    between): the step's file is complete by then, in bfloat16, with the default pages of 64 tokens and a pool so small
    that the second request lands on the first one's pages."""
    name, dtype = "D", "bfloat16"
    a, b = tokens_for(name, 100, salt=11), tokens_for(name, 90, salt=12)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:64], want=[63])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[64:66], want=[1])], end=[]),
        dict(step=2, entries=[dict(id="a", tokens=a[66:], want=[0, 33])], end=["a"]),
        dict(step=3, entries=[dict(id="b", tokens=b[:89], want=[])], end=[]),
        dict(step=4, entries=[dict(id="b", tokens=b[89:], want=[0])], end=["b"]),
    ]
    out = tmp_path / "out"
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folders[name],
                             "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    V = TINY[name]["config"]["vocab_size"]
    pa, pb = plain_logits(plain_models, name, a, dtype), plain_logits(plain_models, name, b, dtype)
    expect = {0: pa[63:64], 1: pa[65:66], 2: pa[[66, 99]], 4: pb[89:90]}
    try:
        for s_ in steps:
            proc.stdin.write(json.dumps(s_) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            while line and not line.startswith("done"):
                line = proc.stdout.readline()          # lines of the first build, if any
            assert line.strip() == f"done {s_['step']}"
            if s_["step"] in expect:
                got = np.fromfile(out / f"{s_['step']}.f32", dtype="<f4").reshape(-1, V)
                check(got, expect[s_["step"]], dtype, f"step {s_['step']}")
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32", "4.f32"]


def test_running_out_of_pages_is_an_error_not_a_wrong_result(model_folders):
    r = runner(model_folders, "A", "float32", 32)
    r.step([dict(id="a", tokens=list(range(30)), want=[])], [])
    with pytest.raises(RuntimeError, match="no pages left"):
        r.step([dict(id="b", tokens=list(range(10)), want=[])], [])


def test_random_configurations_and_cuts(tmp_path):
    """Thirty configurations drawn at random (layers, widths and vocabularies that are no multiple of anything, head
    counts and groups, windows, eps, tied or not, page sizes; 64- and 128-wide heads in bfloat16, seven head sizes in
    32-bit), three requests each, cut at random into portions and single tokens that share steps: every position
    against the plain implementation."""
    from conftest import _cfg
    from vllm_oxide_b200.engine.loading import write_random_model_folder
    from vllm_oxide_b200.engine.trace import TraceRunner
    rng = random.Random(12)
    for case in range(30):
        dtype = rng.choice(DTYPES)
        hd = rng.choice([64, 128]) if dtype == "bfloat16" else rng.choice([16, 32, 48, 64, 80, 128, 144])
        kvh = rng.choice([1, 2, 3, 4])
        group = rng.choice([1, 2, 3, 4, 8] if hd <= 64 else [1, 2, 4])
        layers = rng.randint(1, 3)
        window = rng.choice([None, None, rng.randint(3, 70)])
        cfg = _cfg(num_hidden_layers=layers, hidden_size=rng.choice([8 * rng.randint(2, 40), 64 * rng.randint(1, 5), rng.randint(10, 300)]),
                   num_attention_heads=kvh * group, num_key_value_heads=kvh, head_dim=hd,
                   intermediate_size=rng.choice([8 * rng.randint(2, 60), 64 * rng.randint(1, 6), rng.randint(10, 500)]),
                   vocab_size=rng.randint(20, 1200), rope_theta=rng.choice([1e4, 5e5, 1e6]),
                   rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-4]), max_position_embeddings=512,
                   tie_word_embeddings=rng.random() < 0.5)
        if window:
            cfg.update(use_sliding_window=True, sliding_window=window, max_window_layers=rng.randint(0, layers))
        bs = rng.choice([16, 32, 64])
        folder = str(tmp_path / f"case{case}")
        os.makedirs(folder)
        write_random_model_folder(folder, cfg, case, "fan_in", torch.float32)
        plain_cfg, weights = P.read_folder(folder)
        lengths = [rng.randint(1, 160) for _ in range(3)]
        g = torch.Generator().manual_seed(case)
        reqs = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
        pool = sum((n + bs - 1) // bs * bs for n in lengths)
        r = TraceRunner(folder, dtype, pool, bs)
        pos, got = [0, 0, 0], [[], [], []]
        while any(p < n for p, n in zip(pos, lengths)):
            entries, ended = [], []
            for i in range(3):
                if pos[i] >= lengths[i] or rng.random() < 0.25:
                    continue                          # this request sits the step out
                m = min(rng.choice([1, 1, 2, 3, 17, bs, bs + 1, 40]), lengths[i] - pos[i])
                entries.append(dict(id=f"r{i}", tokens=reqs[i][pos[i]:pos[i] + m], want=list(range(m))))
                pos[i] += m
                if pos[i] >= lengths[i]:
                    ended.append(f"r{i}")
            if not entries:
                continue
            out, at = r.step(entries, ended), 0
            for e in entries:
                got[int(e["id"][1:])].append(out[at:at + len(e["tokens"])])
                at += len(e["tokens"])
        what = f"case {case}: {dtype}, pages of {bs}, {cfg}"
        for i, toks in enumerate(reqs):
            truth = P.forward_logits(plain_cfg, weights, toks, torch.float64).numpy()
            want = truth if dtype == "float32" else Both(truth, P.forward_logits(plain_cfg, weights, toks, torch.bfloat16).double().numpy())
            check(np.concatenate(got[i]), want, dtype, f"{what}, request of {len(toks)}")
        assert r.manager.check_invariants() == "", what
        assert all(r.manager.num_free_blocks(grp) == pool // bs for grp in range(r.manager.num_groups)), what
