"""The scheduler's decisions, with a fake model: admission, token budget, portions, decoding,
finishing, and what happens when pages run out.

Cases follow the reference's (vllm-oxide, crates/vllm-oxide/src/engine/scheduler.rs:472-743:
small budgets force portions, max_num_seqs, decode after prefill, EOS / max_tokens / ignore_eos,
preemption with a tiny pool) and the engine loop with a mock model (crates/vllm-oxide/src/engine/mod.rs:295-443).
"""
import pytest

from vllm_oxide_b200 import host


def make(pages=16, bs=4, budget=100, max_seqs=8, max_len=256, eos=-1, prefix=False, window=0, slots=None):
    m = host.KvCacheManager([host.GroupSpec(bs, pages, window)], slots or max_seqs, prefix)
    return m, host.Scheduler(m, budget, max_seqs, max_len, eos)


def params(max_tokens=4, ignore_eos=False, temperature=0.0):
    p = host.SchedSamplingParams()
    p.max_tokens, p.ignore_eos, p.temperature = max_tokens, ignore_eos, temperature
    return p


def run(s, token=lambda seq_id, k: 100 + k, max_steps=10000, trace=None):
    """Drives the scheduler with a fake sampler; returns {id: generated tokens}."""
    done, count = {}, {}
    for _ in range(max_steps):
        if not s.has_unfinished():
            return done
        entries = s.schedule()
        assert entries, "an empty step while requests are unfinished"
        if trace is not None:
            trace.append([(e.id, e.start, e.n, e.wants_logits) for e in entries])
        sampled = []
        for e in entries:
            if e.wants_logits:
                k = s.sequence(e.id).num_generated
                sampled.append(token(e.id, k))
        for o in s.postprocess(sampled):
            done[o.id] = (list(o.token_ids), o.finish_reason)
    raise AssertionError("the scheduler did not finish")


def test_prompt_is_cut_under_the_budget_and_no_token_is_sampled_for_an_unfinished_portion():
    m, s = make(pages=64, budget=10)
    rid = s.add_request(list(range(25)), params(3))
    trace = []
    out = run(s, trace=trace)
    assert trace[0] == [(rid, 0, 10, False)] and trace[1] == [(rid, 10, 10, False)] and trace[2] == [(rid, 20, 5, True)]
    assert trace[3] == [(rid, 25, 1, True)] and len(trace) == 5
    assert out[rid] == ([100, 101, 102], "length")
    assert m.num_free_blocks(0) == 64 and m.check_invariants() == ""


def test_budget_covers_all_requests_and_decodes_go_first():
    m, s = make(pages=64, budget=12)
    a = s.add_request(list(range(8)), params(5))
    trace = []
    b = None
    steps = 0
    done = {}
    while s.has_unfinished():
        if steps == 1:
            b = s.add_request(list(range(30)), params(2))
        entries = s.schedule()
        trace.append([(e.id, e.start, e.n, e.wants_logits) for e in entries])
        assert sum(e.n for e in entries) <= 12
        for o in s.postprocess([7 for e in entries if e.wants_logits]):
            done[o.id] = list(o.token_ids)
        steps += 1
    assert trace[0] == [(a, 0, 8, True)]
    assert trace[1] == [(a, 8, 1, True), (b, 0, 11, False)]          # decode token first, the rest of the budget to b
    assert trace[2] == [(a, 9, 1, True), (b, 11, 11, False)]
    assert trace[3] == [(a, 10, 1, True), (b, 22, 8, True)]
    assert done[a] == [7] * 5 and done[b] == [7] * 2


def test_continuous_admission_and_max_num_seqs():
    m, s = make(pages=64, budget=100, max_seqs=2)
    ids = [s.add_request([1, 2, 3], params(2)) for _ in range(3)]
    first = s.schedule()
    assert [e.id for e in first] == ids[:2] and s.num_waiting == 1       # third waits for a free seat
    s.postprocess([5, 5])
    second = s.schedule()
    assert [e.id for e in second] == ids[:2]
    s.postprocess([5, 5])                                                 # both finish (max_tokens 2)
    third = s.schedule()
    assert [(e.id, e.start, e.n) for e in third] == [(ids[2], 0, 3)]


def test_eos_stops_unless_ignored():
    m, s = make(eos=42)
    a = s.add_request([1, 2], params(10))
    b = s.add_request([1, 2], params(3, ignore_eos=True))
    out = run(s, token=lambda rid, k: 42 if k == 1 else 9)
    assert out[a] == ([9, 42], "stop") and out[b] == ([9, 42, 9], "length")


def test_requests_that_can_never_fit_are_refused():
    m, s = make(pages=4, bs=4, max_len=64)
    with pytest.raises(RuntimeError, match="pages"):
        s.add_request(list(range(10)), params(8))       # 18 tokens need 5 pages
    with pytest.raises(RuntimeError, match="max_model_len"):
        s.add_request(list(range(60)), params(8))
    with pytest.raises(RuntimeError, match="empty"):
        s.add_request([], params(1))
    s.add_request(list(range(8)), params(8))            # exactly 4 pages: accepted


def test_out_of_pages_preempts_the_newest_and_recomputes_prompt_and_generated_tokens():
    m, s = make(pages=6, bs=4, budget=100)
    a = s.add_request(list(range(10)), params(12))      # grows to 22 tokens = 6 pages
    b = s.add_request(list(range(50, 57)), params(6))   # 7 + 6 = 13 tokens = 4 pages
    trace = []
    out = run(s, token=lambda rid, k: 1000 * (rid + 1) + k, trace=trace)
    assert out[a][0] == [1000 + k for k in range(12)] and out[b][0] == [2000 + k for k in range(6)]
    assert s.stats.preemptions >= 1
    # the step after b's preemption holds only a; when b comes back it is recomputed from position 0
    # over its prompt plus what it had generated, and then wants logits again
    back = [e for step in trace for e in step if e[0] == b and e[1] == 0]
    assert len(back) >= 2 and back[-1][2] > 7 and back[-1][3]
    assert m.num_free_blocks(0) == 6 and m.check_invariants() == ""


def test_no_admission_in_a_step_that_preempted():
    m, s = make(pages=5, bs=4, budget=100)
    a = s.add_request(list(range(8)), params(9))
    b = s.add_request(list(range(8)), params(2))
    s.schedule(); s.postprocess([1, 1])                 # both computed: 8 tokens each = 2 pages each, 1 page free
    entries = s.schedule()                              # a takes the last page; b finds none, is preempted, not re-admitted
    assert [(e.id, e.n) for e in entries] == [(a, 1)]
    assert s.waiting_ids() == [b] and s.running_ids() == [a]
    assert not m.has_request(b)


def test_prefix_cache_shortens_the_second_request():
    m, s = make(pages=32, bs=4, prefix=True)
    shared = list(range(200, 216))
    a = s.add_request(shared + [1, 2], params(1))
    run(s)
    b = s.add_request(shared + [3, 4, 5], params(1))
    entries = s.schedule()
    assert [(e.id, e.start, e.n) for e in entries] == [(b, 16, 3)]
    assert s.stats.prefix_hit_tokens == 16 and s.sequence(b).num_cached == 16
    s.postprocess([0])
    assert m.check_invariants() == ""


def test_window_group_frees_pages_during_decoding():
    m, s = make(pages=6, bs=4, window=6, max_len=200)
    # 6 pages can never hold 60 tokens at once; with the window they are handed back as decoding goes on
    with pytest.raises(RuntimeError, match="pages"):
        s.add_request(list(range(5)), params(55))
    m, s = make(pages=16, bs=4, window=6, max_len=200)
    a = s.add_request(list(range(5)), params(55))
    low = 16
    while s.has_unfinished():
        entries = s.schedule()
        s.postprocess([3 for e in entries if e.wants_logits])
        low = min(low, m.num_free_blocks(0))
    assert low >= 16 - 3 and m.num_free_blocks(0) == 16


def test_many_requests_tiny_pool_all_finish_with_their_own_tokens():
    m, s = make(pages=10, bs=4, budget=16, max_seqs=4, max_len=40)
    want = {}
    for i in range(12):
        rid = s.add_request(list(range(i + 1, i + 1 + (3 * i) % 11 + 1)), params(5 + i % 4))
        want[rid] = [rid * 100 + k for k in range(5 + i % 4)]
    out = run(s, token=lambda rid, k: rid * 100 + k)
    assert {k: v[0] for k, v in out.items()} == want
    assert m.num_free_blocks(0) == 10 and m.num_requests == 0 and m.check_invariants() == ""


def test_the_step_written_straight_from_the_sequences_equals_the_step_built_from_entries():
    """fill_batch (the scheduler writes the step's arrays from its sequences) against fill_step_batch over
    batch_entries(), array for array, over a run with portions, decodes and a preemption; the summary says what the
    step holds; the sampling settings and keys of the sampled rows are the ones sample_requests() reports."""
    import numpy as np
    from vllm_oxide_b200.sampling import row_key
    m, s = make(pages=10, bs=4, budget=9, max_seqs=4)
    for i, n in enumerate([13, 3, 7, 6]):
        p = params(6, temperature=0.5 * i)
        p.top_k, p.top_p, p.seed, p.own_seed = i, 1.0 - 0.1 * i, 1000 + i, i % 2 == 1
        s.add_request(list(range(10 * i, 10 * i + n)), p)
    steps = 0
    while s.has_unfinished():
        assert s.schedule_step() == len(s.last_entries())
        entries = s.batch_entries()
        summ = s.summary()
        assert summ.num_requests == len(entries) and summ.num_tokens == sum(len(e.tokens) for e in entries)
        assert summ.num_rows == sum(len(e.want) for e in entries) and summ.all_single == all(len(e.tokens) == 1 for e in entries)
        assert summ.max_pages == max(len(m.block_table(e.id, 0)) for e in entries)
        L = host.BatchLayout(summ.num_tokens + 3, summ.num_requests + 1, summ.num_rows + 2, 1, summ.max_pages)
        a, b = np.full(L.total, 77, np.int32), np.full(L.total, 88, np.int32)
        ca = s.fill_batch(L, a)
        cb = host.fill_step_batch(m, entries, L, b)
        fresh = slice(L.state_fresh, L.state_fresh + L.B)          # "fresh" is taken by whoever asks first
        a[fresh] = b[fresh] = 0
        assert np.array_equal(a, b)
        assert (ca.num_tokens, ca.num_requests, ca.num_rows, ca.num_decode, ca.max_q, ca.max_context) == \
               (cb.num_tokens, cb.num_requests, cb.num_rows, cb.num_decode, cb.max_q, cb.max_context)
        reqs = s.sample_requests()
        t, p_, k, keys = np.zeros(8, np.float32), np.zeros(8, np.float32), np.zeros(8, np.int32), np.zeros(8, np.uint64)
        rows, penalties = s.fill_sampling(t, p_, k, keys)
        assert rows == len(reqs) and not penalties
        for r, (rid, generated, temp, top_k, top_p, seed, _, key_id) in enumerate(reqs):
            assert (t[r], k[r]) == (np.float32(temp), top_k) and p_[r] == np.float32(top_p)
            assert int(keys[r]) == row_key(seed, key_id, generated) == s.row_key(seed, key_id, generated)
        s.postprocess([5] * rows)
        steps += 1
    assert s.stats.preemptions > 0 and s.stats.steps == steps
    assert s.stats.scheduled_requests >= steps and s.stats.sampled_rows == 4 * 6 and s.stats.context_tokens > 0
    with pytest.raises(RuntimeError, match="no request"):
        s.sequence(0)                                              # finished requests are forgotten
