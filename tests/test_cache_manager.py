"""The cache manager on the host: pages, block tables per group, windows, prefix hashes, state slots.

Cases restate the reference's (vllm-oxide, crates/vllm-oxide/src/engine/block_pool.rs:392-885,
crates/vllm-oxide/src/engine/kv_cache_manager.rs:190-339) with small pages, and add what the
reference does not have: groups with windows, state slots, random orders of requests.
"""
import random

import pytest

from vllm_oxide_b200 import host


def mgr(groups=((4, 8, 0),), slots=4, prefix=False):
    return host.KvCacheManager([host.GroupSpec(*g) for g in groups], slots, prefix)


def test_hash_vectors_and_chain():
    assert host.xxh64(b"", 0) == 0xEF46DB3751D8E999          # published test vectors of the algorithm
    assert host.xxh64(b"a", 0) == 0xD24EC4F1A98C6E5B
    assert host.xxh64(b"abc", 0) == 0x44BC2CF5AD770999
    long = bytes(range(100))
    assert host.xxh64(long, 0) != host.xxh64(long, 1)
    a = host.chain_hash(-1, [1, 2, 3, 4])
    assert a == host.chain_hash(-1, [1, 2, 3, 4])
    assert a != host.chain_hash(-1, [1, 2, 4, 3])              # order-sensitive (block_pool.rs tests)
    assert host.chain_hash(a, [5, 6, 7, 8]) != host.chain_hash(-1, [5, 6, 7, 8])   # prefix-sensitive
    import struct
    assert host.chain_hash(-1, [7, 9]) == struct.unpack("<q", struct.pack("<Q", host.xxh64(struct.pack("<II", 7, 9), 0)))[0]


def test_pool_order_and_double_free():
    p = host.BlockPool(3, 4)
    a, b = p.allocate(), p.allocate()
    assert (a, b) == (0, 1) and p.num_free == 1            # pages leave the front
    p.release(a)
    assert p.free_order() == [2, 0]                        # and come back at the back
    with pytest.raises(RuntimeError, match="freed twice"):
        p.release(a)
    p.retain(b)
    p.release(b)
    assert p.ref_count(b) == 1 and not p.is_free(b)        # shared page: 2 -> 1
    p.release(b)
    assert p.is_free(b)
    for _ in range(3):
        p.allocate()
    with pytest.raises(RuntimeError, match="out of pages"):
        p.allocate()


def test_slot_mapping_across_a_page_boundary():
    m = mgr()
    m.add_request(7)
    assert m.ensure(7, 0, 6)
    t = m.block_table(7, 0)
    assert len(t) == 2
    assert m.slot_mapping(7, 0, 2, 4) == [t[0] * 4 + 2, t[0] * 4 + 3, t[1] * 4 + 0, t[1] * 4 + 1]
    assert m.slot_mapping(7, 0, 6, 3) == [t[1] * 4 + 2, t[1] * 4 + 3, -1]    # no page: -1 (kv_cache_manager.rs:131)


def test_ensure_is_all_or_nothing_and_growth_by_one_page():
    m = mgr(((4, 3, 0),))
    m.add_request(1); m.add_request(2)
    assert m.ensure(1, 0, 8) and m.num_free_blocks(0) == 1
    assert not m.ensure(2, 0, 5) and m.num_free_blocks(0) == 1 and m.block_table(2, 0) == []
    assert m.ensure(1, 8, 1) and m.num_free_blocks(0) == 0      # ninth token needs a third page
    assert m.pages_needed(1, 9, 3) == [0] and m.pages_needed(1, 9, 4) == [1]
    m.free_request(1)
    assert m.num_free_blocks(0) == 3 and m.check_invariants() == ""


def test_pages_are_freed_last_first():
    m = mgr(((2, 4, 0),))
    m.add_request(1)
    m.ensure(1, 0, 6)
    t = list(m.block_table(1, 0))
    m.free_request(1)
    assert m.free_order(0) == [3] + t[::-1]                     # block_pool.rs:293-309


def test_window_group_gives_pages_back_as_the_window_passes():
    m = mgr(((4, 16, 0), (4, 16, 6)))
    m.add_request(1)
    assert m.ensure(1, 0, 10)
    m.advance(1, 10)      # next query at 10 reads positions > 4: page 0 (0..3) is gone, page 1 (4..7) stays
    assert m.block_table(1, 0) == [0, 1, 2]
    assert m.block_table(1, 1) == [-1, 1, 2] and m.num_free_blocks(1) == 14
    for pos in range(10, 30):
        assert m.ensure(1, pos, 1)
        m.advance(1, pos + 1)
        held = [b for b in m.block_table(1, 1) if b >= 0]
        assert len(held) <= 3                                    # ceil((6 + 4) / 4)
        first_needed = pos + 1 - 6 + 1
        assert all(b >= 0 for i, b in enumerate(m.block_table(1, 1)) if (i + 1) * 4 > first_needed and i * 4 <= pos)
        assert m.check_invariants() == ""
    assert len([b for b in m.block_table(1, 0) if b >= 0]) == 8  # the all-keys group keeps everything
    m.free_request(1)
    assert m.num_free_blocks(0) == 16 and m.num_free_blocks(1) == 16 and m.check_invariants() == ""


def test_a_large_portion_holds_all_its_pages_at_once_in_a_window_group():
    m = mgr(((4, 8, 5),))
    m.add_request(1)
    assert m.ensure(1, 0, 30) and m.num_free_blocks(0) == 0
    m.advance(1, 30)
    assert [b >= 0 for b in m.block_table(1, 0)] == [False] * 6 + [True, True]


def test_prefix_cache_hits_share_full_pages_but_never_the_last():
    m = mgr(((4, 8, 0),), prefix=True)
    toks = list(range(100, 112))
    m.add_request(1)
    assert m.lookup_prefix(1, toks) == 0
    m.ensure(1, 0, 12)
    m.commit(1, toks, 12)
    t1 = list(m.block_table(1, 0))
    m.add_request(2)
    assert m.lookup_prefix(2, toks) == 8            # 3 full pages, the last is never taken (block_pool.rs:198-227)
    assert m.block_table(2, 0) == t1[:2] and m.ref_count(0, t1[0]) == 2
    assert m.ensure(2, 8, 4) and m.block_table(2, 0)[2] != t1[2]
    m.add_request(3)
    assert m.lookup_prefix(3, toks[:4] + [9, 9, 9, 9, 1]) == 4     # stops at the first miss
    m.free_request(1); m.free_request(2); m.free_request(3)
    assert m.num_free_blocks(0) == 8 and m.check_invariants() == ""
    m.add_request(4)
    assert m.lookup_prefix(4, toks + [1]) == 12     # freed pages stay discoverable until they are reused
    assert m.num_free_blocks(0) == 5
    m.free_request(4)
    m.add_request(5)
    m.ensure(5, 0, 32)                               # takes every page: the old contents are forgotten
    m.free_request(5)
    m.add_request(6)
    assert m.lookup_prefix(6, toks + [1]) == 0
    m.free_request(6)


def test_what_could_be_restored_is_a_question_that_takes_nothing():
    """`restorable_tokens` answers what `lookup_prefix` would give a new request, and leaves every count as it was;
    with a window group (prefix caching off) nothing can be restored."""
    m = mgr(((4, 8, 0), (4, 8, 0)), prefix=True)
    toks = list(range(200, 214))
    assert m.restorable_tokens(toks) == 0
    m.add_request(1)
    m.ensure(1, 0, 14)
    m.commit(1, toks, 14)
    free = (m.num_free_blocks(0), m.num_free_blocks(1))
    page = m.block_table(1, 0)[0]
    assert m.restorable_tokens(toks) == 12 and m.restorable_tokens(toks[:12]) == 8     # never the page of the last token
    assert m.restorable_tokens(toks[:4] + [1, 2, 3, 4, 5]) == 4 and m.restorable_tokens([7] + toks) == 0
    assert (m.num_free_blocks(0), m.num_free_blocks(1)) == free and m.ref_count(0, page) == 1
    m.add_request(2)
    assert m.lookup_prefix(2, toks) == 12            # the same answer, and now the pages are taken
    m.free_request(1); m.free_request(2)
    assert m.restorable_tokens(toks) == 12 and m.check_invariants() == ""
    u = mgr(((4, 8, 0), (8, 8, 0)), prefix=True)     # pages of two sizes: no hits
    u.add_request(1)
    u.ensure(1, 0, 14)
    u.commit(1, toks, 14)
    assert u.restorable_tokens(toks) == 0


def test_prefix_cache_is_off_with_pages_of_two_sizes():
    assert not mgr(((4, 8, 0), (8, 8, 0)), prefix=True).prefix_caching
    assert mgr(((4, 8, 0), (4, 9, 0)), prefix=True).prefix_caching
    assert mgr(((4, 8, 0), (4, 8, 6)), prefix=True).prefix_caching


def test_a_prefix_hit_in_a_window_group_takes_only_the_pages_a_later_query_reads():
    """Pages of 4, a group that keeps all keys and one with a window of 6.  After 14 tokens the window group has given
    pages 0 and 1 back, but a freed page stays discoverable until it is used again; a new request with the same
    tokens takes pages 0..2 of the first group and, of the window group, pages 1 and 2 (a query at position 12 reads
    keys 7..11), leaving entry 0 empty.  Once the window group's old pages have been overwritten, the hit shrinks to
    what every group can still supply."""
    m = mgr(((4, 16, 0), (4, 6, 6)), prefix=True)
    toks = list(range(300, 314))
    m.add_request(1)
    m.ensure(1, 0, 14)
    m.commit(1, toks, 14)
    m.advance(1, 14)
    t_full, t_win = list(m.block_table(1, 0)), list(m.block_table(1, 1))
    assert [b >= 0 for b in t_win] == [False, False, True, True]
    first_pages = [m.slot_mapping(1, 1, 8, 1)[0] // 4]                     # the window group's page of positions 8..11
    assert m.restorable_tokens(toks) == 12
    m.add_request(2)
    assert m.lookup_prefix(2, toks) == 12
    assert m.block_table(2, 0) == t_full[:3]
    w2 = m.block_table(2, 1)
    assert w2[0] == -1 and w2[1] >= 0 and w2[2] == first_pages[0] and m.ref_count(1, w2[2]) == 2
    assert m.ensure(2, 12, 2)
    m.commit(2, toks, 14)
    m.advance(2, 14)                                                      # starts releasing where the hit began
    assert [b >= 0 for b in m.block_table(2, 1)] == [False, False, True, True] and m.check_invariants() == ""
    m.free_request(1); m.free_request(2)
    assert m.num_free_blocks(1) == 6 and m.restorable_tokens(toks) == 12   # still discoverable
    m.add_request(3)
    assert m.ensure(3, 0, 24)                                             # takes all six pages of the window group
    m.free_request(3)
    assert m.restorable_tokens(toks) == 0 and m.check_invariants() == ""
    # a window as long as the prefix: the window group needs every page too
    k = mgr(((4, 16, 0), (4, 16, 40)), prefix=True)
    k.add_request(1)
    k.ensure(1, 0, 14)
    k.commit(1, toks, 14)
    k.add_request(2)
    assert k.lookup_prefix(2, toks) == 12 and all(b >= 0 for b in k.block_table(2, 1))


def test_state_slots():
    m = mgr(slots=2)
    assert m.add_request(1) and m.add_request(2)
    assert not m.add_request(3) and not m.has_request(3)
    assert {m.state_slot(1), m.state_slot(2)} == {0, 1}
    s = m.state_slot(1)
    m.free_request(1)
    assert m.add_request(3) and m.state_slot(3) == s
    with pytest.raises(RuntimeError, match="already live"):
        m.add_request(3)
    with pytest.raises(RuntimeError, match="no live request"):
        m.free_request(1)
    assert m.check_invariants() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Requests arrive, grow in portions of random size, are preempted or end, in random order:
    no page is lost, held twice or freed twice, and slot maps of live requests never collide."""
    rng = random.Random(seed)
    groups = ((4, 24, 0), (4, 24, 9)) if seed % 2 else ((8, 20, 0),)
    m = mgr(groups, slots=5, prefix=(seed % 2 == 0 or seed >= 3))        # seeds 3 and 5: hits in a window group too

    def readable(rid, done):
        """Every position that a query at position `done` reads has a page, in every group."""
        for g in range(m.num_groups):
            w = m.group(g).window
            lo = max(0, done - w + 1) if w > 0 else 0
            if done > lo:
                assert all(s >= 0 for s in m.slot_mapping(rid, g, lo, done - lo)), (rid, g, lo, done)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            if m.add_request(next_id):
                toks = [rng.randrange(6) for _ in range(rng.randrange(1, 70))]
                live[next_id] = dict(tokens=toks, done=m.lookup_prefix(next_id, toks))
                assert live[next_id]["done"] < len(toks)
                readable(next_id, live[next_id]["done"])
                next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            r = live[rid]
            left = len(r["tokens"]) - r["done"]
            if left == 0:
                r["tokens"].append(rng.randrange(6)); left = 1
            n = rng.randrange(1, left + 1)
            if m.ensure(rid, r["done"], n):
                slots = m.slot_mapping(rid, 0, r["done"], n)
                assert all(s >= 0 for s in slots)
                r["done"] += n
                m.commit(rid, r["tokens"], r["done"])
                m.advance(rid, r["done"])
                readable(rid, r["done"])
        elif op < 0.9 and live:
            rid = rng.choice(list(live))
            m.release_pages(rid)                      # preempted: pages back, request stays
            live[rid]["done"] = m.lookup_prefix(rid, live[rid]["tokens"])
            readable(rid, live[rid]["done"])
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        assert m.check_invariants() == ""
        if not m.prefix_caching:
            for g in range(m.num_groups):
                held = [b for rid in live for b in m.block_table(rid, g) if b >= 0]
                assert len(held) == len(set(held))
                assert len(held) + m.num_free_blocks(g) == m.group(g).num_blocks
    for rid in list(live):
        m.free_request(rid)
    for g in range(m.num_groups):
        assert m.num_free_blocks(g) == m.group(g).num_blocks
    assert m.num_free_state_slots == 5 and m.check_invariants() == ""


def test_batch_builder_layout_and_padding():
    import numpy as np
    m = mgr(((4, 8, 0), (4, 8, 6)))
    m.add_request(1); m.add_request(2)
    m.ensure(1, 0, 5); m.ensure(2, 0, 1)
    L = host.BatchLayout(8, 3, 4, 2, 3)
    buf = np.full(L.total, 12345, dtype=np.int32)
    c = host.fill_step_batch(m, [host.BatchEntry(1, 0, [9, 8, 7, 6, 5], [4, 0]), host.BatchEntry(2, 0, [3], [0])], L, buf)
    assert (c.num_tokens, c.num_requests, c.num_rows, c.num_decode, c.max_q, c.max_context) == (6, 2, 3, 1, 5, 5)
    assert buf[L.token_ids:L.token_ids + 8].tolist() == [9, 8, 7, 6, 5, 3, 0, 0]
    assert buf[L.positions:L.positions + 6].tolist() == [0, 1, 2, 3, 4, 0]
    assert buf[L.token_req:L.token_req + 8].tolist() == [0, 0, 0, 0, 0, 1, -1, -1]
    assert buf[L.cu_q:L.cu_q + 4].tolist() == [0, 5, 6, 6]
    assert buf[L.context_lens:L.context_lens + 3].tolist() == [5, 1, 0]
    assert buf[L.logit_rows:L.logit_rows + 3].tolist() == [4, 0, 5]
    sm1 = buf[L.slot_mapping + 8:L.slot_mapping + 16].tolist()
    assert sm1[:6] == m.slot_mapping(1, 1, 0, 5) + m.slot_mapping(2, 1, 0, 1) and sm1[6:] == [-1, -1]
    bt = buf[L.block_tables:L.block_tables + 2 * 3 * 3].reshape(2, 3, 3)
    assert bt[0, 0, :2].tolist() == m.block_table(1, 0) and bt[0, 0, 2] == -1 and (bt[:, 2] == -1).all()
    assert buf[L.state_fresh:L.state_fresh + 2].tolist() == [1, 1]
    host.fill_step_batch(m, [host.BatchEntry(2, 0, [3], [])], L, buf)
    assert buf[L.state_fresh] == 0                               # fresh only once
    with pytest.raises(RuntimeError, match="no page"):
        host.fill_step_batch(m, [host.BatchEntry(2, 1, [3, 4, 5, 6], [])], L, buf)
    with pytest.raises(RuntimeError, match="exceeds"):
        host.fill_step_batch(m, [host.BatchEntry(1, 0, list(range(9)), [])], L, buf)
    with pytest.raises(RuntimeError, match="outside the portion"):
        host.fill_step_batch(m, [host.BatchEntry(2, 0, [3], [1])], L, buf)
