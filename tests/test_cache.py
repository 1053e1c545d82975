"""Cache manager (no GPU): pages, block tables, groups with a window, state slots."""
import random

import pytest
import torch

from tiny_llm_b200.cache import CacheManager, KVNeed, PageError, PagePool, StateNeed


def test_pool_hands_out_in_order_and_refuses_double_free():
    # the reference's own pool test: ids 0..9 in order, over-allocation and double free fail
    # (tests/runtime/test_page_pool.cpp:5-23)
    pool = PagePool(10)
    assert pool.allocate(10, "r") == list(range(10))
    assert pool.allocate(1, "r") is None and pool.num_free == 0
    pool.free([3, 4], "r")
    with pytest.raises(PageError, match="twice"):
        pool.free([3], "r")
    with pytest.raises(PageError, match="held by"):
        pool.free([5], "other")
    assert pool.allocate(2, "s") == [4, 3]  # LIFO: the page freed last comes back first
    pool.check()


def make(max_tokens=64, page=4, slots=3, window=None, layers=2):
    needs = [KVNeed(2, 16, window) for _ in range(layers)]
    return CacheManager(needs, max_tokens=max_tokens, page_size=page, max_slots=slots)


def test_one_table_per_request_serves_all_layers_of_a_group():
    m = make()
    assert len(m.groups) == 1 and m.groups[0].num_entries == 2
    assert [(r.group, r.entry) for r in m.refs] == [(0, 0), (0, 1)]
    assert m.add_request("a") == 0
    assert m.reserve("a", 9) and m.block_table(0, "a") == [0, 1, 2]
    m.commit("a", 9)
    assert m.reserve("a", 3) and len(m.block_table(0, "a")) == 3   # 12 tokens still fit 3 pages
    m.commit("a", 3)
    assert m.reserve("a", 1) and len(m.block_table(0, "a")) == 4
    m.commit("a", 1)
    m.free_request("a")
    assert m.groups[0].pool.num_free == 16
    m.check()


def test_reserve_takes_all_or_nothing_and_slots_run_out():
    m = make(max_tokens=16, page=4, slots=2)
    m.add_request("a"), m.add_request("b")
    assert m.add_request("c") is None
    assert m.reserve("a", 12)
    assert not m.reserve("b", 8) and m.block_table(0, "b") == []
    assert m.reserve("b", 4)
    with pytest.raises(PageError):
        m.add_request("a")
    m.commit("a", 12)
    with pytest.raises(PageError, match="commits"):
        m.commit("b", 5)
    m.free_request("a")
    with pytest.raises(PageError):
        m.free_request("a")
    m.check()


def test_groups_with_different_needs_have_pools_of_their_own():
    needs = [KVNeed(2, 16), KVNeed(2, 16, window=6), KVNeed(2, 16), StateNeed((3, 5)), None, KVNeed(1, 32)]
    m = CacheManager(needs, max_tokens=32, page_size=4, max_slots=2)
    assert len(m.groups) == 3
    assert [(r.group, r.entry, r.state) for r in m.refs] == [(0, 0, None), (1, 0, None), (0, 1, None),
                                                              (None, None, 0), (None, None, None), (2, 0, None)]
    m.allocate_storage(torch.float32, "cpu")
    assert m.groups[0].kv.shape == (2, 2, 8, 2, 4, 16) and m.groups[2].kv.shape == (1, 2, 8, 1, 4, 32)
    assert m.slots.tensors[0].shape == (2, 3, 5)
    m.add_request("a")
    assert m.reserve("a", 20)
    m.commit("a", 20)
    full, win = m.block_table(0, "a"), m.block_table(1, "a")
    assert full == [0, 1, 2, 3, 4]
    # next token is position 20 and sees keys 15..20: pages 0..2 (positions 0..11) are behind the window
    assert win == [-1, -1, -1, 3, 4] and m.groups[1].pool.num_free == 6
    assert m.reserve("a", 4)
    m.commit("a", 4)   # next position 24 sees 19..24: page 3 (12..15) is gone too
    assert m.block_table(1, "a")[:4] == [-1, -1, -1, -1] and m.groups[1].pool.num_used == 2
    m.check()
    m.free_request("a")
    assert all(g.pool.num_used == 0 for g in m.groups)


def test_state_slot_is_zeroed_when_handed_out():
    m = CacheManager([StateNeed((4,))], max_tokens=8, page_size=4, max_slots=2)
    m.allocate_storage(torch.float32, "cpu")
    s = m.add_request("a")
    m.slots.tensors[0][s] += 7.0
    m.free_request("a")
    s2 = m.add_request("b")
    assert s2 == s and float(m.slots.tensors[0][s2].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_lose_no_page(seed, window):
    rng = random.Random(seed)
    m = make(max_tokens=96, page=4, slots=4, window=window)
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{next_id}"
            next_id += 1
            assert m.add_request(rid) is not None
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            before = [g.pool.num_free for g in m.groups]
            if m.reserve(rid, n):
                m.commit(rid, n)
                live[rid] += n
                assert m.kv_len[rid] == live[rid]
                table = m.block_table(0, rid)
                held = [p for p in table if p >= 0]
                assert len(table) == -(-live[rid] // 4)
                if window is None:
                    assert len(held) == len(table)
                else:
                    first = max(0, live[rid] - window + 1) // 4
                    assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:])
            else:
                assert [g.pool.num_free for g in m.groups] == before   # nothing taken
        elif live:
            rid = rng.choice(sorted(live))
            m.free_request(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.free_request(rid)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups) and m.slots.num_free == 4
