"""The cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""

from dataclasses import dataclass

import pytest
import torch
from hypothesis import given, settings, strategies as st

from pyre_b200.cache import CacheManager, OutOfPages, PageAllocator, pages_for
from pyre_b200.parts import PagedKVSpec, StateSpec


@dataclass(frozen=True)
class G:
    spec: object
    n_layers: int


def manager(num_pages=8, page_size=4, window=None, max_requests=4, state=False, two_groups=False, allocate=False):
    kv = [G(PagedKVSpec(2, 16, None), 2)]
    if two_groups or window:
        kv = [G(PagedKVSpec(2, 16, None), 2), G(PagedKVSpec(1, 32, window or 6), 1)] if two_groups else [G(PagedKVSpec(2, 16, window), 2)]
    stg = [G(StateSpec((3, 5)), 2)] if state else []
    return CacheManager(kv, stg, page_size, num_pages, max_requests, torch.float32, "cpu", allocate=allocate)


def test_allocator_contract():
    # pyre/paged_cache.py:40-92 and tests/test_paged_cache.py:23-66 of the reference
    a = PageAllocator(3)
    p = [a.allocate(), a.allocate(), a.allocate()]
    assert sorted(p) == [0, 1, 2] and a.num_free == 0 and a.num_used == 3
    with pytest.raises(OutOfPages):
        a.allocate()
    assert isinstance(OutOfPages("x"), MemoryError)
    a.free(p[1])
    assert a.allocate() == p[1]                      # the page freed last goes out first
    a.free(p[0])
    with pytest.raises(ValueError, match="double free"):
        a.free(p[0])
    with pytest.raises(ValueError):
        a.incref(p[0])
    a.incref(p[2])
    assert a.ref_count(p[2]) == 2
    assert a.free(p[2]) is False and a.free(p[2]) is True
    assert not a.can_allocate(3) and a.can_allocate(2)
    a.check()


def test_table_grows_by_pages_and_end_returns_all():
    m = manager(num_pages=8, page_size=4)
    m.begin("a"); m.begin("b")
    assert m.reserve("a", 5) and m.reserve("b", 4)
    assert len(m.groups[0].tables["a"]) == 2 and len(m.groups[0].tables["b"]) == 1
    assert not set(m.groups[0].tables["a"]) & set(m.groups[0].tables["b"])
    m.commit("a", 5); m.commit("b", 4)
    assert m.reserve("a", 8) and len(m.groups[0].tables["a"]) == 2      # still inside the second page
    assert m.reserve("a", 9) and len(m.groups[0].tables["a"]) == 3
    assert not m.reserve("b", 4 + 4 * 5)                               # 5 more pages, only 4 free: nothing is taken
    assert m.stats().pages_free == [4]
    with pytest.raises(ValueError, match="reserved"):
        m.commit("b", 9)
    with pytest.raises(ValueError, match="shrink"):
        m.reserve("a", 3)
    m.check()
    m.end("a"); m.end("b")
    assert m.stats().pages_free == [8] and m.stats().slots_free == 4
    with pytest.raises(ValueError, match="not live"):
        m.end("a")
    with pytest.raises(ValueError, match="already live"):
        m.begin("c"); m.begin("c")


def test_slots_and_block_table_views():
    m = manager(num_pages=8, page_size=4)
    m.begin("a"); m.reserve("a", 10)
    t = m.groups[0].tables["a"]
    s = m.slots_for(0, "a", 3, 4)
    assert s.tolist() == [t[0] * 4 + 3, t[1] * 4, t[1] * 4 + 1, t[1] * 4 + 2]
    m.begin("b"); m.reserve("b", 2)
    rows = m.block_table_rows(0, ["b", "a"])
    assert rows.shape == (2, 3) and rows[0].tolist() == [m.groups[0].tables["b"][0], -1, -1] and rows[1].tolist() == t


def test_window_gives_pages_back_when_passed():
    m = manager(num_pages=6, page_size=4, window=6)
    m.begin("a")
    held = []
    for n in range(1, 41):
        assert m.reserve("a", n), f"window of 6 needs at most 3 pages of 4, failed at {n}"
        m.commit("a", n)
        g = m.groups[0]
        # the next token (position n) reads keys n-5..n: every page that holds one of them must be live
        for pos in range(max(0, n - 5), n):
            assert g.tables["a"][pos // 4] >= 0
        held.append(g.pages_held("a"))
        m.check()
    assert max(held) <= 3 and m.groups[0].tables["a"][0] == -1
    with pytest.raises(RuntimeError, match="given back"):
        m.slots_for(0, "a", 0, 1)
    m.end("a")
    assert m.stats().pages_free == [6]


def test_groups_reserve_together_or_not_at_all():
    m = manager(num_pages=3, page_size=4, two_groups=True)
    m.begin("a")
    assert m.reserve("a", 12)
    m.commit("a", 12)                    # the windowed group (6) now holds pages 1..2 only
    assert m.stats().pages_free == [0, 1]
    m.begin("b")
    assert not m.reserve("b", 1)         # the full group is exhausted: the windowed group keeps its free page
    assert m.stats().pages_free == [0, 1]
    m.end("a")
    assert m.reserve("b", 1)
    m.check()


def test_state_slots_are_zeroed_and_bounded():
    m = manager(max_requests=2, state=True, allocate=True)
    m.begin("a")
    sa = m.state.slot_of["a"]
    m.state.buffers[0][:, sa] = 7.0
    m.begin("b")
    assert not m.has_free_slot()
    with pytest.raises(OutOfPages, match="state slots"):
        m.begin("c")
    m.end("a")
    m.begin("c")
    assert m.state.slot_of["c"] == sa and float(m.state.buffers[0][:, sa].abs().max()) == 0.0
    assert m.state.buffers[0].shape == (2, 2 + 1, 3, 5)      # the requests' slots and the scratch slot


@settings(max_examples=150, deadline=None)
@given(st.data())
def test_random_orders_keep_every_page_accounted(data):
    window = data.draw(st.sampled_from([None, 5, 16]))
    m = manager(num_pages=data.draw(st.integers(4, 12)), page_size=data.draw(st.sampled_from([2, 4, 8])),
                window=window, max_requests=4)
    next_id, live = 0, {}
    for _ in range(data.draw(st.integers(5, 60))):
        op = data.draw(st.sampled_from(["begin", "grow", "grow", "grow", "end"]))
        if op == "begin" and m.has_free_slot():
            m.begin(next_id); live[next_id] = 0; next_id += 1
        elif op == "grow" and live:
            r = data.draw(st.sampled_from(sorted(live)))
            new_len = live[r] + data.draw(st.integers(1, 9))
            free_before = m.stats().pages_free[0]
            if m.reserve(r, new_len):
                m.slots_for(0, r, live[r], new_len - live[r])       # every new position has a page
                m.commit(r, new_len); live[r] = new_len
            else:
                assert m.stats().pages_free[0] == free_before        # a refusal takes nothing
        elif op == "end" and live:
            r = data.draw(st.sampled_from(sorted(live)))
            m.end(r); del live[r]
        rows = m.block_table_rows(0, sorted(live))                   # rows are kept as arrays between changes: check() compares
        m.check()
        g = m.groups[0]
        for i, r in enumerate(sorted(live)):
            assert rows[i, :len(g.tables[r])].tolist() == g.tables[r]
        for r, n in live.items():
            if window is None:
                assert g.pages_held(r) == max(pages_for(n, m.page_size), len([p for p in g.tables[r] if p >= 0]))
            else:
                assert g.pages_held(r) <= pages_for(window + 8, m.page_size) + 2
    for r in list(live):
        m.end(r)
    assert m.stats().pages_free == [m.num_pages] and m.stats().slots_free == 4


def test_a_windowed_group_gets_a_pool_of_its_own_size():
    """Pages per group: the group that keeps every token gets the full count, the group with a window
    only what its window (plus a step's tokens) can hold per request.  Requests then grow far beyond
    the small pool's capacity in tokens without the windowed group ever running out."""
    from pyre_b200.cache import pages_per_group
    kv = [G(PagedKVSpec(2, 16, None), 2), G(PagedKVSpec(1, 32, 11), 1)]
    counts = pages_per_group(kv, page_size=4, full_pages=120, max_requests=3, step_tokens=8)
    assert counts == [120, 3 * (pages_for(11 - 1 + 8, 4) + 1)] == [120, 18]
    assert pages_per_group(kv, 4, 5, 3, 8) == [5, 5]                    # never more than the full group has
    m = CacheManager(kv, [], 4, counts, 3, torch.float32, "cpu", allocate=False)
    assert [g.num_pages for g in m.groups] == [120, 18] and m.stats().pages_total == [120, 18]
    for r in "abc":
        m.begin(r)
    length = {r: 0 for r in "abc"}
    while length["a"] < 150:
        for r in "abc":
            step = 8 if length[r] < 64 else 1                            # portions of a prompt, then decoding
            assert m.reserve(r, length[r] + step), f"request {r} at {length[r]}: a pool ran out"
            length[r] += step
            m.commit(r, length[r])
        m.check()
        assert m.groups[1].allocator.num_used <= 18
    assert m.groups[0].allocator.num_used == 3 * pages_for(length["a"], 4)
    with pytest.raises(ValueError, match="page counts"):
        CacheManager(kv, [], 4, [8], 3, torch.float32, "cpu", allocate=False)


def test_specs_say_what_they_cost():
    assert PagedKVSpec(4, 128, None).bytes_per_token(2) == 2 * 4 * 128 * 2
    assert PagedKVSpec(4, 128, None).tokens_held(2048) is None and PagedKVSpec(4, 128, 512).tokens_held(64) == 575
    assert StateSpec((3, 5), torch.float32).bytes_per_request() == 60 and StateSpec((8,), torch.bfloat16).bytes_per_request() == 16
