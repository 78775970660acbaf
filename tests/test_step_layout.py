"""The flat batch that a step hands to the kernels, checked on the CPU: token rows, positions,
entry boundaries, wanted rows, where each token's keys go (slot mapping), the block tables of
every group, the state slots, and the rows with which a captured decode step is padded.  The
stepper is built without a device (no error word, no pinned staging); ``build_context`` with
``upload=False`` returns the host array and a factory that lays views over any int32 tensor."""

import random
import types

import pytest
import torch

from pyre_b200.cache import CacheManager, OutOfPages
from pyre_b200.engine.step import StepEntry, Stepper
from pyre_b200.parts import PagedKVSpec, StateSpec


class G:
    def __init__(self, spec, n_layers):
        self.spec, self.n_layers = spec, n_layers


def make_stepper(page_size=4, num_pages=32, max_requests=4, window=None, vocab=100, state=False):
    groups = [G(PagedKVSpec(2, 16, None), 2)]
    if window is not None:
        groups.append(G(PagedKVSpec(1, 32, window), 1))
    state_groups = [G(StateSpec((3,), torch.float32), 2)] if state else []
    cache = CacheManager(groups, state_groups, page_size, num_pages, max_requests, torch.float32, "cpu", allocate=False)
    st = object.__new__(Stepper)
    st.model = types.SimpleNamespace(vocab_size=vocab, dtype=torch.float32, device=torch.device("cpu"))
    st.cache, st.device, st.error_flag = cache, torch.device("cpu"), None
    return st, cache


def context(st, entries, **kw):
    make, flat = st.build_context(entries, upload=False, **kw)
    return make(torch.from_numpy(flat.copy())), flat


def test_mixed_step_layout():
    st, cache = make_stepper(page_size=4)
    for r in "abc":
        cache.begin(r)
    # "a" has 6 tokens cached, "b" 3, "c" none
    for r, n in (("a", 6), ("b", 3)):
        assert cache.reserve(r, n)
        cache.commit(r, n)
    entries = [StepEntry("a", [7], [0]), StepEntry("c", [1, 2, 3, 4, 5], [4]), StepEntry("b", [9, 8], [])]
    ctx, flat = context(st, entries)
    assert (ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows) == (8, 3, 2)
    assert ctx.token_ids.tolist() == [7, 1, 2, 3, 4, 5, 9, 8]
    assert ctx.positions.tolist() == [6, 0, 1, 2, 3, 4, 3, 4]
    assert ctx.seq_of_token.tolist() == [0, 1, 1, 1, 1, 1, 2, 2]
    assert ctx.cu_seqlens.tolist() == [0, 1, 6, 8]
    assert ctx.logit_rows.tolist() == [0, 5]
    assert ctx.start_pos_host.tolist() == [6, 0, 3] and ctx.max_context == 7 and ctx.max_new_tokens_per_seq == 5
    kv = ctx.kv_group(0)
    table = kv.block_table.tolist()
    ta, tc, tb = cache.groups[0].tables["a"], cache.groups[0].tables["c"], cache.groups[0].tables["b"]
    assert (len(ta), len(tc), len(tb)) == (2, 2, 2)            # 7, 5 and 5 tokens in pages of 4
    assert table[0][:2] == ta and table[1][:2] == tc and table[2][:2] == tb
    want = [ta[1] * 4 + 2] + [tc[p // 4] * 4 + p % 4 for p in range(5)] + [tb[p // 4] * 4 + p % 4 for p in (3, 4)]
    assert kv.slot_mapping.tolist() == want
    assert len(set(want)) == len(want)                         # no two tokens share a slot
    # every piece of the flat array starts on a 16-byte boundary
    for t in (ctx.token_ids, ctx.positions, ctx.seq_of_token, ctx.cu_seqlens, ctx.logit_rows, kv.slot_mapping, kv.block_table):
        assert t.storage_offset() % 4 == 0
    # nothing is committed by laying the step out
    assert cache.length("a") == 6 and cache.length("c") == 0


def test_entries_are_checked_before_anything_is_taken():
    st, cache = make_stepper(vocab=50)
    cache.begin("a")
    free = cache.stats().pages_free
    for bad, msg in [([StepEntry("a", [], [])], "at least one token"),
                     ([StepEntry("a", [50], [0])], "outside"),
                     ([StepEntry("a", [-1, 2], [0])], "outside"),
                     ([StepEntry("a", list(range(9)) + [77], [])], "outside"),
                     ([StepEntry("a", [1, 2], [2])], "wanted place"),
                     ([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])], "twice"),
                     ([], "at least one entry")]:
        with pytest.raises(ValueError, match=msg):
            st.build_context(bad, upload=False)
    with pytest.raises(KeyError):
        st.build_context([StepEntry("nobody", [1], [0])], upload=False)
    assert cache.stats().pages_free == free and cache.length("a") == 0


def test_out_of_pages_is_an_error_that_names_the_request():
    st, cache = make_stepper(page_size=4, num_pages=2)
    cache.begin("a")
    with pytest.raises(OutOfPages, match="'a'"):
        st.build_context([StepEntry("a", list(range(9)), [8])], upload=False)
    cache.check()


def test_window_group_has_its_own_pages_and_a_table_with_holes():
    st, cache = make_stepper(page_size=4, window=6)
    cache.begin("a")
    assert cache.reserve("a", 21)
    cache.commit("a", 21)                                       # the window group keeps keys 16.. only
    full, win = cache.groups
    assert win.tables["a"][:3] == [-1, -1, -1] and win.tables["a"][4] >= 0 and full.pages_held("a") == 6
    ctx, _ = context(st, [StepEntry("a", [5, 6], [1])])
    assert len(ctx.kv_groups) == 2 and ctx.kv_group(1).window == 6 and ctx.kv_group(0).window is None
    t0, t1 = ctx.kv_group(0).block_table.tolist()[0], ctx.kv_group(1).block_table.tolist()[0]
    assert all(p >= 0 for p in t0[:6]) and t1[:3] == [-1, -1, -1] and all(p >= 0 for p in t1[4:6])
    for g, group in enumerate(cache.groups):
        pages = group.tables["a"]
        assert ctx.kv_group(g).slot_mapping.tolist() == [pages[5] * 4 + 1, pages[5] * 4 + 2]
    cache.check()


def test_padded_decode_step_uses_scratch_page_and_slot():
    st, cache = make_stepper(page_size=4, window=6, state=True)
    lens = {"a": 5, "b": 9, "c": 1}
    for r, n in lens.items():
        cache.begin(r)
        assert cache.reserve(r, n)
        cache.commit(r, n)
    entries = [StepEntry(r, [10 + i], [0], feed=(i if r != "b" else None)) for i, r in enumerate(lens)]
    ctx, flat = context(st, entries, table_width=16, pad_to=8)
    assert (ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows) == (8, 8, 8)
    assert ctx.token_ids.tolist() == [10, 11, 12, 0, 0, 0, 0, 0]
    assert ctx.positions.tolist() == [5, 9, 1, 0, 0, 0, 0, 0]
    assert ctx.cu_seqlens.tolist() == list(range(9)) and ctx.logit_rows.tolist() == list(range(8))
    dst, src = ctx.feed_dst, ctx.feed_src
    assert dst.tolist() == [0, -1, 2, -1, -1, -1, -1, -1] and src.tolist()[:3] == [0, 0, 2]
    for g, group in enumerate(cache.groups):
        kv = ctx.kv_group(g)
        assert tuple(kv.block_table.shape) == (8, 16)
        assert kv.slot_mapping.tolist()[3:] == [group.scratch_page * 4] * 5
        assert (kv.block_table[3:] == group.scratch_page).all()
        assert group.scratch_page == group.num_pages             # beyond what the allocator hands out
        for b, (r, n) in enumerate(lens.items()):
            assert kv.slot_mapping[b].item() == group.tables[r][n // 4] * 4 + n % 4
    sv = ctx.state_group(0)
    assert sv.slots.tolist() == [cache.state.slot_of[r] for r in lens] + [cache.state.scratch_slot] * 5
    assert cache.state.scratch_slot == cache.state.max_requests
    # the shape of the flat array depends on (rows, table width) only: a captured step can be fed again
    for r, n in lens.items():
        cache.commit(r, n + 1)
    _, flat2 = context(st, [StepEntry(r, [3], [0]) for r in lens], table_width=16, pad_to=8)
    assert flat2.shape == flat.shape
    with pytest.raises(ValueError, match="single tokens"):
        st.build_context([StepEntry("a", [1, 2], [1])], upload=False, pad_to=4)


@pytest.mark.parametrize("seed", range(5))
def test_random_steps_write_every_position_once(seed):
    """Random portions of up to four live requests with few pages: over a request's life every
    position is written to exactly one slot of a page the request holds at that time, pages of ended
    requests come back, and no two live positions ever share a slot."""
    rnd = random.Random(seed)
    page = rnd.choice([2, 4, 8])
    st, cache = make_stepper(page_size=page, num_pages=24, window=rnd.choice([None, 5, 9]))
    live, owner_of_slot = {}, [{} for _ in cache.groups]
    next_id = 0
    for _ in range(200):
        while len(live) < 4 and rnd.random() < 0.5:
            cache.begin(next_id)
            live[next_id] = rnd.randint(3, 40)                   # tokens this request will bring in all
            next_id += 1
        entries = []
        for r in rnd.sample(sorted(live), k=rnd.randint(0, len(live))):
            left = live[r] - cache.length(r)
            n = min(left, rnd.choice([1, 1, 2, 3, 7]))
            if n > 0 and cache.can_reserve(r, cache.length(r) + n):
                entries.append(StepEntry(r, [rnd.randrange(100) for _ in range(n)], [n - 1]))
                assert cache.reserve(r, cache.length(r) + n)
        if entries:
            ctx, _ = context(st, entries, reserve=False)
            for g, group in enumerate(cache.groups):
                table = ctx.kv_group(g).block_table.tolist()
                for b, e in enumerate(entries):                      # the rows are the tables as they stand now
                    held = group.tables[e.request]
                    assert table[b][:len(held)] == held and all(p == -1 for p in table[b][len(held):])
                slots = ctx.kv_group(g).slot_mapping.tolist()
                pos = ctx.positions.tolist()
                seq = ctx.seq_of_token.tolist()
                for s, p, b in zip(slots, pos, seq):
                    r = entries[b].request
                    assert s // page == group.tables[r][p // page] and s % page == p % page
                    holder = owner_of_slot[g].get(s)
                    assert holder is None or holder[0] not in live or group.tables[holder[0]][holder[1] // page] != s // page, \
                        f"slot {s} of group {g} still belongs to {holder}"
                    owner_of_slot[g][s] = (r, p)
            for e in entries:
                cache.commit(e.request, cache.length(e.request) + len(e.tokens))
        for r in [r for r in live if cache.length(r) == live[r]]:
            cache.end(r)
            del live[r]
        cache.check()
    for r in list(live):
        cache.end(r)
    assert all(f == 24 for f in cache.stats().pages_free)


def test_step_runs_the_model_on_the_batch_and_commits_lengths(monkeypatch):
    """``Stepper.step`` end to end with a stand-in model and a host-side token feed: the model sees the
    context of the batch, fed tokens replace the stand-ins before it runs, lengths are committed after."""
    from pyre_b200.kernels import ops

    st, cache = make_stepper(page_size=4)
    seen = {}

    def forward(ctx):
        seen["tokens"], seen["rows"] = ctx.token_ids.tolist(), ctx.logit_rows.tolist()
        return torch.arange(ctx.num_logit_rows, dtype=torch.float32)[:, None]

    def feed_tokens(token_ids, dst, src, prev):
        for d, s in zip(dst.tolist(), src.tolist()):
            if d >= 0:
                token_ids[d] = prev[s]

    monkeypatch.setattr(ops, "feed_tokens", feed_tokens)
    st.model.forward = forward
    st.cuda_graphs, st.steps_run = False, 0
    st._staging = types.SimpleNamespace(upload=lambda flat: torch.from_numpy(flat.copy()))
    for r in "ab":
        cache.begin(r)
    st.step([StepEntry("a", [4, 5, 6], [2]), StepEntry("b", [7, 8], [])])
    assert seen == {"tokens": [4, 5, 6, 7, 8], "rows": [2]} and (cache.length("a"), cache.length("b")) == (3, 2)
    sampled = torch.tensor([41, 42], dtype=torch.int32)          # ids of the step before, "on the device"
    logits = st.step([StepEntry("b", [9, 0], [1], feed=1), StepEntry("a", [0], [0], feed=0)], fed_from=sampled)
    assert seen == {"tokens": [9, 42, 41], "rows": [1, 2]} and logits.shape == (2, 1)
    assert (cache.length("a"), cache.length("b")) == (4, 4) and st.steps_run == 2
    with pytest.raises(ValueError, match="sampled ids were not given"):
        st.step([StepEntry("a", [0], [0], feed=0)])
    cache.check()
