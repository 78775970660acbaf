"""The scheduler's decisions on the CPU, with a fake step that "computes" the next token
as a function of the request's whole history: any scheduling (portions, mixing,
preemption and recompute) must give each request the same tokens as running it alone."""

from dataclasses import dataclass

import pytest
import torch

from pyre_b200.cache import CacheManager
from pyre_b200.engine.scheduler import PENDING, Scheduler
from pyre_b200.parts import PagedKVSpec
from pyre_b200.sampling import SamplingParams


@dataclass(frozen=True)
class G:
    spec: object
    n_layers: int


def make(num_pages, page_size=4, max_num_seqs=4, budget=16, chunk=8, max_model_len=256):
    cache = CacheManager([G(PagedKVSpec(1, 16, None), 1)], [], page_size, num_pages, max_num_seqs, torch.float32,
                         "cpu", allocate=False)
    return Scheduler(cache, max_num_seqs, budget, chunk, max_model_len), cache


def fake_token(history):
    return (sum((i + 1) * t for i, t in enumerate(history)) * 2654435761 >> 7) % 97


def drive(sched, cache, log=None, max_steps=10_000):
    """Run to the end; checks the plan of every step against the rules."""
    done = {}
    fed = {}      # seq_id -> tokens whose keys/values are "in the cache"
    for _ in range(max_steps):
        if not sched.has_unfinished():
            break
        plan = sched.schedule()
        if log is not None:
            log.append([(s.request.seq_id, s.start, s.count, s.samples) for s in plan])
        assert sum(s.count for s in plan) <= sched.max_num_batched_tokens
        assert len({s.request.seq_id for s in plan}) == len(plan)
        sampled = []
        for s in plan:
            r = s.request
            assert s.count <= sched.prefill_chunk and s.count >= 1
            assert cache.length(r.seq_id) == s.start                 # the step continues where the cache ends
            assert cache.reserved[r.seq_id] >= s.start + s.count     # and has its pages
            if s.start == 0:
                fed[r.seq_id] = []
            assert len(fed[r.seq_id]) == s.start
            fed[r.seq_id] += r.tokens(s.start, s.count)
            cache.commit(r.seq_id, s.start + s.count)
            assert s.samples == (s.start + s.count == r.cur_len)
            if s.samples:
                sampled.append(fake_token(fed[r.seq_id]))
        for r in sched.update(plan, sampled):
            done[r.seq_id] = r
        cache.check()
    assert not sched.has_unfinished(), "scheduler did not finish"
    return done


def alone(prompt, n, eos=None):
    h, out = list(prompt), []
    for _ in range(n):
        t = fake_token(h); out.append(t); h.append(t)
        if eos is not None and t == eos:
            break
    return out


def test_budget_portions_and_decode_first():
    sched, cache = make(num_pages=64, budget=10, chunk=6)
    a = sched.add_request(list(range(1, 14)), SamplingParams(max_new_tokens=3))     # 13 prompt tokens
    b = sched.add_request([5, 6, 7], SamplingParams(max_new_tokens=4))
    log = []
    done = drive(sched, cache, log)
    # step 0: a gets a portion of 6 (chunk), b its whole prompt of 3 (budget 10 allows it) and samples
    assert log[0] == [(a.seq_id, 0, 6, False), (b.seq_id, 0, 3, True)]
    # step 1: b decodes first (1 token), then a's next portion
    assert log[1] == [(b.seq_id, 3, 1, True), (a.seq_id, 6, 6, False)]
    # step 2: both have one token left to run (a's last prompt token, b's decode), oldest first
    assert log[2] == [(a.seq_id, 12, 1, True), (b.seq_id, 4, 1, True)]
    assert done[a.seq_id].generated == alone(range(1, 14), 3) and done[b.seq_id].generated == alone([5, 6, 7], 4)
    assert cache.stats().pages_free == [64] and not cache.live()
    assert done[a.seq_id].finish_reason == "length"


def test_max_num_seqs_and_fifo_admission():
    sched, cache = make(num_pages=64, max_num_seqs=2, budget=64, chunk=64)
    rs = [sched.add_request([i + 1, i + 2], SamplingParams(max_new_tokens=2 + i)) for i in range(4)]
    log = []
    done = drive(sched, cache, log)
    assert [e[0] for e in log[0]] == [0, 1]            # only two admitted
    first_seen = {}
    for n, step in enumerate(log):
        for e in step:
            first_seen.setdefault(e[0], n)
    assert first_seen[2] <= first_seen[3] and first_seen[2] > 0
    for i, r in enumerate(rs):
        assert done[r.seq_id].generated == alone([i + 1, i + 2], 2 + i)


def test_eos_is_kept_and_ends_the_request():
    prompt = [3, 1, 4, 1, 5]
    full = alone(prompt, 12)
    eos = full[4]
    sched, cache = make(num_pages=64)
    r = sched.add_request(prompt, SamplingParams(max_new_tokens=12, eos_id=eos))
    r2 = sched.add_request(prompt, SamplingParams(max_new_tokens=12, eos_id=eos, ignore_eos=True))
    done = drive(sched, cache)
    first = full.index(eos)
    assert done[r.seq_id].generated == full[:first + 1] and done[r.seq_id].finish_reason == "eos"
    assert done[r2.seq_id].generated == full and done[r2.seq_id].finish_reason == "length"


def test_pages_run_out_last_admitted_is_preempted_and_recomputed():
    # 6 pages of 4 tokens.  Two requests of 8 prompt tokens fill 4 pages; decoding 10 tokens each needs 10 pages.
    sched, cache = make(num_pages=6, page_size=4, budget=32, chunk=32)
    a = sched.add_request(list(range(10, 18)), SamplingParams(max_new_tokens=10))
    b = sched.add_request(list(range(20, 28)), SamplingParams(max_new_tokens=10))
    log = []
    done = drive(sched, cache, log)
    assert sched.stats.preempted >= 1
    assert done[b.seq_id].preemptions >= 1 and done[a.seq_id].preemptions == 0      # the one admitted last gives way
    assert done[a.seq_id].generated == alone(range(10, 18), 10)
    assert done[b.seq_id].generated == alone(range(20, 28), 10)                     # tokens survive the recompute
    # after the preemption b restarts from position 0 with prompt + generated tokens
    restarts = [e for step in log for e in step if e[0] == b.seq_id and e[1] == 0]
    assert len(restarts) >= 2 and restarts[1][2] > 8
    assert cache.stats().pages_free == [6]


def test_request_too_large_for_the_pool_ends_with_cache_full():
    sched, cache = make(num_pages=3, page_size=4, budget=64, chunk=64)
    big = sched.add_request(list(range(1, 11)), SamplingParams(max_new_tokens=50))     # needs > 12 tokens
    small = sched.add_request([1, 2], SamplingParams(max_new_tokens=2))
    huge = sched.add_request(list(range(1, 40)), SamplingParams(max_new_tokens=2))     # prompt alone exceeds the pool
    done = drive(sched, cache)
    assert done[big.seq_id].finish_reason == "cache_full" and len(done[big.seq_id].generated) >= 1
    assert done[big.seq_id].generated == alone(range(1, 11), 50)[:len(done[big.seq_id].generated)]
    assert done[small.seq_id].generated == alone([1, 2], 2)
    assert done[huge.seq_id].finish_reason == "cache_full" and done[huge.seq_id].generated == []
    assert cache.stats().pages_free == [3]


def test_max_model_len_and_prompt_checks():
    sched, cache = make(num_pages=64, max_model_len=10)
    r = sched.add_request([1, 2, 3, 4, 5, 6], SamplingParams(max_new_tokens=50))
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add_request(list(range(10)), SamplingParams())
    with pytest.raises(ValueError, match="at least one"):
        sched.add_request([], SamplingParams())
    done = drive(sched, cache)
    assert done[r.seq_id].finish_reason == "max_model_len" and done[r.seq_id].cur_len == 10


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_match_running_alone(seed):
    import random
    rnd = random.Random(seed)
    sched, cache = make(num_pages=rnd.randint(8, 20), page_size=rnd.choice([2, 4, 8]), max_num_seqs=rnd.randint(2, 4),
                        budget=rnd.randint(4, 24), chunk=rnd.randint(2, 12))
    cap = cache.num_pages * cache.page_size
    reqs = []
    for _ in range(10):
        prompt = [rnd.randint(0, 96) for _ in range(rnd.randint(1, 14))]
        n = rnd.randint(1, 12)
        reqs.append((sched.add_request(prompt, SamplingParams(max_new_tokens=n)), prompt, n))
    done = drive(sched, cache)
    for r, prompt, n in reqs:
        want = alone(prompt, n)
        got = done[r.seq_id]
        if got.finish_reason == "cache_full":
            assert len(prompt) + n > cap - cache.page_size and got.generated == want[:len(got.generated)]
        else:
            assert got.generated == want
    assert cache.stats().pages_free == [cache.num_pages]


def drive_lookahead(sched, cache, max_steps=10_000):
    """As ``drive``, but every step is planned and started before the tokens of the step before are
    known to the scheduler (they stand as PENDING); the fake device knows them, as the real one does."""
    done = {}
    fed = {}
    flight = None        # (plan, sampled) of the step whose tokens the scheduler has not seen yet
    for _ in range(max_steps):
        if not sched.has_unfinished() and flight is None:
            break
        plan = sched.schedule()
        started = None
        if plan:
            assert sum(s.count for s in plan) <= sched.max_num_batched_tokens
            sampled = []
            for s in plan:
                r = s.request
                assert cache.length(r.seq_id) == s.start and cache.reserved[r.seq_id] >= s.start + s.count
                toks = r.tokens(s.start, s.count)
                assert PENDING not in toks[:-1]                 # only the newest token may still be on the device
                if toks[-1] == PENDING:
                    assert flight is not None and r.pending == 1
                    toks[-1] = flight[1][r.feed_row]
                if s.start == 0:
                    fed[r.seq_id] = []
                assert len(fed[r.seq_id]) == s.start
                fed[r.seq_id] += toks
                cache.commit(r.seq_id, s.start + s.count)
                if s.samples:
                    sampled.append(fake_token(fed[r.seq_id]))
            sched.launched(plan)
            started = (plan, sampled)
        if flight is not None:
            for r in sched.resolve(*flight):
                done[r.seq_id] = r
        flight = started
        cache.check()
    assert not sched.has_unfinished() and flight is None, "scheduler did not finish"
    for r in done.values():
        assert r.pending == 0 and PENDING not in r.generated
    return done


@pytest.mark.parametrize("seed", range(8))
def test_lookahead_gives_the_same_tokens(seed):
    """One step in flight while the next is planned: same tokens as running alone, with ends of
    sequence (a token too many is computed and dropped), length limits, preemption and recompute."""
    import random
    rnd = random.Random(100 + seed)
    sched, cache = make(num_pages=rnd.randint(8, 20), page_size=rnd.choice([2, 4, 8]), max_num_seqs=rnd.randint(2, 4),
                        budget=rnd.randint(4, 24), chunk=rnd.randint(2, 12), max_model_len=rnd.choice([20, 256]))
    cap = cache.num_pages * cache.page_size
    reqs = []
    for _ in range(12):
        prompt = [rnd.randint(0, 96) for _ in range(rnd.randint(1, 14))]
        n = rnd.randint(1, 12)
        eos = rnd.choice([None, None] + alone(prompt, n)[:3])     # often a token that really comes up
        reqs.append((sched.add_request(prompt, SamplingParams(max_new_tokens=n, eos_id=eos)), prompt, n, eos))
    done = drive_lookahead(sched, cache)
    for r, prompt, n, eos in reqs:
        want = alone(prompt, n, eos)[:max(0, sched.max_model_len - len(prompt))]
        got = done[r.seq_id]
        if got.finish_reason == "cache_full":
            assert got.generated == want[:len(got.generated)]
        else:
            assert got.generated == want, (got.finish_reason, got.generated, want)
    assert cache.stats().pages_free == [cache.num_pages]


def test_a_prompt_is_admitted_only_if_it_will_fit_whole():
    """Beside running requests, a waiting request is admitted when the pools will hold its whole prompt after
    the running ones have finished theirs (and grown by a page each); admitting its first portion earlier only
    buys a preemption that throws the portion away.  Outputs are the same either way."""
    results = {}
    for whole in (True, False):
        sched, cache = make(num_pages=12, page_size=4, max_num_seqs=4, budget=16, chunk=8)    # 48 tokens of cache
        sched.admit_whole_prompts = whole
        prompts = [[3, 1, 4, 1, 5, 9, 2, 6] * 3, [2, 7, 1, 8, 2, 8, 1, 8] * 3, [1, 6, 1, 8, 0, 3, 3, 9] * 2]   # 24, 24, 16 tokens
        for p in prompts:
            sched.add_request(p, SamplingParams(max_new_tokens=2))
        log = []
        done = drive(sched, cache, log)
        for k, p in enumerate(prompts):
            assert done[k].generated == alone(p, 2)
        results[whole] = (sched.stats.preempted, sched.stats.scheduled_tokens, log)
        assert cache.stats().pages_free == [cache.num_pages]
    # 24 + 24 tokens fill the twelve pages: the second request does not fit whole beside the first, which still
    # has to grow; with the rule it waits (no preemption), without it its first portion is computed and thrown away
    assert results[True][0] == 0
    assert results[False][0] >= 1 and results[False][1] > results[True][1]
    first_start_of_second = next(n for n, step in enumerate(results[True][2]) if any(s[0] == 1 for s in step))
    assert first_start_of_second > 3      # not before the first request has made room by finishing


def test_step_record_tells_prompt_portions_from_decoded_tokens():
    from pyre_b200.engine.scheduler import step_record

    sched, cache = make(num_pages=64, budget=10, chunk=6)
    a = sched.add_request(list(range(1, 9)), SamplingParams(max_new_tokens=3))       # 8 tokens: portions of 6 and 2
    b = sched.add_request([5, 6, 7], SamplingParams(max_new_tokens=3))
    records = []
    for _ in range(4):
        plan = sched.schedule()
        for s in plan:
            cache.commit(s.request.seq_id, s.start + s.count)
        records.append(step_record(sched.stats.steps - 1, plan, cache, sched.stats, 0.0015))
        sched.update(plan, [fake_token(s.request.tokens(0, s.start + s.count)) for s in plan if s.samples])
    first, second, third = records[0], records[1], records[2]
    assert (first["step"], first["tokens"], first["requests"], first["prompt_tokens"], first["decoded_tokens"]) == (0, 9, 2, 9, 0)
    assert first["sampling"] == 1 and first["host_ms"] == 1.5 and first["preempted_so_far"] == 0
    assert first["pages_free"] == [64 - 2 - 1]                                        # 6 and 3 tokens in pages of 4
    assert (second["tokens"], second["prompt_tokens"], second["decoded_tokens"], second["sampling"]) == (3, 2, 1, 2)
    assert (third["tokens"], third["prompt_tokens"], third["decoded_tokens"]) == (2, 0, 2)
    assert a.seq_id != b.seq_id
