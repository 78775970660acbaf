"""The engine's loop on the CPU: ``Engine.step`` / ``run`` / ``generate`` with the real scheduler and
cache manager, and a stand-in for the device (a stepper that "computes" the next token from the request's
whole history, a sampler that hands its ids through).  Whatever the loop does (a step started before the
last one's ids were read, portions, preemption and recompute), every request gets the tokens it would get
alone, the step log has one record per step, and every page comes back."""

import contextlib
import random
import types

import pytest
import torch

from pyre_b200.cache import CacheManager
from pyre_b200.config import EngineConfig
from pyre_b200.engine.engine import Engine
from pyre_b200.engine.scheduler import Scheduler
from pyre_b200.parts import PagedKVSpec
from pyre_b200.sampling import SamplingParams

VOCAB = 97


def next_token(history):
    return (sum((i + 1) * t for i, t in enumerate(history)) * 2654435761 >> 7) % VOCAB


def alone(prompt, params):
    out = []
    while len(out) < params.max_new_tokens:
        out.append(next_token(list(prompt) + out))
        if params.eos_id is not None and out[-1] == params.eos_id:
            break
    return out


class G:
    def __init__(self, spec, n_layers):
        self.spec, self.n_layers = spec, n_layers


class FakeStepper:
    """Keeps each request's tokens as the cache would hold them; the "logits" of a wanted place are
    the next token itself."""

    def __init__(self, cache):
        self.cache, self.history, self.steps = cache, {}, 0
        self.error_flag = torch.zeros(1, dtype=torch.int32)

    def step(self, entries, reserve=True, fed_from=None):
        assert not reserve                                   # the scheduler has reserved the pages
        out = []
        for e in entries:
            toks = list(e.tokens)
            if e.feed is not None:
                assert fed_from is not None and toks[-1] == 0
                toks[-1] = int(fed_from[e.feed])             # the id the step before sampled, never seen by the host
            assert all(0 <= t < VOCAB for t in toks)
            start = self.cache.length(e.request)
            hist = self.history.setdefault(e.request, [])
            del hist[start:]                                 # a preempted request starts again from nothing
            assert len(hist) == start
            hist += toks
            self.cache.commit(e.request, len(hist))
            assert list(e.want) in ([], [len(toks) - 1])
            if e.want:
                out.append(next_token(hist))
        self.steps += 1
        return torch.tensor(out, dtype=torch.int32)

    def check_device_errors(self):
        raise AssertionError("no error was raised")


class FakeSampler:
    def sample_async(self, logits, params, token_index):
        assert logits.shape[0] == len(params) == len(token_index)
        return types.SimpleNamespace(ids=logits)

    def read(self, ticket):
        return ticket.ids.tolist()


def make_engine(monkeypatch, num_pages, lookahead, page_size=4, max_num_seqs=4, budget=16, chunk=8, max_model_len=256):
    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())
    cache = CacheManager([G(PagedKVSpec(1, 16, None), 1)], [], page_size, num_pages, max_num_seqs, torch.float32, "cpu",
                         allocate=False)
    eng = object.__new__(Engine)
    eng.engine_config = EngineConfig(lookahead=lookahead, record_steps=True)
    eng.model = types.SimpleNamespace(device="cpu", vocab_size=VOCAB)
    eng.cache, eng.stepper, eng.sampler = cache, FakeStepper(cache), FakeSampler()
    eng.scheduler = Scheduler(cache, max_num_seqs, budget, chunk, max_model_len)
    eng.max_model_len = max_model_len
    eng._requests, eng._flight = {}, None
    eng._err_host, eng._err_turn = [torch.zeros(1, dtype=torch.int32) for _ in range(2)], 0
    eng.step_log = []
    return eng


@pytest.mark.parametrize("lookahead", [True, False])
@pytest.mark.parametrize("seed", range(4))
def test_generate_gives_each_request_what_it_gets_alone(monkeypatch, seed, lookahead):
    rnd = random.Random(seed)
    eng = make_engine(monkeypatch, num_pages=rnd.choice([10, 14, 40]), lookahead=lookahead,
                      budget=rnd.randint(6, 24), chunk=rnd.randint(2, 12))
    prompts = [[rnd.randrange(VOCAB) for _ in range(rnd.randint(1, 22))] for _ in range(rnd.randint(2, 9))]
    params = [SamplingParams(max_new_tokens=rnd.randint(1, 12), eos_id=rnd.choice([None, rnd.randrange(VOCAB)]))
              for _ in prompts]
    outs = eng.generate(prompts, params)
    for p, sp, o in zip(prompts, params, outs):
        if o.finish_reason == "cache_full":
            assert len(p) + sp.max_new_tokens > eng.cache.num_pages * eng.cache.page_size
            continue
        assert o.token_ids == alone(p, sp), (p, sp)
        assert o.finish_reason == ("eos" if sp.eos_id is not None and o.token_ids[-1] == sp.eos_id else "length")
        assert o.prompt_ids == p
    assert not eng.has_unfinished() and eng.step() == []
    eng.cache.check()
    assert eng.cache.live() == [] and eng.cache.stats().pages_free == [eng.cache.num_pages]
    # one record per step that ran, in order, and their tokens add up to what the scheduler planned
    log = eng.step_log
    assert [r["step"] for r in log] == list(range(len(log))) and len(log) == eng.stepper.steps == eng.scheduler.stats.steps
    assert sum(r["tokens"] for r in log) == eng.scheduler.stats.scheduled_tokens
    assert all(r["tokens"] <= eng.scheduler.max_num_batched_tokens and r["host_ms"] >= 0 for r in log)
    assert log[-1]["preempted_so_far"] == eng.scheduler.stats.preempted == sum(o.preemptions for o in outs)


def test_the_reference_s_two_calls(monkeypatch):
    """``add_request`` + ``run`` as in the reference (pyre/scheduler.py:40-44,105-114): ids by seq_id."""
    eng = make_engine(monkeypatch, num_pages=40, lookahead=True)
    a = eng.add_request([5, 17, 3], max_new_tokens=6)
    b = eng.add_request([9, 9], max_new_tokens=4, eos_id=next_token([9, 9]))
    with pytest.raises(ValueError, match="outside"):
        eng.add_request([5, VOCAB], max_new_tokens=2)
    with pytest.raises(ValueError, match="at least one prompt token"):
        eng.add_request([], max_new_tokens=2)
    results = eng.run()
    assert results == {a: alone([5, 17, 3], SamplingParams(max_new_tokens=6)), b: [next_token([9, 9])]}
    assert eng.stats()["finished"] == 2 and eng.stats()["pages_free"] == [40]


def test_a_raised_error_word_is_reported_when_the_step_is_read(monkeypatch):
    eng = make_engine(monkeypatch, num_pages=40, lookahead=True)

    def raise_it():
        raise RuntimeError("a kernel gave up")

    eng.stepper.check_device_errors = raise_it
    eng.add_request([1, 2, 3], max_new_tokens=4)
    eng.step()                                   # started, not yet read
    eng.stepper.error_flag[0] = 2                # a kernel of the next step raises the device's error word
    eng.step()                                   # reads the first step (clean), starts the second (copies the word)
    with pytest.raises(RuntimeError, match="gave up"):
        eng.step()                               # reads the second step: the word it carries is reported


def test_engine_options_are_checked_and_the_caller_s_configuration_is_left_alone(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)      # everything below ends before a device is touched
    ec = EngineConfig(dtype="float32")
    with pytest.raises(TypeError, match="unknown engine option 'pages'"):
        Engine("somewhere", ec, pages=3)
    with pytest.raises(ValueError, match="cache_memory_fraction"):
        Engine("somewhere", ec, cache_memory_fraction=1.5)
    with pytest.raises(ValueError, match="either a model folder or config"):
        Engine(None, ec, page_size=8)
    with pytest.raises(FileNotFoundError):
        Engine("/nonexistent/model/folder", ec, page_size=8, dtype="bfloat16")
    assert ec.page_size == 16 and ec.cache_memory_fraction is None and ec.dtype is torch.float32
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine("somewhere")
