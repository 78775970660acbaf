"""Continuous batching above the step function: which tokens of which requests run next.

Host logic only; it talks to a ``CacheManager`` and returns a plan, so it is tested on
the CPU with a fake step.  What the reference does (pyre/scheduler.py:27-114): a FIFO
``waiting`` list, a ``running`` list bounded by ``max_batch``, each admitted request
prefilled alone and whole, then one decode step per iteration for all running requests,
no look at free pages (exhaustion is a MemoryError that ends ``run``).  Here:

* every iteration is ONE mixed step under a token budget: first one token for every
  request that is decoding, then portions of prompts (at most ``prefill_chunk`` tokens of
  a request) while budget is left, oldest request first;
* a request is admitted when a state slot is free, its first portion fits in the pools and, beside running
  requests, the pools will hold its WHOLE prompt once the running ones have finished theirs and grown by a page
  each (``admit_whole_prompts``; with a cache of 40 % of what 64 requests need at once, this turns 171
  preemptions and 3.4 times the work into 4 preemptions and 6 % more work);
* when pages run out for a request that is already running, the request admitted LAST
  is preempted: its pages and slot go back, it returns to the FRONT of the waiting list
  and later recomputes prompt + tokens generated so far in portions; tokens already
  produced are kept, and the sampler's noise is keyed by token index, so the final output
  is what it would have been;
* a request that cannot grow even when it is alone in the cache ends with reason
  ``"cache_full"``;
* the token that completes a request (end-of-sequence id or the last allowed token) is
  kept (pyre/scheduler.py:82), and a finished request takes part in no further step
  (the reference lets a request that finishes at admission decode once more).

A step may be planned while the tokens of the step before are still on the device:
``launched`` records a step that has been started (its sampled tokens stand in the requests
as ``PENDING``), ``resolve`` fills in the values when they have arrived.  ``update`` is the
two in a row.  With one step in flight a request may run one token past its end-of-sequence
token; that token is dropped when it arrives.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from ..cache import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1     # a token that has been sampled on the device and not yet been read back


@dataclass
class Request:
    seq_id: int
    prompt_ids: list[int]
    params: SamplingParams
    generated: list[int] = field(default_factory=list)
    status: str = WAITING
    num_computed: int = 0          # tokens whose keys and values are in the cache
    finish_reason: "str | None" = None
    preemptions: int = 0
    pending: int = 0               # steps in flight that will deliver a token of this request
    closed: bool = False           # the tokens in flight complete it by length: nothing more is asked for
    feed_row: int = -1             # row of its newest pending token among the ids of the step in flight
    logits: dict = field(default_factory=dict)   # index of a generated token -> the logits it was chosen from (if asked for)

    @property
    def cur_len(self) -> int:
        return len(self.prompt_ids) + len(self.generated)

    @property
    def done(self) -> bool:
        return self.status == FINISHED

    def token_at(self, i: int) -> int:
        n = len(self.prompt_ids)
        return self.prompt_ids[i] if i < n else self.generated[i - n]

    def tokens(self, start: int, count: int) -> list[int]:
        """A new list of the tokens at positions start .. start + count - 1 (prompt, then generated)."""
        n, end = len(self.prompt_ids), start + count
        if end <= n:
            return self.prompt_ids[start:end]
        if start >= n:
            return self.generated[start - n:end - n]
        return self.prompt_ids[start:] + self.generated[:end - n]


@dataclass
class Scheduled:
    """One entry of the next step: ``count`` tokens of ``request`` from ``start``; the step's
    last token completes what is known of the request iff ``samples``."""

    request: Request
    start: int
    count: int
    samples: bool
    slot: int = -1                 # index in ``request.generated`` of the token this entry samples (set by ``launched``)


@dataclass
class SchedulerStats:
    steps: int = 0
    admitted: int = 0
    preempted: int = 0
    finished: int = 0
    scheduled_tokens: int = 0


def step_record(index: int, plan: "Sequence[Scheduled]", cache: CacheManager, stats: SchedulerStats,
                host_seconds: float) -> dict:
    """What one step did, for a log of a run: its tokens and requests (prompt portions and decoded tokens apart),
    how many of its entries sample, the pages left in every group afterwards, the preemptions so far, and the
    host's time in the call.  The reference records only totals per run (bench/harness.py:84-135)."""
    decoded = sum(1 for s in plan if s.count == 1 and s.samples and s.start >= len(s.request.prompt_ids))
    return {"step": index, "tokens": sum(s.count for s in plan), "requests": len(plan), "decoded_tokens": decoded,
            "prompt_tokens": sum(s.count for s in plan) - decoded, "sampling": sum(1 for s in plan if s.samples),
            "pages_free": list(cache.stats().pages_free), "preempted_so_far": stats.preempted,
            "host_ms": round(host_seconds * 1e3, 3)}


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk: int, max_model_len: int, admit_whole_prompts: bool = True):
        self.cache = cache
        self.admit_whole_prompts = admit_whole_prompts
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk = prefill_chunk
        self.max_model_len = max_model_len
        self.waiting: list[Request] = []
        self.running: list[Request] = []     # in order of admission
        self._next_seq = 0
        self._finished_now: list[Request] = []
        self.stats = SchedulerStats()

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], params: SamplingParams) -> Request:
        prompt = [int(t) for t in prompt_ids]
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(prompt) >= self.max_model_len:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room under max_model_len {self.max_model_len}")
        r = Request(self._next_seq, prompt, params)
        self._next_seq += 1
        self.waiting.append(r)
        return r

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def _preempt(self, victim: Request) -> None:
        self.cache.end(victim.seq_id)
        self.running.remove(victim)
        victim.status = WAITING
        victim.num_computed = 0
        victim.preemptions += 1
        self.waiting.insert(0, victim)
        self.stats.preempted += 1

    def _finish(self, r: Request, reason: str) -> None:
        if r.status == RUNNING:
            self.cache.end(r.seq_id)
            self.running.remove(r)
        elif r in self.waiting:
            self.waiting.remove(r)    # preempted, and the token that was in flight meanwhile ends it
        r.status = FINISHED
        r.finish_reason = reason
        self.stats.finished += 1
        self._finished_now.append(r)

    def schedule(self) -> list[Scheduled]:
        """Plan the next step and reserve its pages.  May preempt or finish requests
        (see the module text); returns [] only if nothing is left to run."""
        budget = self.max_num_batched_tokens
        plan: list[Scheduled] = []
        planned: set[int] = set()
        aborted: list[Request] = []

        def try_schedule(r: Request) -> bool:
            nonlocal budget
            remaining = r.cur_len - r.num_computed
            count = min(remaining, self.prefill_chunk, budget)
            if count <= 0:
                return False
            while not self.cache.reserve(r.seq_id, r.num_computed + count):
                # the most recently admitted request that is not yet in this step's plan gives way
                victims = [v for v in reversed(self.running) if v.seq_id not in planned]
                victim = victims[0] if victims else None
                if victim is None or victim is r:
                    if len(self.running) == 1 and victim is r:
                        aborted.append(r)   # alone and still too large for the pools
                    elif victim is r:
                        self._preempt(r)
                    return False
                self._preempt(victim)
            plan.append(Scheduled(r, r.num_computed, count, r.num_computed + count == r.cur_len))
            planned.add(r.seq_id)
            budget -= count
            return True

        decoding, in_prompt = [], []
        for r in self.running:
            if not r.closed:
                left = r.cur_len - r.num_computed
                if left == 1:
                    decoding.append(r)
                elif left > 1:
                    in_prompt.append(r)
        # 1. requests that are decoding (one token each), oldest first
        for r in decoding:
            if r.status == RUNNING and budget > 0:
                try_schedule(r)
        # 2. requests in the middle of their prompt (or of a recompute); one that step 1 preempted is no longer running
        for r in in_prompt:
            if r.status == RUNNING and budget > 0 and r.seq_id not in planned:
                try_schedule(r)
        for r in aborted:
            self._finish(r, "cache_full")
        # 3. admit waiting requests while there is budget, a slot and room for a first portion
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs and self.cache.has_free_slot():
            r = self.waiting[0]
            if r.pending:
                break    # preempted with a token still in flight: its recompute needs the value
            count = min(r.cur_len, self.prefill_chunk, budget)
            self.cache.begin(r.seq_id)
            if self.running and self.admit_whole_prompts and not self._room_for_whole_prompt(r):
                self.cache.end(r.seq_id)
                break
            if not self.cache.reserve(r.seq_id, count):
                self.cache.end(r.seq_id)
                if not self.running:
                    # the pools are empty and the first portion still does not fit
                    self.waiting.pop(0)
                    self._finish(r, "cache_full")
                    continue
                break
            self.waiting.pop(0)
            r.status = RUNNING
            self.running.append(r)
            self.stats.admitted += 1
            plan.append(Scheduled(r, 0, count, count == r.cur_len))
            planned.add(r.seq_id)
            budget -= count
        if plan:
            self.stats.steps += 1
            self.stats.scheduled_tokens += sum(s.count for s in plan)
        return plan

    def _room_for_whole_prompt(self, r: Request) -> bool:
        """Would the pools still hold this request's whole prompt (and its first token) once every running request
        has finished its own prompt and taken one more page?  If not, admitting it now only leads to a preemption
        (its own, as the request admitted last) that throws away the portions it has computed by then."""
        need = self.cache.pages_missing(r.seq_id, min(r.cur_len + 1, self.max_model_len))
        free = self.cache.stats().pages_free
        for g in range(len(need)):
            owed = len(self.running)                              # a page of growth per running request
            for q in self.running:
                if q.cur_len - q.num_computed > 1:
                    owed += self.cache.pages_missing(q.seq_id, q.cur_len)[g]
            if free[g] < need[g] + owed:
                return False
        return True

    # ------------------------------------------------------------------ results
    def launched(self, plan: Sequence[Scheduled]) -> None:
        """Record that the step of ``plan`` has been started: its tokens count as computed and
        every token it samples stands in its request as ``PENDING`` until ``resolve``."""
        row = 0
        for s in plan:
            r = s.request
            r.num_computed = s.start + s.count
            if not s.samples:
                continue
            s.slot = len(r.generated)
            r.generated.append(PENDING)
            r.pending += 1
            r.feed_row = row
            row += 1
            if len(r.generated) >= r.params.max_new_tokens or r.cur_len >= self.max_model_len:
                r.closed = True

    def resolve(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> list[Request]:
        """The ids sampled by the step of ``plan`` (one per entry with ``samples`` set, in plan
        order) have arrived.  Returns the requests that finished since the last call, those
        that ``schedule`` ended with "cache_full" included."""
        it = iter(sampled)
        for s in plan:
            if not s.samples:
                continue
            tok = int(next(it))
            r = s.request
            r.pending -= 1
            if s.slot >= len(r.generated):
                continue                      # the request ended before this token (end of sequence one step earlier)
            r.generated[s.slot] = tok
            if r.status == FINISHED:
                continue                      # ended by the scheduler while the step was in flight; the token is kept
            p = r.params
            if p.eos_id is not None and tok == p.eos_id and not p.ignore_eos:
                del r.generated[s.slot + 1:]  # a token asked for beyond the end is dropped when it arrives
                self._finish(r, "eos")
            elif s.slot + 1 >= p.max_new_tokens:
                self._finish(r, "length")
            elif len(r.prompt_ids) + s.slot + 1 >= self.max_model_len:
                self._finish(r, "max_model_len")
        finished, self._finished_now = self._finished_now, []
        return finished

    def update(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> list[Request]:
        """Record a finished step: ``sampled`` holds one token per plan entry with
        ``samples`` set, in plan order.  Returns the requests that finished since the last
        call, those that ``schedule`` ended with "cache_full" included."""
        self.launched(plan)
        return self.resolve(plan, sampled)
