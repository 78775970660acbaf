"""The Python entry point: a model folder (or a configuration and a seed) in, token ids out.

The reference has no engine class (pyre/engine.py is a stub); its de-facto entry is
``Scheduler.add_request(prompt_ids, max_new_tokens, eos_id)`` followed by ``run()``, which
returns ``{seq_id: generated ids}`` (pyre/scheduler.py:40-44,105-114).  ``Engine`` keeps
those two calls with the same names and meanings and adds ``generate`` for a list of
prompts.  Tokens in, tokens out: a tokenizer is not part of the engine (the reference
borrows one from another package in its server only, pyre/server/app.py:54-68).
"""

from __future__ import annotations

import contextlib
import dataclasses
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import numpy as np
import torch

from ..cache import CacheManager, pages_per_group
from ..config import EngineConfig, ModelConfig, architecture_of, load_config
from ..kernels import build, lib
from ..models.model import Model
from ..sampling import Sampler, SamplingParams
from .scheduler import PENDING, Request, Scheduler, step_record
from .step import StepEntry, Stepper


@dataclass
class RequestOutput:
    seq_id: int
    prompt_ids: list[int]
    token_ids: list[int]
    finish_reason: str
    preemptions: int = 0
    logits: "np.ndarray | None" = None     # [len(token_ids), vocab] fp32, with SamplingParams.return_logits


class Engine:
    def __init__(self, model: "str | Path | None" = None, engine_config: "EngineConfig | None" = None, *,
                 config: "ModelConfig | None" = None, seed: "int | None" = None, **overrides):
        """``Engine("path/to/model")`` loads config.json and the safetensors files of the
        folder; ``Engine(config=cfg, seed=0)`` draws random weights on the device.
        Keyword ``overrides`` set fields of ``EngineConfig`` (``dtype="float32"``, ...)."""
        if not torch.cuda.is_available():
            raise RuntimeError("pyre_b200 needs a CUDA device (sm_100a); there is no CPU path")
        unknown = [k for k in overrides if k not in EngineConfig.__dataclass_fields__]
        if unknown:
            raise TypeError(f"unknown engine option {unknown[0]!r}")
        # a copy: the caller's configuration object is not changed by the overrides
        ec = dataclasses.replace(engine_config or EngineConfig(), **overrides)
        self.engine_config = ec
        if (model is None) == (config is None):
            raise ValueError("give either a model folder or config= with seed=")
        self.model_config = load_config(model) if model is not None else config
        spec = architecture_of(self.model_config).build(self.model_config)
        self.model = Model(spec, ec.dtype, ec.device)
        build.ensure_built(self.model.kernel_libraries())
        with torch.cuda.device(self.model.device):
            if model is not None:
                self.model.load_weights(model)
            else:
                self.model.init_random(int(seed or 0))
        # max_position_embeddings is a default for the longest sequence, not a hard limit (the
        # reference never enforces it); ``max_model_len`` in the engine configuration overrides it
        max_positions = spec.max_positions or (1 << 20)
        default_tokens = min(max_positions, 8192) * min(ec.max_num_seqs, 8)
        num_pages = ec.resolve_num_pages(default_tokens)
        if ec.num_pages is None and ec.max_cache_tokens is None and ec.cache_memory_fraction:
            num_pages = self._pages_for_memory(ec)
        self.max_model_len = min(ec.max_model_len or max_positions, num_pages * ec.page_size)
        # a group that keeps every token gets num_pages; a windowed group only what its window can hold
        counts = pages_per_group(self.model.kv_groups, ec.page_size, num_pages, ec.max_num_seqs,
                                 min(ec.prefill_chunk, ec.max_num_batched_tokens))
        self.cache = CacheManager(self.model.kv_groups, self.model.state_groups, ec.page_size, counts,
                                  ec.max_num_seqs, ec.dtype, ec.device)
        self.cache.set_poison(ec.debug_poison_freed_pages)
        self.stepper = Stepper(self.model, self.cache, max_positions=max_positions, cuda_graphs=ec.cuda_graphs)
        self.scheduler = Scheduler(self.cache, ec.max_num_seqs, ec.max_num_batched_tokens, ec.prefill_chunk,
                                   self.max_model_len, admit_whole_prompts=ec.admit_whole_prompts)
        self.sampler = Sampler(ec.device)
        self._requests: dict[int, Request] = {}
        self._flight = None      # (plan, sampling ticket, error word) of the step whose ids have not been read yet
        pinned = self.model.device.type == "cuda"
        self._err_host = [torch.zeros(1, dtype=torch.int32, pin_memory=pinned) for _ in range(2)]
        self._err_turn = 0
        self.step_log: "list[dict] | None" = [] if ec.record_steps else None
        self.kernel_times: dict = {}      # with time_kernels: class -> {"us": device time so far, "launches": n}
        self._waited = 0.0                # seconds of the current call spent waiting for a step's ids

    def _pages_for_memory(self, ec: EngineConfig) -> int:
        """Pages of a group that keeps every token, so that all pools and state buffers together take
        ``cache_memory_fraction`` of the memory that is free now (the weights are on the device), less a reserve
        for the activations of the largest step.  Every group's spec says what it costs (``bytes_per_token``,
        ``tokens_held``; ``bytes_per_request`` for state), so a windowed group or a mixer with state is counted
        for what it takes."""
        free, _total = torch.cuda.mem_get_info(self.model.device)
        elem = torch.empty((), dtype=ec.dtype).element_size()
        groups = self.model.kv_groups
        page_bytes = [g.n_layers * g.spec.bytes_per_token(elem) * ec.page_size for g in groups]
        state_bytes = sum(g.n_layers * (ec.max_num_seqs + 1) * g.spec.bytes_per_request() for g in self.model.state_groups)
        if not any(page_bytes):
            return 1
        # activations of a step: a few buffers as wide as the widest matrix output per token (the vocabulary aside),
        # fp32 logits of the wanted rows (one per request in generation), and a gigabyte for everything small
        widest = max([t.shape[0] for t in self.model.tensor_table().values()
                      if len(t.shape) == 2 and t.shape[0] != self.model.vocab_size] or [4096])
        reserve = ec.max_num_batched_tokens * widest * 8 + ec.max_num_seqs * self.model.vocab_size * 8 + (1 << 30)
        budget = int(free * ec.cache_memory_fraction) - reserve - state_bytes
        step_tokens = min(ec.prefill_chunk, ec.max_num_batched_tokens)

        def cost(full_pages: int) -> int:      # every pool has one page more than it hands out
            counts = pages_per_group(groups, ec.page_size, full_pages, ec.max_num_seqs, step_tokens)
            return sum(b * (n + 1) for b, n in zip(page_bytes, counts))

        if budget < cost(1):
            raise RuntimeError(f"cache_memory_fraction {ec.cache_memory_fraction} of {free / 2**30:.1f} GiB free leaves no room "
                               f"for a page per group ({cost(1) / 2**20:.1f} MiB) after a reserve of {reserve / 2**30:.1f} GiB "
                               f"and {state_bytes / 2**20:.1f} MiB of per-request state")
        lo, hi = 1, max(2, budget // max(1, min(b for b in page_bytes if b)))
        while lo < hi:                          # the largest page count whose pools fit
            mid = (lo + hi + 1) // 2
            if cost(mid) <= budget:
                lo = mid
            else:
                hi = mid - 1
        return lo

    # ------------------------------------------------------------------ the reference's two calls
    def add_request(self, prompt_ids: Sequence[int], max_new_tokens: int = 16, eos_id: "int | None" = None,
                    temperature: float = 0.0, seed: int = 0, params: "SamplingParams | None" = None) -> int:
        """Queue a request; returns its ``seq_id`` (pyre/scheduler.py:40-44)."""
        vocab = self.model.vocab_size
        if any(not 0 <= int(t) < vocab for t in prompt_ids):
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        p = params or SamplingParams(temperature=temperature, seed=seed, max_new_tokens=max_new_tokens, eos_id=eos_id)
        r = self.scheduler.add_request(prompt_ids, p)
        self._requests[r.seq_id] = r
        return r.seq_id

    def step(self) -> list[RequestOutput]:
        """One scheduler iteration: plan, run the mixed batch, sample, record.  Returns the
        requests that finished in it.

        With ``lookahead`` (the default) the step is started before the ids of the step before
        have been read: the tokens it needs from that step are taken on the device, and the host
        reads the older ids while the GPU is busy with the new step.  A request's result is then
        returned one call later, and a request that hits its end-of-sequence token has computed
        one token too many (dropped).  The ids are the same either way."""
        sched = self.scheduler
        t_call = time.perf_counter()
        self._waited = 0.0
        plan = sched.schedule()
        flight = None
        if plan:
            prev = self._flight
            entries = []
            for s in plan:
                toks = s.request.tokens(s.start, s.count)
                feed = None
                if toks[-1] == PENDING:
                    toks[-1], feed = 0, s.request.feed_row
                entries.append(StepEntry(s.request.seq_id, toks, [s.count - 1] if s.samples else [], feed))
            timing = self.stepper.kernel_timing() if self.engine_config.time_kernels else contextlib.nullcontext()
            with torch.cuda.device(self.model.device), timing as timer:
                logits = self.stepper.step(entries, reserve=False, fed_from=prev[1].ids if prev and prev[1] is not None else None)
                # the device's error flag travels with the ids: a kernel that gave up (bounded wait, bad index) is
                # reported when this step is read, without a synchronisation of its own
                err = self._err_host[self._err_turn]
                self._err_turn ^= 1
                err.copy_(self.stepper.error_flag, non_blocking=True)
                sampling = [s for s in plan if s.samples]
                keep = [k for k, s in enumerate(sampling) if s.request.params.return_logits]
                if keep:
                    # only requests that ask for their logits pay for this copy (and for the wait it brings)
                    rows = logits[keep].to("cpu").numpy()
                    for k, row in zip(keep, rows):
                        sampling[k].request.logits[len(sampling[k].request.generated)] = row
                ticket = self.sampler.sample_async(logits, [s.request.params for s in sampling],
                                                   [len(s.request.generated) for s in sampling]) if sampling else None
            sched.launched(plan)
            flight = (plan, ticket, err)
        if self._flight is not None:
            self._land(self._flight)
        self._flight = flight
        if flight is not None and not (self.engine_config.lookahead and not self.engine_config.time_kernels):
            self._land(flight)
            self._flight = None
        step_kernels = None
        if plan and self.engine_config.time_kernels:
            step_kernels = timer.totals()
            for cls, t in step_kernels.items():
                acc = self.kernel_times.setdefault(cls, {"us": 0.0, "launches": 0})
                acc["us"] += t["us"]
                acc["launches"] += t["launches"]
        if self.step_log is not None and plan:
            # host_ms: the call's own work (planning, laying out, launching); wait_ms: the part of the call spent
            # waiting for an earlier step's ids.  While wait_ms is well above zero the GPU is the slower side.
            self.step_log.append(step_record(sched.stats.steps - 1, plan, self.cache, sched.stats,
                                             time.perf_counter() - t_call - self._waited))
            self.step_log[-1]["wait_ms"] = round(self._waited * 1e3, 3)
            if step_kernels is not None:
                self.step_log[-1]["kernel_us"] = {cls: round(t["us"], 1) for cls, t in step_kernels.items()}
        outs = []
        for sid in [sid for sid, r in self._requests.items() if r.done and not r.pending]:
            r = self._requests.pop(sid)
            kept = None
            if r.params.return_logits:      # a token computed beyond an end-of-sequence token was dropped, and so are its logits
                kept = np.stack([r.logits[k] for k in range(len(r.generated))]) if r.generated else \
                    np.empty((0, self.model.vocab_size), dtype=np.float32)
            outs.append(RequestOutput(r.seq_id, r.prompt_ids, list(r.generated), r.finish_reason or "", r.preemptions, kept))
        return outs

    def _land(self, flight) -> None:
        """Read the ids of a started step and let the scheduler record them."""
        plan, ticket, err = flight
        t_wait = time.perf_counter()
        ids = self.sampler.read(ticket) if ticket is not None else []
        self._waited += time.perf_counter() - t_wait      # the host had nothing left to do but wait for the GPU
        if ticket is not None and int(err[0]) != 0:
            self.stepper.check_device_errors()      # raises with the kernel's reason
        self.scheduler.resolve(plan, ids)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._flight is not None or any(r.done for r in self._requests.values())

    def run(self) -> dict[int, list[int]]:
        """Run every queued request to its end: ``{seq_id: generated ids}`` (pyre/scheduler.py:105-114)."""
        results = {}
        while self.has_unfinished():
            for out in self.step():
                results[out.seq_id] = out.token_ids
        return results

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], params: "SamplingParams | Sequence[SamplingParams] | None" = None
                 ) -> list[RequestOutput]:
        """Token ids of several prompts in, one ``RequestOutput`` per prompt out (in order)."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        order = [self.add_request(p, params=sp) for p, sp in zip(prompts, params)]
        done: dict[int, RequestOutput] = {}
        while self.has_unfinished():
            for out in self.step():
                done[out.seq_id] = out
        return [done[sid] for sid in order]

    def stats(self) -> dict:
        s, c = self.scheduler.stats, self.cache.stats()
        return {"steps": s.steps, "admitted": s.admitted, "preempted": s.preempted, "finished": s.finished,
                "scheduled_tokens": s.scheduled_tokens, "pages_free": c.pages_free, "pages_total": c.pages_total,
                "kernel_launches": lib.launch_count}
