"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere.  The
step runs only the tokens it is given, as one ragged batch, against the cache that
earlier steps left, and returns fp32 logits at the wanted places.  The reference has
two disjoint functions instead: one sequence with any number of tokens
(``forward_paged``, pyre/model.py:250-294) or many sequences with one token each
(``forward_paged_batch``, pyre/model.py:296-342).
"""

from __future__ import annotations

import contextlib
import time

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from ..kernels import lib
from ..models.model import Model
from ..parts.base import collect_launch_keys
from .context import KVView, StateView, StepContext


# The model's ``max_position_embeddings`` is not enforced here: the reference parses it and never
# uses it (pyre/config.py:60), and rotary angles are computed from the position itself.
MAX_EXACT_POSITION = 1 << 24


def device_guard(device):
    """Makes ``device`` the current CUDA device for a block of code.  Kernels are launched on the
    current device's stream and tensor maps are encoded in its context, so everything that launches
    for a model runs under this guard, whichever device was current when the caller came in."""
    device = torch.device(device)
    return torch.cuda.device(device) if device.type == "cuda" else contextlib.nullcontext()


@dataclass
class StepEntry:
    """The next tokens of one live request and the places among them whose logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    feed: "int | None" = None     # the entry's last token is row ``feed`` of the ids that the step before sampled
                                  # (still on the device); ``tokens[-1]`` is then a stand-in


class _Staging:
    """Pinned host buffers for the step's integer arrays: one copy to the device per step.
    Two buffers alternate; a buffer is rewritten only after its last copy has finished."""

    def __init__(self, device):
        self.device = device
        self.bufs = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.bytes_uploaded = 0

    def stage(self, flat: np.ndarray) -> torch.Tensor:
        """Copy ``flat`` into the pinned buffer whose turn it is; returns that host tensor."""
        i = self.turn
        n = flat.shape[0]
        if self.bufs[i] is None or self.bufs[i].shape[0] < n:
            self.bufs[i] = torch.empty(max(n, 4096) * 2, dtype=torch.int32, pin_memory=True)
            self.events[i] = None
        if self.events[i] is not None:
            self.events[i].synchronize()
        host = self.bufs[i][:n]
        host.numpy()[:] = flat
        self.bytes_uploaded += n * 4
        return host

    def mark_copied(self) -> None:
        """The copy out of the current pinned buffer has been issued on the current stream."""
        ev = torch.cuda.Event()
        ev.record()
        self.events[self.turn] = ev
        self.turn ^= 1

    def upload(self, flat: np.ndarray) -> torch.Tensor:
        host = self.stage(flat)
        dev = torch.empty(flat.shape[0], dtype=torch.int32, device=self.device)
        dev.copy_(host, non_blocking=True)
        self.mark_copied()
        return dev


@dataclass
class _DecodeGraph:
    """A captured decode step: the static integer buffer its kernels read, the context whose
    tensors are views of it, the captured launch sequence and the logits it leaves."""

    flat_dev: torch.Tensor
    ctx: StepContext
    graph: "torch.cuda.CUDAGraph"
    logits: torch.Tensor
    replays: int = 0


class Stepper:
    """Binds a model to a cache manager and runs steps.

    Steps that hold only single decoded tokens (one per entry, each wanting its logits) are
    launch-bound: a few hundred small kernels.  With ``cuda_graphs`` such a step is
    captured once per shape (number of rows, width of the block tables, split count of
    the attention) into a CUDA graph whose kernels read a static integer buffer; later
    steps of that shape copy their integers into the buffer and replay the graph.  The
    arithmetic is the same launch sequence either way.  Above four entries the step is
    padded to the next of a few sizes with rows that belong to no request (they write to
    the cache's scratch page and scratch slot, and their logits are dropped)."""

    MAX_GRAPHS = 48
    MIN_TABLE_WIDTH = 16      # pages; narrower block tables are padded to this

    @staticmethod
    def padded_size(n: int) -> int:
        """Rows of the captured step that serves ``n`` decoded tokens.  A batch that shrinks by one request at a
        time would otherwise capture a graph per size; the rows added cost next to nothing (a step of few tokens
        is bound by reading the weights)."""
        if n <= 4:
            return n
        q = 4 if n <= 16 else 8 if n <= 64 else 16
        return -(-n // q) * q

    def __init__(self, model: Model, cache: CacheManager, max_positions: "int | None" = None,
                 cuda_graphs: bool = False):
        self.model, self.cache = model, cache
        self.device = model.device
        self.max_positions = max_positions
        self._staging = _Staging(self.device)
        from ..kernels import ops
        self.error_flag = ops.device_error_flag(self.device)   # one flag per device, raised by any kernel
        self.steps_run = 0
        self.cuda_graphs = bool(cuda_graphs) and model.graph_safe and torch.device(self.device).type == "cuda"
        self._graphs: dict[tuple, _DecodeGraph] = {}
        self._graph_pool = None
        self.graph_replays = 0
        self.graph_captures = 0
        self.capture_seconds = 0.0      # host time spent on first steps of a shape (eager run + capture)
        self.launches_per_graph: dict[tuple, int] = {}

    def build_context(self, entries: Sequence[StepEntry], reserve: bool = True, table_width: "int | None" = None,
                      upload: bool = True, pad_to: int = 0):
        """Check the entries, make room in the cache (unless the caller has) and lay the
        batch out flat.  Raises OutOfPages if a pool is too small; nothing is taken then.
        ``table_width`` pads the block tables to a fixed width (the layout of a captured
        step must not change); ``upload=False`` returns (context factory, flat host array)
        for a caller that owns the device buffer.  ``pad_to`` (steps of single tokens only)
        appends rows that belong to no request until the step has that many: token 0 at
        position 0 of a sequence whose only page is the scratch page, wanting its logits
        (the rows after the entries' own)."""
        cache = self.cache
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        vocab = self.model.vocab_size
        starts, counts = [], []
        tok_list: list[int] = []
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 1:      # a decoded token: the common case by far
                if not 0 <= e.tokens[0] < vocab:
                    raise ValueError(f"request {e.request!r}: token id outside [0, {vocab})")
                tok_list.append(e.tokens[0])
            elif n == 0:
                raise ValueError(f"request {e.request!r}: an entry needs at least one token")
            else:
                if n <= 8:      # a tiny portion: plain integers are cheaper than an array
                    lo, hi = min(e.tokens), max(e.tokens)
                else:
                    toks = np.asarray(e.tokens)
                    lo, hi = toks.min(), toks.max()
                if lo < 0 or hi >= vocab:
                    raise ValueError(f"request {e.request!r}: token id outside [0, {vocab})")
                tok_list.extend(e.tokens)
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request!r}: wanted place {w} outside its {n} tokens")
            start = cache.length(e.request)
            if start + n > MAX_EXACT_POSITION:
                raise ValueError(f"request {e.request!r}: position {start + n} is beyond {MAX_EXACT_POSITION}, the "
                                 f"largest that converts to fp32 exactly for the rotary angles")
            starts.append(start)
            counts.append(n)
        if reserve:
            for e, s, n in zip(entries, starts, counts):
                if not cache.reserve(e.request, s + n):
                    # nothing of this step stays half-reserved in a way that matters: pages
                    # taken for earlier entries remain theirs and are used by a later step
                    raise OutOfPages(f"request {e.request!r}: no pages left to grow from {s} to {s + n} tokens "
                                     f"(free pages per group: {cache.stats().pages_free})")

        B = len(entries)
        T = len(tok_list)
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(counts, out=cu[1:])
        token_ids = np.asarray(tok_list, dtype=np.int32)
        if T == B:      # one token per entry
            positions = np.asarray(starts, dtype=np.int32)
            seq_of_token = np.arange(B, dtype=np.int32)
        else:
            positions = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, counts)])
            seq_of_token = np.repeat(np.arange(B, dtype=np.int32), counts)
        rows = [int(cu[b]) + w for b, e in enumerate(entries) for w in e.want]
        logit_rows = np.asarray(rows, dtype=np.int32)
        reqs = [e.request for e in entries]
        # one slot per entry (so the layout depends on the batch's shape only): where a fed token goes, or -1
        feed_dst = np.asarray([int(cu[b + 1]) - 1 if e.feed is not None else -1 for b, e in enumerate(entries)], dtype=np.int32)
        feed_src = np.asarray([e.feed if e.feed is not None else 0 for e in entries], dtype=np.int32)

        P = max(0, pad_to - B)
        if P:
            if T != B or len(rows) != B:
                raise ValueError("only a step of single tokens that all want their logits can be padded")
            zeros = np.zeros(P, dtype=np.int32)
            token_ids = np.concatenate([token_ids, zeros])
            positions = np.concatenate([positions, zeros])
            seq_of_token = np.arange(B + P, dtype=np.int32)
            cu = np.arange(B + P + 1, dtype=np.int32)
            logit_rows = np.arange(B + P, dtype=np.int32)
            feed_dst = np.concatenate([feed_dst, zeros - 1])
            feed_src = np.concatenate([feed_src, zeros])
            starts = starts + [0] * P

        pieces = [token_ids, positions, seq_of_token, cu, logit_rows, feed_dst, feed_src]
        tables = []
        ps = cache.page_size
        for g, group in enumerate(cache.groups):
            if T == B:
                slot_list = []
                for r, s_ in zip(reqs, starts):
                    page = group.tables[r][s_ // ps]
                    if page < 0:
                        raise RuntimeError(f"request {r!r}: a token would be written to a page already given back")
                    slot_list.append(page * ps + s_ % ps)
                slots = np.asarray(slot_list, dtype=np.int32)
            else:
                slots = np.concatenate([cache.slots_for(g, e.request, s_, n) for e, s_, n in zip(entries, starts, counts)])
            table = cache.block_table_rows(g, reqs, table_width)
            if P:
                slots = np.concatenate([slots, np.full(P, group.scratch_page * ps, dtype=np.int32)])
                table = np.concatenate([table, np.full((P, table.shape[1]), group.scratch_page, dtype=np.int32)])
            tables.append(table.shape)
            pieces += [slots, table.reshape(-1)]
        state_slots = np.asarray([cache.state.slot_of[r] for r in reqs] + [cache.state.scratch_slot] * P, dtype=np.int32)
        pieces.append(state_slots)

        # every piece starts on a 16-byte boundary of the flat buffer
        offsets, total = [], 0
        for p in pieces:
            offsets.append(total)
            total += -(-p.shape[0] // 4) * 4
        flat = np.zeros(max(total, 4), dtype=np.int32)
        for o, p in zip(offsets, pieces):
            flat[o:o + p.shape[0]] = p
        new_lens = [s + n for s, n in zip(starts, counts)]      # of the entries; the padding rows commit nothing

        def make(dev: torch.Tensor) -> StepContext:
            return self._make_context(dev, offsets, pieces, tables, entries, new_lens, cu, starts, state_slots,
                                      T + P, B + P, len(rows) + P)

        if not upload:
            return make, flat
        return make(self._staging.upload(flat))

    def _make_context(self, dev, offsets, pieces, tables, entries, new_lens, cu, starts, state_slots, T, B, R):
        cache = self.cache

        def view(i):
            return dev[offsets[i]:offsets[i] + pieces[i].shape[0]]

        ctx = StepContext(
            dtype=self.model.dtype, device=self.device, num_tokens=T, num_seqs=B, num_logit_rows=R,
            token_ids=view(0), positions=view(1), seq_of_token=view(2), cu_seqlens=view(3), logit_rows=view(4),
            cu_seqlens_host=cu, start_pos_host=np.asarray(starts, dtype=np.int64), error_flag=self.error_flag,
            feed_dst=view(5), feed_src=view(6), entries=list(entries), new_lens=list(new_lens))
        k = 7
        for g, group in enumerate(cache.groups):
            ctx.kv_groups.append(KVView(group.pool, view(k + 1).view(tables[g]), view(k), group.page_size,
                                        group.spec.window))
            k += 2
        slots_dev = view(k)
        for buf in cache.state.buffers:
            ctx.state_groups.append(StateView(buf, slots_dev, state_slots))
        return ctx

    def _feed(self, ctx: StepContext, entries: Sequence[StepEntry], fed_from: "torch.Tensor | None") -> None:
        """Put the ids that the step before sampled (``fed_from``, on the device) into this step's token array."""
        if any(e.feed is not None for e in entries):
            if fed_from is None:
                raise ValueError("an entry asks for a token of the step before, but its sampled ids were not given")
            from ..kernels import ops
            ops.feed_tokens(ctx.token_ids, ctx.feed_dst, ctx.feed_src, fed_from)

    def run_context(self, ctx: StepContext, fed_from: "torch.Tensor | None" = None) -> torch.Tensor:
        with device_guard(self.device):
            self._feed(ctx, ctx.entries, fed_from)
            logits = self.model.forward(ctx)
        for e, new_len in zip(ctx.entries, ctx.new_lens):
            self.cache.commit(e.request, new_len)
        self.steps_run += 1
        return logits

    def step(self, entries: Sequence[StepEntry], reserve: bool = True, fed_from: "torch.Tensor | None" = None) -> torch.Tensor:
        """fp32 logits [R, vocab] on the device, R = total number of wanted places, in the
        order of the entries and of each entry's ``want``.  The tensor is valid until the
        next step (a replayed graph writes its logits to the same memory every time).
        ``fed_from``: the int32 ids that the step before sampled, for entries with ``feed``."""
        with device_guard(self.device):
            if self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
                return self._graph_step(entries, reserve, fed_from)
            return self.run_context(self.build_context(entries, reserve), fed_from)

    @contextlib.contextmanager
    def kernel_timing(self, lead_ms: float = 25.0):
        """``with stepper.kernel_timing() as timer:`` steps taken inside run kernel by kernel (no captured
        graphs) with CUDA events around every launch; ``timer.totals()`` gives device microseconds per kernel
        class (norm, qkv, rotary+write, attention, o, gate_up, down, head, sampler, ...).  A delay of ``lead_ms``
        is queued first so that the host's launches are ahead of the GPU (a step of 28 layers is a few hundred
        launches, a few milliseconds of host time)."""
        from ..kernels import ops
        graphs, self.cuda_graphs = self.cuda_graphs, False
        try:
            with device_guard(self.device), lib.timing() as timer:
                if lead_ms > 0:
                    ops.delay(lead_ms)
                    timer.records.clear()      # the delay itself is no kernel of the step; its end event starts the first one
                yield timer
        finally:
            self.cuda_graphs = graphs

    # ------------------------------------------------------------------ captured decode steps
    def _graph_step(self, entries: Sequence[StepEntry], reserve: bool, fed_from: "torch.Tensor | None" = None) -> torch.Tensor:
        cache = self.cache
        need = 1
        for e in entries:
            need = max(need, -(-(cache.length(e.request) + 1) // cache.page_size))
        width = max(self.MIN_TABLE_WIDTH, 1 << (need - 1).bit_length())      # power-of-two buckets keep the layout stable
        n, rows = len(entries), self.padded_size(len(entries))
        make, flat = self.build_context(entries, reserve, table_width=width, upload=False, pad_to=rows)
        new_lens = [cache.length(e.request) + 1 for e in entries]
        key = (rows, width, self._splits_key(rows, max(new_lens)), flat.shape[0])
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            # first step of this shape: run it eagerly (its result is this step's result), then
            # capture the same launch sequence on a static buffer for the steps to come
            t_capture = time.perf_counter()
            flat_dev = torch.empty(flat.shape[0], dtype=torch.int32, device=self.device)
            self._copy_flat(flat_dev, flat)
            ctx = make(flat_dev)
            self._feed(ctx, entries, fed_from)
            eager_logits = self.model.forward(ctx).clone()
            ctx.scratch.clear()
            before = lib.launch_count
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self.model.forward(ctx)
            self.launches_per_graph[key] = lib.launch_count - before
            self._graphs[key] = _DecodeGraph(flat_dev, ctx, graph, logits)
            result = eager_logits[:n]
            self.graph_captures += 1
            self.capture_seconds += time.perf_counter() - t_capture
        else:
            self._copy_flat(g.flat_dev, flat)
            self._feed(g.ctx, entries, fed_from)     # outside the graph: writes the static token array before the replay
            g.graph.replay()
            g.replays += 1
            self.graph_replays += 1
            lib.launch_count += self.launches_per_graph[key]
            result = g.logits[:n]
        for e, new_len in zip(entries, new_lens):
            cache.commit(e.request, new_len)
        self.steps_run += 1
        return result

    def _splits_key(self, n_entries: int, max_context: int) -> tuple:
        """What the parts' kernels derive from host-side facts of a decode step (``Part.launch_key``);
        a captured graph is reused only while these stay the same."""
        out = set()
        for part in self.model.parts():
            out |= collect_launch_keys(part, n_entries, max_context)
        return tuple(sorted(out, key=repr))

    def _copy_flat(self, flat_dev: torch.Tensor, flat: np.ndarray) -> None:
        host = self._staging.stage(flat)
        flat_dev.copy_(host, non_blocking=True)
        self._staging.mark_copied()

    def check_device_errors(self) -> None:
        """Raise if a kernel of an earlier step raised the device's error flag (synchronises)."""
        from ..kernels import ops
        with device_guard(self.device):
            ops.check_device_errors(self.device)
