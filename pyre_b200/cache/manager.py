"""The cache manager: paged keys and values with a block table per request, in groups,
and slots of fixed-size state.

Groups.  Layers whose mixers need the same of the cache (``PagedKVSpec``: heads, head
size, window) form a group.  A group has its own pool ``[layers, pages, 2, kv_heads,
page_size, head_dim]`` (one page number addresses the same page in every layer of the
group, as in the reference, pyre/paged_cache.py:107), its own allocator and its own
block table per request.  A group with a window gives a page back as soon as every
position in it lies before the window of any token still to come; a group without one
gives pages back when the request ends.  The reference has one implicit group and frees
only at the end (pyre/paged_cache.py:163-167).  Each pool has one page more than the
allocator hands out (``scratch_page``), and each state buffer one slot more
(``scratch_slot``): they belong to the rows with which a captured decode step is padded
to a common size.

State.  Beside the pages there is a slot per live request for state of fixed size
(``StateSpec``), in buffers ``[layers, max_requests + 1, *shape]`` per state group, zeroed when
a request begins.  An architecture without such state has no buffers, but requests
still take and return a slot, so the bookkeeping is exercised.

Lifecycle of a request: ``begin`` -> (``reserve`` new length -> step -> ``commit``)* -> ``end``.
``reserve`` takes pages in every group or in none; it answers False when a pool is
too small at the moment, and the caller decides what to do (the scheduler preempts).
Lengths are committed by the caller after the step; kernels never touch bookkeeping
(the reference advances lengths inside the forward, pyre/paged_cache.py:176-201).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec
from .allocator import OutOfPages, PageAllocator


def pages_for(n_tokens: int, page_size: int) -> int:
    return -(-n_tokens // page_size)


def pages_per_group(kv_groups: Sequence, page_size: int, full_pages: int, max_requests: int, step_tokens: int) -> list[int]:
    """How many pages each paged group gets when a group that keeps every token gets ``full_pages``.  A group
    whose spec bounds what a request holds (``spec.tokens_held(step_tokens)``: a window) never needs more than
    ``max_requests`` times the pages of that many tokens (one more per request, because a window rarely starts
    on a page's edge), so its pool is that small; its memory goes to the groups that keep everything."""
    out = []
    for g in kv_groups:
        held = g.spec.tokens_held(step_tokens) if hasattr(g.spec, "tokens_held") else None
        if held is None:
            out.append(int(full_pages))
        else:
            out.append(max(1, min(int(full_pages), max_requests * (pages_for(held, page_size) + 1))))
    return out


class PagedGroup:
    """Pages and block tables of one group of layers."""

    def __init__(self, spec: PagedKVSpec, n_layers: int, page_size: int, num_pages: int,
                 dtype: torch.dtype, device, allocate_pool: bool = True):
        self.spec, self.n_layers, self.page_size, self.num_pages = spec, n_layers, page_size, num_pages
        self.allocator = PageAllocator(num_pages)
        self.tables: dict[Hashable, list[int]] = {}      # logical page -> physical page, -1 once given back
        self.first_live: dict[Hashable, int] = {}        # first logical page not yet given back
        self._rows: dict[Hashable, np.ndarray] = {}      # tables as arrays, dropped whenever a table changes
        # one page beyond the allocator's range belongs to no request: the rows that pad a captured step to a
        # common size write their token there and read it back
        self.scratch_page = num_pages
        self.pool = None
        if allocate_pool:
            self.pool = torch.zeros((n_layers, num_pages + 1, 2, spec.n_kv_heads, page_size, spec.head_dim),
                                    dtype=dtype, device=device)
        self.poison = False

    # a token at position p of a request with `length` tokens cached needs keys from here on
    def _first_needed_page(self, start_pos: int) -> int:
        if self.spec.window is None:
            return 0
        return max(0, start_pos - self.spec.window + 1) // self.page_size

    def begin(self, req) -> None:
        self.tables[req] = []
        self.first_live[req] = 0

    def pages_missing(self, req, new_len: int) -> int:
        return max(0, pages_for(new_len, self.page_size) - len(self.tables[req]))

    def take(self, req, n_pages: int) -> None:
        self.tables[req].extend(self.allocator.allocate_many(n_pages))
        self._rows.pop(req, None)

    def grow(self, req, new_len: int) -> None:
        self.take(req, self.pages_missing(req, new_len))

    def row(self, req) -> np.ndarray:
        """The request's block table as an int32 array; kept until the table changes (a page taken or
        given back), which in decoding happens once in ``page_size`` steps."""
        r = self._rows.get(req)
        if r is None:
            r = self._rows[req] = np.asarray(self.tables[req], dtype=np.int32)
        return r

    def release_passed(self, req, length: int) -> list[int]:
        """Give back the pages that no token at position >= length will read."""
        if self.spec.window is None:
            return []
        table = self.tables[req]
        keep_from = min(self._first_needed_page(length), len(table))
        freed = []
        for lp in range(self.first_live[req], keep_from):
            if table[lp] >= 0:
                if self.allocator.free(table[lp]):
                    freed.append(table[lp])
                table[lp] = -1
                self._rows.pop(req, None)
        self.first_live[req] = max(self.first_live[req], keep_from)
        self._poison(freed)
        return freed

    def end(self, req) -> list[int]:
        freed = []
        for page in self.tables.pop(req):
            if page >= 0 and self.allocator.free(page):
                freed.append(page)
        self.first_live.pop(req)
        self._rows.pop(req, None)
        self._poison(freed)
        return freed

    def _poison(self, pages: Sequence[int]) -> None:
        """Debug aid: fill pages that went back to the pool with NaN, so that a read of a
        page that is no longer owned shows up in the logits."""
        if self.poison and self.pool is not None and pages:
            idx = torch.as_tensor(list(pages), dtype=torch.long, device=self.pool.device)
            self.pool[:, idx] = float("nan")

    def pages_held(self, req) -> int:
        return sum(1 for p in self.tables[req] if p >= 0)


class StateSlots:
    """Slots of fixed-size per-request state, one buffer per state group."""

    def __init__(self, groups: Sequence[tuple[StateSpec, int]], max_requests: int, device, allocate: bool = True):
        self.max_requests = max_requests
        self._free = list(range(max_requests - 1, -1, -1))
        self.slot_of: dict[Hashable, int] = {}
        self.specs = [g for g, _ in groups]
        self.scratch_slot = max_requests     # a slot beyond the requests' own, for the rows that pad a captured step
        self.buffers: list[torch.Tensor | None] = []
        for spec, n_layers in groups:
            self.buffers.append(torch.zeros((n_layers, max_requests + 1, *spec.shape), dtype=spec.dtype, device=device)
                                if allocate else None)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, req) -> int:
        if req in self.slot_of:
            raise ValueError(f"request {req!r} already holds a state slot")
        if not self._free:
            raise OutOfPages(f"all {self.max_requests} state slots are in use")
        slot = self._free.pop()
        self.slot_of[req] = slot
        for buf in self.buffers:
            if buf is not None:
                buf[:, slot].zero_()
        return slot

    def release(self, req) -> None:
        self._free.append(self.slot_of.pop(req))


@dataclass
class CacheStats:
    pages_total: list[int] = field(default_factory=list)
    pages_free: list[int] = field(default_factory=list)
    slots_free: int = 0
    live_requests: int = 0


class CacheManager:
    def __init__(self, kv_groups: Sequence, state_groups: Sequence, page_size: int, num_pages: "int | Sequence[int]",
                 max_requests: int, dtype: torch.dtype, device, allocate: bool = True):
        """``kv_groups`` / ``state_groups``: objects with ``.spec`` and ``.n_layers`` (the model's
        ``KVGroup`` / ``StateGroup``).  ``num_pages``: one number for every paged group, or one per group
        (``pages_per_group`` gives a windowed group the small pool it needs)."""
        self.page_size = int(page_size)
        counts = [int(num_pages)] * len(kv_groups) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(counts) != len(kv_groups):
            raise ValueError(f"{len(counts)} page counts for {len(kv_groups)} paged groups")
        self.num_pages = max(counts, default=int(num_pages) if isinstance(num_pages, int) else 0)
        self.groups = [PagedGroup(g.spec, g.n_layers, self.page_size, n, dtype, device, allocate)
                       for g, n in zip(kv_groups, counts)]
        self.state = StateSlots([(g.spec, g.n_layers) for g in state_groups], max_requests, device, allocate)
        self.lengths: dict[Hashable, int] = {}
        self.reserved: dict[Hashable, int] = {}

    # ------------------------------------------------------------------ lifecycle
    def has_free_slot(self) -> bool:
        return self.state.num_free > 0

    def begin(self, req) -> None:
        if req in self.lengths:
            raise ValueError(f"request {req!r} is already live")
        self.state.acquire(req)
        for g in self.groups:
            g.begin(req)
        self.lengths[req] = 0
        self.reserved[req] = 0

    def can_reserve(self, req, new_len: int) -> bool:
        return all(g.allocator.can_allocate(g.pages_missing(req, new_len)) for g in self.groups)

    def pages_missing(self, req, new_len: int) -> list[int]:
        return [g.pages_missing(req, new_len) for g in self.groups]

    def reserve(self, req, new_len: int) -> bool:
        """Make room for the request to grow to ``new_len`` tokens; all groups or none."""
        if new_len < self.lengths[req]:
            raise ValueError(f"request {req!r} holds {self.lengths[req]} tokens; cannot shrink to {new_len}")
        groups = self.groups
        missing = [g.pages_missing(req, new_len) for g in groups]     # mostly zeros: a page lasts page_size tokens
        for g, m in zip(groups, missing):
            if m > g.allocator.num_free:
                return False
        for g, m in zip(groups, missing):
            if m:
                g.take(req, m)
        if new_len > self.reserved[req]:
            self.reserved[req] = new_len
        return True

    def commit(self, req, new_len: int) -> None:
        """The step that wrote tokens up to ``new_len`` has been issued: record the length
        and give back pages that a window has passed."""
        if new_len > self.reserved[req]:
            raise ValueError(f"request {req!r}: commit of {new_len} tokens but only {self.reserved[req]} reserved")
        self.lengths[req] = new_len
        for g in self.groups:
            g.release_passed(req, new_len)

    def end(self, req) -> None:
        if req not in self.lengths:
            raise ValueError(f"request {req!r} is not live (ended twice?)")
        for g in self.groups:
            g.end(req)
        self.state.release(req)
        del self.lengths[req]
        del self.reserved[req]

    def length(self, req) -> int:
        return self.lengths[req]

    def live(self) -> list:
        return list(self.lengths)

    def set_poison(self, on: bool) -> None:
        for g in self.groups:
            g.poison = on

    # ------------------------------------------------------------------ views for a step
    def block_table_rows(self, group: int, reqs: Sequence, width: int | None = None) -> np.ndarray:
        g = self.groups[group]
        rows = [g.row(r) for r in reqs]
        if width is None:
            width = max((r.shape[0] for r in rows), default=0)
        out = np.full((len(reqs), max(width, 1)), -1, dtype=np.int32)
        for i, r in enumerate(rows):
            out[i, :r.shape[0]] = r
        return out

    def slots_for(self, group: int, req, start: int, count: int) -> np.ndarray:
        """Physical slot (page * page_size + offset) of positions start..start+count-1."""
        g = self.groups[group]
        pos = np.arange(start, start + count, dtype=np.int64)
        table = np.asarray(g.tables[req], dtype=np.int64)
        pages = table[pos // self.page_size]
        if (pages < 0).any():
            raise RuntimeError(f"request {req!r}: a token would be written to a page already given back")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def stats(self) -> CacheStats:
        return CacheStats([g.num_pages for g in self.groups], [g.allocator.num_free for g in self.groups],
                          self.state.num_free, len(self.lengths))

    def check(self) -> None:
        """Invariants over all groups: no page lost, none held twice, none free and held."""
        for g in self.groups:
            g.allocator.check()
            held: dict[int, int] = {}
            for table in g.tables.values():
                for p in table:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p, n in held.items():
                if g.allocator.ref_count(p) != n:
                    raise AssertionError(f"page {p}: held by {n} tables, ref count {g.allocator.ref_count(p)}")
            for r, row in g._rows.items():
                if row.tolist() != g.tables[r]:
                    raise AssertionError(f"request {r!r}: the cached row of its block table is stale")
            if len(held) != g.allocator.num_used:
                raise AssertionError(f"{g.allocator.num_used} pages in use but {len(held)} are in block tables")
