"""The flat batch of one step, as the parts see it."""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class KVView:
    """A paged group during one step."""

    pool: torch.Tensor            # [layers, pages, 2, kv_heads, page_size, head_dim]
    block_table: torch.Tensor     # int32 [B, W]: logical page -> physical page, -1 where none
    slot_mapping: torch.Tensor    # int32 [T]: page * page_size + offset where each token's k/v go
    page_size: int
    window: "int | None"


@dataclass
class StateView:
    """A state group during one step: ``buffer[layer, slots[b]]`` is request b's state."""

    buffer: torch.Tensor          # [layers, max_requests + 1, *shape]; the last slot is scratch
    slots: torch.Tensor           # int32 [B] on the device
    slots_host: np.ndarray


@dataclass
class StepContext:
    """All tokens of a step as ONE ragged batch: entry b (a request) brings tokens
    ``cu_seqlens[b]..cu_seqlens[b+1]`` at positions ``start_pos[b]..``; a decoded token is
    an entry with one token.  Parts read the device tensors; the ``*_host`` copies are
    for launch decisions (largest portion, longest context) and for parts that must walk
    the entries in order."""

    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    token_ids: torch.Tensor       # int32 [T]
    positions: torch.Tensor       # int32 [T] absolute position of each token in its sequence
    seq_of_token: torch.Tensor    # int32 [T] index of the entry each token belongs to
    cu_seqlens: torch.Tensor      # int32 [B + 1]
    logit_rows: torch.Tensor      # int32 [R] token rows whose logits are wanted
    cu_seqlens_host: np.ndarray
    start_pos_host: np.ndarray    # int [B] tokens already cached per entry
    kv_groups: list[KVView] = field(default_factory=list)
    state_groups: list[StateView] = field(default_factory=list)
    scratch: dict = field(default_factory=dict)   # per-step values shared between layers (rotary tables)
    error_flag: "torch.Tensor | None" = None
    # the stepper's own: where tokens sampled by the step before enter this one (``token_ids[feed_dst[b]] =
    # sampled[feed_src[b]]`` where feed_dst[b] >= 0), the entries of the step and the lengths to commit after it
    feed_dst: "torch.Tensor | None" = None
    feed_src: "torch.Tensor | None" = None
    entries: list = field(default_factory=list)
    new_lens: list = field(default_factory=list)

    def kv_group(self, index: int) -> KVView:
        return self.kv_groups[index]

    def state_group(self, index: int) -> StateView:
        return self.state_groups[index]

    @property
    def max_new_tokens_per_seq(self) -> int:
        return int(np.diff(self.cu_seqlens_host).max()) if self.num_seqs else 0

    @property
    def max_context(self) -> int:
        if not self.num_seqs:
            return 0
        return int((self.start_pos_host + np.diff(self.cu_seqlens_host)).max())
