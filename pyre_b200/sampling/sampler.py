"""Device-side sampling of one token per row of logits."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


@dataclass
class SampleTicket:
    ids: torch.Tensor      # [R] int32 on the device
    host: torch.Tensor     # the same in pinned host memory, valid once ``done`` has passed
    done: "torch.cuda.Event"


class Sampler:
    """Greedy and temperature sampling in one kernel launch; one device-to-host copy of
    the chosen ids per step (the reference copies once per request, pyre/scheduler.py:94)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.bytes_uploaded = 0      # sampling parameters sent to the device
        self.bytes_downloaded = 0    # chosen ids read back
        self._host = [None, None]    # pinned buffers for the ids; two tickets may be open at a time
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], token_index: Sequence[int]) -> list[int]:
        """``logits`` [R, V] fp32; ``params[r]`` and ``token_index[r]`` (how many tokens row r's
        request has generated so far) select the rule and the noise of row r."""
        if logits.shape[0] == 0:
            return []
        return self.read(self.sample_async(logits, params, token_index))

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams], token_index: Sequence[int]):
        """Launch the sampling of ``sample`` and the copy of its ids to pinned host memory without
        waiting for them: returns a ticket for ``read``; ``ticket.ids`` are the int32 ids on the device."""
        R = logits.shape[0]
        if all(p.temperature == 0.0 for p in params):
            ids = ops.sample(logits)
        else:
            seeds = np.asarray([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=np.int64)
            small = np.empty((2, R), dtype=np.int32)
            small[0] = np.asarray([p.temperature for p in params], dtype=np.float32).view(np.int32)
            small[1] = np.asarray(token_index, dtype=np.int32)
            seeds_dev = torch.from_numpy(seeds).to(self.device)
            small_dev = torch.from_numpy(small).to(self.device)
            temperature = small_dev[0].view(torch.float32)
            self.bytes_uploaded += seeds.nbytes + small.nbytes
            tix = small_dev[1]
            ids = ops.sample(logits, temperature, seeds_dev, tix)
        self.bytes_downloaded += R * 4
        i = self._turn
        self._turn ^= 1
        if self._host[i] is None or self._host[i].shape[0] < R:
            self._host[i] = torch.empty(max(R, 256), dtype=torch.int32, pin_memory=True)
        host = self._host[i][:R]
        host.copy_(ids, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return SampleTicket(ids, host, done)

    def read(self, ticket: "SampleTicket") -> list[int]:
        """Wait for a ticket's ids and return them."""
        ticket.done.synchronize()
        return ticket.host.tolist()
