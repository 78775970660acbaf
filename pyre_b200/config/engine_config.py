"""Engine-side settings: everything that is not a property of the model.

The reference scatters these: a module constant ``BLOCK_SIZE = 16`` in two files
(pyre/paged_cache.py:37, pyre/kernels/paged_attn.py:23) and the arguments of
``Scheduler(num_blocks, max_batch, device, dtype)`` (pyre/scheduler.py:28).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}


def parse_dtype(name: "str | torch.dtype") -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"unsupported compute dtype {name}; choose bfloat16 or float32")
        return name
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}; choose bfloat16 or float32") from None


@dataclass
class EngineConfig:
    """How a model is served on one GPU.

    ``dtype``: ``bfloat16`` (weights and cache in bf16, fp32 accumulation, fp32
    softmax/norm/rotary/residual) or ``float32`` (every tensor and every product in
    IEEE fp32, no reduced-precision matrix mode).
    ``page_size``: tokens per cache page (the reference's BLOCK_SIZE).
    ``max_cache_tokens``: capacity of the paged pools in tokens; ``num_pages`` wins if set.
    ``cache_memory_fraction``: with neither of the two, size the pools to this fraction of the
    device memory that is free once the weights are loaded (less a reserve for the activations
    of the largest step); None keeps a small default (8 requests of 8,192 tokens).
    ``max_num_seqs``: most requests live at once (also the number of state slots).
    ``max_num_batched_tokens``: token budget of one step.
    ``prefill_chunk``: most prompt tokens of one request in one step.
    ``max_model_len``: longest sequence (prompt + output); defaults to the model's
    ``max_position_embeddings`` capped by the cache capacity.
    ``admit_whole_prompts``: beside running requests, admit a request only when the pools will hold its
    whole prompt (see ``engine/scheduler.py``); off: admit as soon as its first portion fits.
    ``lookahead``: start a step before the ids sampled by the step before have reached the
    host (they are fed on the device); the host work of a step then hides behind the GPU's.
    ``record_steps``: keep one record per step in ``Engine.step_log`` (tokens, requests, pages free,
    preemptions, the host's time in the call); off by default.
    ``time_kernels``: a measuring mode: every step runs kernel by kernel (no captured graphs, no lookahead)
    with CUDA events around each launch; ``Engine.kernel_times`` sums device microseconds per kernel class
    (norm, qkv, rotary+write, attention, o, gate_up, down, head, sampler) and each step-log record carries
    its own.  The reference keeps every measurement with its run (bench/harness.py:84-135).
    """

    dtype: "str | torch.dtype" = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16
    num_pages: int | None = None
    max_cache_tokens: int | None = None
    cache_memory_fraction: float | None = None
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    prefill_chunk: int = 2048
    max_model_len: int | None = None
    cuda_graphs: bool = True
    lookahead: bool = True
    admit_whole_prompts: bool = True
    debug_poison_freed_pages: bool = False
    record_steps: bool = False
    time_kernels: bool = False

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if self.cache_memory_fraction is not None and not 0.0 < self.cache_memory_fraction <= 1.0:
            raise ValueError("cache_memory_fraction must lie in (0, 1]")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0 or self.prefill_chunk <= 0:
            raise ValueError("max_num_seqs, max_num_batched_tokens and prefill_chunk must be positive")

    def resolve_num_pages(self, default_tokens: int) -> int:
        if self.num_pages is not None:
            return int(self.num_pages)
        tokens = self.max_cache_tokens if self.max_cache_tokens is not None else default_tokens
        return max(1, -(-int(tokens) // self.page_size))
