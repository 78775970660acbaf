"""The vocabulary of model parts.

A model is put together from parts of eight categories: ``embed``, ``norm``,
``position``, ``mixer``, ``ffn``, ``block``, ``head`` and ``tail``.  A part

* is described by data: ``PartSpec(kind, params)``; ``kind`` is looked up in the
  registry of its category, ``params`` are the sizes and constants it is built with
  (a part never reads a model configuration and never knows which model it is in);
* lists the checkpoint tensors it owns (``tensors()``: local name -> ``TensorSpec``);
* takes them on the device (``load``), packing them as its kernels want;
* computes on a ``StepContext`` (``pyre_b200.engine.context``), the flat batch of one step.

Interfaces by category (``ctx`` is the StepContext, T its number of tokens):

    embed     forward(ctx) -> x                     fp32 residual stream [T, width]
    norm      forward(ctx, x, delta=None, rows=None, update_x=True) -> h
              h = norm(x + delta) in the activation dtype; writes the sum back to x
              when update_x; with rows, only those rows (gathered), x untouched
    position  apply(ctx, qkv, bias, heads, kv, cache_layer) -> q
              ``qkv``: the stacked projections of the step's tokens [T, (nh + 2 nkv) hd] (a tensor or
              ``kernels.ops.PartialSums``), ``bias`` fp32 or None, ``heads`` a HeadGeometry, ``kv`` the KVView
              of the mixer's cache group.  The part adds the bias, encodes the tokens' positions into the
              queries and keys in whatever way is its own, stores every token's key and value at
              ``kv.slot_mapping`` in ``cache_layer`` (None: store nothing) and returns the queries
              [T, nh hd].  ``PositionEncoding.store`` does the storing for encodings that bring no fused kernel
    mixer     forward(ctx, h, call) -> [T, width]    ``call`` (BoundCall) names the cache
              layer or state layer of this use of the mixer; cache_spec()/state_spec()
              say what it needs from the cache manager
    ffn       forward(ctx, h) -> [T, width]
    block     forward(ctx, x, pending, call) -> (x, pending)   ``pending`` is a branch
              output not yet added to x; the next norm adds it (fused).  A branch output
              (what a mixer or a feed-forward returns, hence ``delta`` and ``pending``) is a
              tensor [T, width] in the activation dtype, or ``kernels.ops.PartialSums`` (fp32
              partial sums that the built-in norm adds up), or ``kernels.ops.DeferredProduct`` (a
              product of few tokens that the built-in norm launches with the residual add folded
              in); a part that needs a plain tensor calls ``kernels.ops.materialize`` on it.
              Likewise a norm may hand a consumer that declares ``takes_scaled_rows``
              ``kernels.ops.ScaledRows`` instead of a tensor (see ``PreNormBlock``)
    head      forward(ctx, h_rows) -> fp32 logits [R, vocab]
    tail      forward(ctx, x, pending) -> fp32 logits [R, vocab] at ``ctx.logit_rows``: everything after the last
              block (the built-in one: a norm over the wanted rows, then a head)

A new part is a class with these methods and one ``register_part`` call; nothing else
in the package has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from ..weights.specs import TensorSpec

CATEGORIES = ("embed", "norm", "position", "mixer", "ffn", "block", "head", "tail")


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class PagedKVSpec:
    """What an attention-like mixer needs from the paged cache: per token and layer,
    keys and values of ``n_kv_heads * head_dim`` elements each.  ``window``: only the
    last ``window`` positions are ever read (None = all), so older pages may be given back."""

    n_kv_heads: int
    head_dim: int
    window: int | None = None

    def bytes_per_token(self, element_size: int) -> int:
        """Bytes of one token's keys and values in one layer of the group."""
        return 2 * self.n_kv_heads * self.head_dim * element_size

    def tokens_held(self, step_tokens: int) -> "int | None":
        """The most tokens of one request whose pages are held at a time, when a step brings it at most
        ``step_tokens`` new ones: None = all of them (no window); with a window, the window of the step's first
        token and the step's own tokens."""
        return None if self.window is None else self.window - 1 + step_tokens


@dataclass(frozen=True)
class StateSpec:
    """State of fixed size per request and per use of the mixer, kept across steps in a
    slot of the cache manager; it starts as zeros when a request begins."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def bytes_per_request(self) -> int:
        """Bytes of one request's state in one layer of the group."""
        n = 1
        for d in self.shape:
            n *= int(d)
        return n * torch.empty((), dtype=self.dtype).element_size()


@dataclass(frozen=True)
class HeadGeometry:
    """How the columns of stacked q, k, v projections divide into heads: ``n_heads`` query heads, then
    ``n_kv_heads`` key heads, then as many value heads, ``head_dim`` columns each."""

    n_heads: int
    n_kv_heads: int
    head_dim: int

    @property
    def width(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim


@dataclass(frozen=True)
class BoundCall:
    """One entry of the layer schedule, resolved against the cache manager's groups."""

    index: int                 # position in the schedule
    block: int                 # which block's weights
    kv_group: int | None = None
    kv_layer: int = 0          # layer index inside the group's pool
    kv_write: bool = True      # False: read what another call wrote
    state_group: int | None = None
    state_layer: int = 0


class Part:
    category: str = ""
    # True if forward() only launches work on the current stream from device-side inputs
    # (no host reads of the step's arrays, no host synchronisation): such a part may be
    # captured in a CUDA graph and replayed for later steps of the same shape.
    graph_safe: bool = False

    def __init__(self, dtype: torch.dtype, device: torch.device):
        self.dtype = dtype
        self.device = device

    def tensors(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by ``tensors()`` (already on the device, already in
        their roles' dtypes)."""

    def kernel_libraries(self) -> list[str]:
        return []

    def children(self) -> "dict[str, Part]":
        """Sub-parts by the name prefix of their tensors."""
        return {}

    def launch_key(self, n_rows: int, max_context: int) -> tuple:
        """What this part's launches take from host-side facts of a step of single tokens
        (``n_rows`` of them, the longest sequence ``max_context`` tokens long) beyond the
        shapes of the step's arrays: a split count, a choice between kernels.  A captured
        step is replayed only for steps whose parts give the same keys.  Hashable items."""
        return ()


class PositionEncoding(Part):
    """Base of the ``position`` parts.  The encoding owns what happens between the q/k/v projections and the
    cache: a mixer hands it the stacked projections and gets the queries back, with keys and values stored.
    The mixer assumes nothing about the encoding (no tables, no rotary width)."""

    category = "position"

    def apply(self, ctx, qkv, bias, heads: HeadGeometry, kv, cache_layer):
        """No encoding at all: bias added, keys and values stored as projected."""
        return self.store(qkv, bias, heads, kv, cache_layer)

    @staticmethod
    def store(qkv, bias, heads: HeadGeometry, kv, cache_layer):
        """For an encoding without a fused kernel of its own: it transforms the projections first (any way it
        likes) and calls this to add ``bias`` (or None), write every token's key and value to the pages and
        split off the queries."""
        from ..kernels import ops
        return ops.qkv_rope_write(qkv, bias, None, None, cache_layer, kv.slot_mapping, heads.n_heads, heads.n_kv_heads,
                                  heads.head_dim, 0, kv.page_size)


_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")
    if kind in _REGISTRY[category] and not replace:
        raise ValueError(f"{category} part {kind!r} is already registered")
    _REGISTRY[category][kind] = cls


def registered_parts(category: str) -> list[str]:
    return sorted(_REGISTRY[category])


def make_part(category: str, spec: PartSpec, dtype: torch.dtype, device) -> Part:
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise ValueError(f"unknown {category} part {spec.kind!r}; registered: {registered_parts(category)}") from None
    part = cls(dtype=dtype, device=torch.device(device), **dict(spec.params))
    part.category = category
    return part


def collect_tensors(part: Part, prefix: str = "") -> dict[str, TensorSpec]:
    """Full names of a part's tensors and of its sub-parts', under ``prefix``."""
    out = {prefix + name: spec for name, spec in part.tensors().items()}
    for sub_prefix, child in part.children().items():
        out.update(collect_tensors(child, prefix + sub_prefix))
    return out


def load_part(part: Part, tensors: Mapping[str, torch.Tensor], prefix: str = "") -> None:
    part.load({name: tensors[prefix + name] for name in part.tensors()})
    for sub_prefix, child in part.children().items():
        load_part(child, tensors, prefix + sub_prefix)


def all_graph_safe(part: Part) -> bool:
    return bool(part.graph_safe) and all(all_graph_safe(c) for c in part.children().values())


def collect_launch_keys(part: Part, n_rows: int, max_context: int) -> set:
    """The launch keys of a part and of its sub-parts for a step of single tokens."""
    key = getattr(part, "launch_key", None)
    out = {tuple(key(n_rows, max_context))} if key is not None else set()
    for child in part.children().values():
        out |= collect_launch_keys(child, n_rows, max_context)
    out.discard(())
    return out


def collect_libraries(part: Part) -> list[str]:
    libs = list(part.kernel_libraries())
    for child in part.children().values():
        libs += collect_libraries(child)
    return libs
