"""A model as data: its parts and the order in which its layers run."""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule.

    ``block``: index into ``ModelSpec.blocks`` (an index may appear in several entries:
    the same weights run twice).
    ``cache``: identifier of the cache layer this entry uses; None = a layer of its own.
    Two entries with the same identifier share keys and values: the first one in the
    schedule writes them, later ones need ``write=False`` and read them."""

    block: int
    cache: "int | str | None" = None
    write: bool = True


@dataclass
class ModelSpec:
    """The skeleton of a model is data too: an embedding, blocks run in the order of ``schedule``, and a tail
    (everything after the last block).  ``final_norm`` and ``head`` are a shorthand for the usual tail (a norm over
    the wanted rows, then a head); an architecture that ends otherwise gives ``tail`` itself."""

    embed: PartSpec
    blocks: list[PartSpec]
    final_norm: "PartSpec | None" = None
    head: "PartSpec | None" = None
    schedule: list[LayerCall] = field(default_factory=list)
    # prefixes of the checkpoint names
    embed_prefix: str = "model.embed_tokens."
    block_prefix: str = "model.layers.{i}."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    vocab_size: int = 0
    max_positions: int = 0
    tail: "PartSpec | None" = None
    tail_prefix: str = ""

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [LayerCall(i) for i in range(len(self.blocks))]
        for call in self.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"schedule names block {call.block}, the model has {len(self.blocks)}")
        if self.tail is None:
            if self.final_norm is None or self.head is None:
                raise ValueError("a model needs a tail: give final_norm and head, or tail")
            self.tail = PartSpec("norm_head", {"norm": self.final_norm, "head": self.head,
                                               "names": {"norm": self.final_norm_prefix, "head": self.head_prefix}})
