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
    embed: PartSpec
    blocks: list[PartSpec]
    final_norm: PartSpec
    head: PartSpec
    schedule: list[LayerCall] = field(default_factory=list)
    # prefixes of the checkpoint names
    embed_prefix: str = "model.embed_tokens."
    block_prefix: str = "model.layers.{i}."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."
    vocab_size: int = 0
    max_positions: int = 0

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [LayerCall(i) for i in range(len(self.blocks))]
        for call in self.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"schedule names block {call.block}, the model has {len(self.blocks)}")
