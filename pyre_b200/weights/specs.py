"""What a part says about each tensor it owns: its shape, how it is stored and how
random weights are drawn for it."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor of a part.

    ``role`` decides the storage dtype on the device:
      * ``"matrix"``: operand of a matrix product or a lookup table of activations;
        held in the compute dtype (bfloat16, or float32 on the 32-bit path).
      * ``"vector"``: gains and biases that enter 32-bit arithmetic; always held in
        float32 (a bf16-stored value widens exactly, a 32-bit-stored value stays as it is).
      * ``"keep"``: held in the dtype the file stores it in when that is a 32-bit type
        (state-space constants and the like), else widened to float32.
      * ``"int"``: integer table, held as int32.
    ``init``: ``("normal", mean, std)`` for the random-weights mode.
    ``optional_alias``: name of another tensor that stands in when this one is absent
    (a tied output head reads the embedding table).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: tuple = ("normal", 0.0, 0.02)
    optional_alias: str | None = None
