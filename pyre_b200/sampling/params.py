"""How a request's tokens are chosen and when it stops."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 is greedy (argmax, lowest index on a tie), as the reference
    samples (pyre/scheduler.py:80,94).  ``temperature`` > 0 draws by the Gumbel-max rule
    with noise from (``seed``, index of the generated token, vocabulary entry): the
    tokens of a request depend on its seed only, not on what else is in the batch.
    A request stops after ``max_new_tokens`` tokens or after it has produced ``eos_id``
    (which is kept in the output, pyre/scheduler.py:82), unless ``ignore_eos``.
    ``return_logits``: also give back the fp32 logits each generated token was chosen from
    (``RequestOutput.logits``); they are copied to the host step by step, which makes the engine
    wait for every step in which such a request samples."""

    temperature: float = 0.0
    seed: int = 0
    max_new_tokens: int = 16
    eos_id: "int | None" = None
    ignore_eos: bool = False
    return_logits: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
