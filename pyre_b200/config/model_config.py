"""Typed model configurations, read from an architecture's own ``config.json`` keys.

``Qwen2Config`` holds exactly the keys that the reference's ``ModelConfig`` reads
(pyre/config.py:15-62): five required sizes and six defaulted values.  No size or
constant that ``config.json`` gives appears anywhere else in the package; parts get
them as constructor parameters from the architecture's builder.
"""

from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model: names the key at fault."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations.

    A subclass lists its fields, names its architecture string and implements
    ``from_dict``; ``to_dict`` must write keys that ``from_dict`` reads back to an
    equal object, because the random-weights mode writes a model folder from it.
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        out = dataclasses.asdict(self)
        out["architectures"] = [self.architecture]
        return out

    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))

    def to_json(self, path: str | Path) -> None:
        Path(path).write_text(json.dumps(self.to_dict(), indent=2) + "\n")


def _require(raw: dict[str, Any], key: str, kind=int):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    try:
        value = kind(raw[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key {key!r} must be {kind.__name__}, got {raw[key]!r}") from None
    return value


def _positive(name: str, value: int) -> int:
    if value <= 0:
        raise ConfigError(f"config.json: {name} must be positive, got {value}")
    return value


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """The Qwen2.5 dense decoder as the reference computes it (pyre/model.py).

    Keys and defaults follow pyre/config.py:45-61: ``num_key_value_heads`` defaults
    to the number of heads, ``rms_norm_eps`` to 1e-6, ``rope_theta`` to 10000,
    ``tie_word_embeddings`` to False, ``max_position_embeddings`` to 32768 and
    ``head_dim`` to ``hidden_size // num_attention_heads`` (a null or zero
    ``head_dim`` falls back too, pyre/config.py:48).

    The reference silently ignores ``rope_scaling`` and the sliding-window keys; a
    checkpoint that switches them on would then be computed wrongly, so they are
    refused here with an error that names the key.
    """

    architecture: ClassVar[str] = "Qwen2ForCausalLM"

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    head_dim: int = 0

    def __post_init__(self):
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "vocab_size",
                     "max_position_embeddings"):
            _positive(name, getattr(self, name))
        if not self.head_dim:
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        _positive("head_dim", self.head_dim)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a "
                f"multiple of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")

    @property
    def n_rep(self) -> int:
        """Query heads per key/value head (pyre/config.py:29-32)."""
        return self.num_attention_heads // self.num_key_value_heads

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "Qwen2Config":
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("config.json: rope_scaling is set; scaled rotary frequencies are not implemented")
        if raw.get("use_sliding_window"):
            raise ConfigError("config.json: use_sliding_window is true; this architecture is built without a window")
        hidden = _require(raw, "hidden_size")
        heads = _require(raw, "num_attention_heads")
        _positive("num_attention_heads", heads)
        return cls(
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size"),
            num_hidden_layers=_require(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads") or heads),
            vocab_size=_require(raw, "vocab_size"),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            head_dim=int(raw.get("head_dim") or hidden // heads),
        )
