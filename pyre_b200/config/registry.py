"""One registry from an architecture's name to its configuration class and model builder.

``config.json`` names its model class in ``architectures[0]``; everything in the
package that opens a model folder (engine, command line, trace replay, tests) goes
through ``load_config`` and ``architecture`` here, so a new architecture is added by
one ``register_architecture`` call and no other change.  The reference has a substring
test in its config reader instead (pyre/config.py:38-43).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .model_config import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type[ModelConfig]
    # build(config) -> pyre_b200.models.spec.ModelSpec: the model as data (parts and
    # the order in which layers run), without weights.
    build: Callable[[ModelConfig], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type[ModelConfig], build: Callable[[ModelConfig], Any],
                          *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_cls, build)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES)) or '(none)'}") from None


def architecture_of(config: ModelConfig) -> Architecture:
    return architecture(type(config).architecture)


def config_from_dict(raw: dict[str, Any]) -> ModelConfig:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: key 'architectures' is missing or empty; it names the model class")
    return architecture(archs[0]).config_cls.from_dict(raw)


def load_config(model_dir: str | Path) -> ModelConfig:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {Path(model_dir)}")
    return config_from_dict(json.loads(path.read_text()))


_builtin_done = False


def _ensure_builtin() -> None:
    """Import the package's own architectures on first use (they register themselves)."""
    global _builtin_done
    if not _builtin_done:
        _builtin_done = True
        from ..models import qwen2  # noqa: F401
