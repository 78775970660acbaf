"""Weights from safetensors files, by tensor name.

The reference merges every ``*.safetensors`` shard of the folder into one dictionary
and lets ``load_state_dict`` complain (pyre/loader.py:46-72), reporting at most eight
names.  Here the model gives the table of tensors it expects (name -> TensorSpec) and
the loader checks the files against the whole table before it reads a single tensor:
every missing name, every unexpected name and every wrong shape is listed in ONE
``WeightsError``.  Tensors are then read one at a time (no second full copy on the
host) and converted according to their spec's role.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Mapping

import torch
from safetensors import safe_open

from .specs import TensorSpec


class WeightsError(RuntimeError):
    """The files of a model folder do not match what the model expects."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


def find_shards(model_dir: str | Path) -> list[Path]:
    """All ``*.safetensors`` files of the folder, sorted (pyre/loader.py:46-48)."""
    model_dir = Path(model_dir)
    shards = sorted(model_dir.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors found in {model_dir}")
    return shards


def target_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "matrix":
        return compute
    if spec.role == "vector":
        return torch.float32
    if spec.role == "keep":
        return stored if stored in (torch.float32, torch.int32) else torch.float32
    if spec.role == "int":
        return torch.int32
    raise ValueError(f"unknown tensor role {spec.role!r}")


_INT_TYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_names_and_shapes(expected: Mapping[str, TensorSpec], found: Mapping[str, tuple[tuple[int, ...], str]],
                           where: str) -> None:
    """Raise one WeightsError that lists all three kinds of mismatch.

    ``found`` maps the names in the files to (shape, dtype string)."""
    missing, wrong = [], []
    for name, spec in expected.items():
        if name not in found:
            if spec.optional_alias is not None and spec.optional_alias in found:
                continue
            missing.append(name)
            continue
        shape = tuple(found[name][0])
        if shape != tuple(spec.shape):
            wrong.append((name, tuple(spec.shape), shape))
    unexpected = sorted(n for n in found if n not in expected)
    if not (missing or wrong or unexpected):
        return
    lines = [f"weights in {where} do not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}):")
        lines += [f"    {n}  expected shape {tuple(expected[n].shape)}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}):")
        lines += [f"    {n}  shape {tuple(found[n][0])}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}):")
        lines += [f"    {n}  expected {e}, file has {g}" for n, e, g in wrong]
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def load_tensors(model_dir: str | Path, expected: Mapping[str, TensorSpec], compute: torch.dtype,
                 device: "str | torch.device", sink: Callable[[str, torch.Tensor], None] | None = None
                 ) -> dict[str, torch.Tensor]:
    """Read every expected tensor onto ``device``.

    Returns name -> tensor.  A tensor that is absent but has ``optional_alias`` maps
    to the very same tensor object as its alias (shared storage, unlike the
    reference's second copy, pyre/loader.py:58-61).  ``sink`` is called per tensor as
    soon as it is on the device, so a caller can pack it and drop the original.
    """
    shards = find_shards(model_dir)
    index: dict[str, Path] = {}
    found: dict[str, tuple[tuple[int, ...], str]] = {}
    for shard in shards:
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                sl = f.get_slice(name)
                found[name] = (tuple(sl.get_shape()), str(sl.get_dtype()))
                index[name] = shard
    check_names_and_shapes(expected, found, str(Path(model_dir)))

    out: dict[str, torch.Tensor] = {}
    by_shard: dict[Path, list[str]] = {}
    for name in expected:
        if name in index:
            by_shard.setdefault(index[name], []).append(name)
    for shard, names in by_shard.items():
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in names:
                t = f.get_tensor(name)
                spec = expected[name]
                if spec.role == "int" and t.dtype not in _INT_TYPES:
                    raise WeightsError(f"tensor {name} in {shard} must be an integer table, file has {t.dtype}")
                if spec.role != "int" and not t.dtype.is_floating_point:
                    raise WeightsError(f"tensor {name} in {shard} must be floating point, file has {t.dtype}")
                t = t.to(device=device, dtype=target_dtype(spec, t.dtype, compute)).contiguous()
                out[name] = t
                if sink is not None:
                    sink(name, t)
    for name, spec in expected.items():
        if name not in out:
            out[name] = out[spec.optional_alias]
    return out
