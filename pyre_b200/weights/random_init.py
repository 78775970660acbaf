"""Random weights from a configuration and a seed.

The reference has no such mode (its loader guards against the accidental default
initialisation of ``nn.Module``, pyre/loader.py:54-57).  Two forms:

* ``write_random_model(dir, config, seed)`` writes ``config.json`` and
  ``model.safetensors`` under the checkpoint names, from a CPU generator in a fixed
  order, so any program (this engine, the tests' plain implementation, the reference)
  reads identical tensors.
* ``random_tensors_on_device`` draws each tensor on the GPU from (seed, name); it is for
  sizes at which a file is impractical (tens of GB) and is reproducible per tensor.
"""

from __future__ import annotations

import zlib
from pathlib import Path
from typing import Mapping

import torch
from safetensors.torch import save_file

from ..config import ModelConfig, architecture_of
from .loader import target_dtype
from .specs import TensorSpec


def _draw(spec: TensorSpec, gen: torch.Generator, device, dtype=torch.float32) -> torch.Tensor:
    kind = spec.init[0]
    if kind == "normal":
        _, mean, std = spec.init
        t = torch.empty(spec.shape, dtype=torch.float32, device=device)
        t.normal_(mean, std, generator=gen)
        return t.to(dtype)
    if kind == "randint":
        _, low, high = spec.init
        return torch.randint(low, high, spec.shape, generator=gen, device=device, dtype=torch.int32)
    if kind == "const":
        return torch.full(spec.shape, spec.init[1], dtype=dtype, device=device)
    raise ValueError(f"unknown init {spec.init!r}")


def expected_tensors(config: ModelConfig) -> dict[str, TensorSpec]:
    from ..models.model import tensor_table
    return tensor_table(architecture_of(config).build(config))


def random_state(config: ModelConfig, seed: int, store_dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """Every tensor of the model on the CPU, drawn in the order of the model's table.

    A tensor with ``optional_alias`` whose alias is drawn too is left out when the
    configuration ties them (the model's table then has no entry that needs it)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    state = {}
    for name, spec in expected_tensors(config).items():
        if spec.optional_alias is not None:
            continue  # tied: the alias stands in, nothing is stored
        dtype = torch.int32 if spec.role == "int" else store_dtype
        state[name] = _draw(spec, gen, "cpu", dtype)
    return state


def write_random_model(model_dir: str | Path, config: ModelConfig, seed: int,
                       store_dtype: torch.dtype = torch.float32) -> Path:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    config.to_json(model_dir / "config.json")
    state = random_state(config, seed, store_dtype)
    save_file({k: v.contiguous() for k, v in state.items()}, str(model_dir / "model.safetensors"))
    return model_dir


def random_tensors_on_device(expected: Mapping[str, TensorSpec], seed: int, compute: torch.dtype,
                             device, sink=None) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if spec.optional_alias is not None:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed((int(seed) << 32) ^ zlib.crc32(name.encode()))
        t = _draw(spec, gen, device)
        if spec.role != "int":
            t = t.to(target_dtype(spec, torch.float32, compute))
        out[name] = t
        if sink is not None:
            sink(name, t)
    for name, spec in expected.items():
        if name not in out:
            out[name] = out[spec.optional_alias]
    return out
