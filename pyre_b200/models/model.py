"""The generic model: parts instantiated from a ModelSpec, weights bound to them, the
schedule resolved against cache groups, and one ``forward`` over a StepContext."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..parts.base import (BoundCall, PagedKVSpec, StateSpec, all_graph_safe, collect_libraries, collect_tensors,
                          load_part, make_part)
from ..weights import loader, random_init
from ..weights.specs import TensorSpec
from .spec import ModelSpec


@dataclass(frozen=True)
class KVGroup:
    """Layers whose mixers ask the same of the paged cache; they share pages and block tables."""

    spec: PagedKVSpec
    n_layers: int


@dataclass(frozen=True)
class StateGroup:
    spec: StateSpec
    n_layers: int


def _instantiate(spec: ModelSpec, dtype, device):
    embed = make_part("embed", spec.embed, dtype, device)
    blocks = [make_part("block", b, dtype, device) for b in spec.blocks]
    tail = make_part("tail", spec.tail, dtype, device)
    return embed, blocks, tail


def tensor_table(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Checkpoint name -> TensorSpec for every tensor of the model, in a fixed order
    (embedding, layers in order, final norm, head)."""
    embed, blocks, tail = _instantiate(spec, torch.float32, "meta")
    table = collect_tensors(embed, spec.embed_prefix)
    for i, b in enumerate(blocks):
        table.update(collect_tensors(b, spec.block_prefix.format(i=i)))
    table.update(collect_tensors(tail, spec.tail_prefix))
    return table


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.embed, self.blocks, self.tail = _instantiate(spec, dtype, self.device)
        self.vocab_size = spec.vocab_size
        self.calls, self.kv_groups, self.state_groups = self._bind_schedule()
        self.loaded = False
        self.graph_safe = all(all_graph_safe(p) for p in self.parts())

    def parts(self) -> list:
        """The top-level parts: embedding, blocks, tail."""
        return [self.embed, *self.blocks, self.tail]

    # ------------------------------------------------------------------ schedule
    def _bind_schedule(self):
        kv_specs: list[PagedKVSpec] = []
        kv_layers: list[int] = []
        st_specs: list[StateSpec] = []
        st_layers: list[int] = []
        by_cache_id: dict = {}
        calls = []
        for n, call in enumerate(self.spec.schedule):
            mixer = self.blocks[call.block].mixer
            kv_group = None
            kv_layer = 0
            cspec = mixer.cache_spec() if hasattr(mixer, "cache_spec") else None
            if cspec is not None:
                cache_id = call.cache if call.cache is not None else ("own", n)
                if cache_id in by_cache_id:
                    g, layer, writer_spec = by_cache_id[cache_id]
                    if call.write:
                        raise ValueError(f"schedule entry {n}: cache {cache_id!r} already has a writer; "
                                         f"a later user must have write=False")
                    if writer_spec != cspec:
                        raise ValueError(f"schedule entry {n} reads cache {cache_id!r} written with {writer_spec}, "
                                         f"but its mixer needs {cspec}")
                    kv_group, kv_layer = g, layer
                else:
                    if not call.write:
                        raise ValueError(f"schedule entry {n} reads cache {cache_id!r} before any entry wrote it")
                    if cspec not in kv_specs:
                        kv_specs.append(cspec)
                        kv_layers.append(0)
                    kv_group = kv_specs.index(cspec)
                    kv_layer = kv_layers[kv_group]
                    kv_layers[kv_group] += 1
                    by_cache_id[cache_id] = (kv_group, kv_layer, cspec)
            st_group = None
            st_layer = 0
            sspec = mixer.state_spec() if hasattr(mixer, "state_spec") else None
            if sspec is not None:
                if sspec not in st_specs:
                    st_specs.append(sspec)
                    st_layers.append(0)
                st_group = st_specs.index(sspec)
                st_layer = st_layers[st_group]
                st_layers[st_group] += 1
            calls.append(BoundCall(n, call.block, kv_group, kv_layer, call.write, st_group, st_layer))
        kv_groups = [KVGroup(s, n) for s, n in zip(kv_specs, kv_layers)]
        state_groups = [StateGroup(s, n) for s, n in zip(st_specs, st_layers)]
        return calls, kv_groups, state_groups

    # ------------------------------------------------------------------ weights
    def tensor_table(self) -> dict[str, TensorSpec]:
        return tensor_table(self.spec)

    def _bind(self, tensors) -> None:
        load_part(self.embed, tensors, self.spec.embed_prefix)
        for i, b in enumerate(self.blocks):
            prefix = self.spec.block_prefix.format(i=i)
            load_part(b, tensors, prefix)
            # the block has packed what it needs; drop the originals of this layer
            for name in [n for n in tensors if n.startswith(prefix)]:
                del tensors[name]
        load_part(self.tail, tensors, self.spec.tail_prefix)
        self.loaded = True

    def load_weights(self, model_dir: "str | Path") -> None:
        tensors = loader.load_tensors(model_dir, self.tensor_table(), self.dtype, self.device)
        self._bind(tensors)

    def init_random(self, seed: int) -> None:
        """Random weights drawn on the device, per tensor from (seed, name)."""
        tensors = random_init.random_tensors_on_device(self.tensor_table(), seed, self.dtype, self.device)
        self._bind(tensors)

    def kernel_libraries(self) -> list[str]:
        libs = []
        for part in self.parts():
            libs += collect_libraries(part)
        return list(dict.fromkeys(libs + ["sampling"]))

    # ------------------------------------------------------------------ compute
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through the schedule; fp32 logits [R, vocab] at ``ctx.logit_rows``."""
        if not self.loaded:
            raise RuntimeError("the model has no weights: call load_weights or init_random first")
        x = self.embed.forward(ctx)
        pending = None
        for call in self.calls:
            x, pending = self.blocks[call.block].forward(ctx, x, pending, call)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        return self.tail.forward(ctx, x, pending)


def load_model(model_dir: "str | Path", device: str = "cuda:0", dtype="bfloat16"):
    """A model folder (config.json + safetensors) -> (model with its weights on ``device``, its configuration):
    the reference's ``load_model(path, device, dtype)`` (pyre/loader.py:33-79).  The model class comes from
    the registry by the configuration's architecture name, and the kernel libraries this model and dtype
    need are built if they are not there yet."""
    from ..config import architecture_of, load_config, parse_dtype
    from ..kernels import build

    config = load_config(model_dir)
    model = Model(architecture_of(config).build(config), parse_dtype(dtype), device)
    build.ensure_built(model.kernel_libraries())
    model.load_weights(model_dir)
    return model, config
