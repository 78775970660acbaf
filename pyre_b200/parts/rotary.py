"""Rotary position encoding (pyre/model.py:41-63): half-split pairs, theta from the
configuration, angles in fp32."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import HeadGeometry, PositionEncoding, register_part


class Rotary(PositionEncoding):
    """inv_freq[j] = theta^(-2j / rotary_dim) for j < rotary_dim / 2, computed with the
    reference's fp32 expression (pyre/model.py:45-47); per step, cos and sin of
    float(position) * inv_freq for the step's tokens, shared by all layers that have
    the same settings.  ``rotary_dim`` < head_dim rotates only the first dims of a head.  Bias, rotation of
    q and k and the paged write of k and v are one kernel (``ops.qkv_rope_write``)."""

    graph_safe = True

    def __init__(self, dtype, device, head_dim: int, theta: float, rotary_dim: "int | None" = None,
                 pairing: str = "half"):
        super().__init__(dtype, device)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        if pairing != "half":
            raise ops.UnsupportedSize(f"rotary pairing {pairing!r}: only the half-split pairing is implemented")
        if self.rotary_dim % 8 or self.rotary_dim > self.head_dim:
            raise ops.UnsupportedSize(f"rotary_dim {self.rotary_dim} must be a multiple of 8 and <= head_dim")
        inv = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        self.inv_freq = inv.to(self.device)
        self._key = ("rotary", self.rotary_dim, self.theta)

    def kernel_libraries(self):
        return ["elementwise"]

    def tables(self, ctx):
        tab = ctx.scratch.get(self._key)
        if tab is None:
            tab = ops.rope_table(ctx.positions, self.inv_freq)
            ctx.scratch[self._key] = tab
        return tab


    def apply(self, ctx, qkv, bias, heads: HeadGeometry, kv, cache_layer):
        if heads.head_dim != self.head_dim:
            raise ValueError(f"rotary part built for head_dim {self.head_dim}, used with {heads.head_dim}")
        cos, sin = self.tables(ctx)
        return ops.qkv_rope_write(qkv, bias, cos, sin, cache_layer, kv.slot_mapping, heads.n_heads, heads.n_kv_heads,
                                  heads.head_dim, self.rotary_dim, kv.page_size)


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys are used as projected."""

    graph_safe = True

    def __init__(self, dtype, device):
        super().__init__(dtype, device)

    def kernel_libraries(self):
        return ["elementwise"]


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
