"""Grouped-query attention over the paged cache (pyre/model.py:75-125 for the math,
pyre/model.py:296-342 and pyre/kernels/paged_attn.py for reading pages in place)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import HeadGeometry, PagedKVSpec, Part, PartSpec, make_part, register_part


class Attention(Part):
    """q, k, v projections (stacked into one product); the position encoding (a sub-part, which adds the
    bias, encodes positions into q and k in its own way and writes keys and values to the pages of this
    call's cache layer); attention of every token of the step over its sequence's cached keys; output projection.

    Parameters: ``width`` (model width), ``n_heads``, ``n_kv_heads``, ``head_dim``
    (``n_heads * head_dim`` need not equal ``width``), ``qkv_bias`` / ``o_bias``,
    ``scale`` (default head_dim^-0.5, pyre/model.py:82), ``window`` (None = all keys),
    ``position``, the PartSpec of the position encoding applied to q and k, and ``names``, the checkpoint's
    names of the four projections (default q_proj, k_proj, v_proj, o_proj: an architecture whose checkpoint
    calls them otherwise says so in its builder, no new part needed).
    A query at position p sees keys max(0, p - window + 1)..p.
    """

    DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the q/k/v product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: "PartSpec | None" = None, qkv_bias: bool = True, o_bias: bool = False,
                 scale: "float | None" = None, window: "int | None" = None, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        if self.n_heads % self.n_kv_heads:
            raise ops.UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ops.UnsupportedSize(f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        if o_bias:
            raise ops.UnsupportedSize("an output-projection bias is not implemented")
        if window is not None and window <= 0:
            raise ValueError("window must be positive or None")
        self.qkv_bias = bool(qkv_bias)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        self.window = window
        self.heads = HeadGeometry(self.n_heads, self.n_kv_heads, self.head_dim)
        self.position = make_part("position", position or PartSpec("none"), dtype, device)
        self.w_qkv = self.b_qkv = self.w_o = None

    def children(self):
        # a position encoding with tensors of its own would find them under the mixer's prefix
        return {"": self.position}

    def tensors(self):
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        n = self.names
        t = {}
        # checkpoint order: weight then bias per projection, the output projection last
        for key, rows in (("q", q), ("k", kv), ("v", kv)):
            t[f"{n[key]}.weight"] = TensorSpec((rows, self.width))
            if self.qkv_bias:
                t[f"{n[key]}.bias"] = TensorSpec((rows,), role="vector")
        t[f"{n['o']}.weight"] = TensorSpec((self.width, q))
        return t

    def load(self, tensors):
        n = self.names
        self.w_qkv = torch.cat([tensors[f"{n[k]}.weight"] for k in "qkv"], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[f"{n[k]}.bias"] for k in "qkv"]).contiguous()
        self.w_o = tensors[f"{n['o']}.weight"]

    def kernel_libraries(self):
        libs = ["elementwise"]      # the position encoding, a sub-part, names its own
        if self.dtype == torch.bfloat16 and self.head_dim <= ops.MMA_MAX_HEAD_DIM:
            libs.append("attention_mma")
            if self.head_dim in ops.PREFILL_HEAD_DIMS:
                libs += ["attention_prefill", "attention_tc"]
        else:
            libs.append("attention_generic")
        libs.append("gemm_f32" if self.dtype == torch.float32 else "gemm_tc")
        return libs

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_heads, self.head_dim, self.window)

    def state_spec(self):
        return None

    def launch_key(self, n_rows, max_context):
        # the tensor-core kernel's split count is chosen on the host from these numbers
        return (ops.attention_splits(n_rows, n_rows, self.n_heads, self.n_kv_heads, max_context, self.window),)

    def forward(self, ctx, h, call):
        kv = ctx.kv_group(call.kv_group)
        layer = kv.pool[call.kv_layer]
        with lib.section("qkv"):
            qkv = ops.linear(h, self.w_qkv, partials_ok=True, deferred_ok=("rope", self.head_dim))
        # the position encoding owns the step from projections to cache: bias, its transformation of q and k,
        # the paged write of k and v; the queries come back
        q = self.position.apply(ctx, qkv, self.b_qkv, self.heads, kv, layer if call.kv_write else None)
        if self.dtype == torch.bfloat16 and self.head_dim <= ops.MMA_MAX_HEAD_DIM:
            a = ops.paged_attention_bf16(ctx, q, layer, kv.block_table, self.n_heads, self.n_kv_heads, self.head_dim,
                                         self.scale, self.window)
        else:
            # float32 and head sizes above 128: the exact fp32-arithmetic kernel
            a = ops.paged_attention_generic(q, layer, kv.block_table, ctx.seq_of_token, ctx.positions, self.n_heads,
                                            self.n_kv_heads, self.head_dim, self.scale, self.window)
        with lib.section("o"):
            return ops.linear(a, self.w_o, partials_ok=True, deferred_ok="residual")


register_part("mixer", "attention", Attention)
