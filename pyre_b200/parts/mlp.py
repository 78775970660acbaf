"""Dense gated feed-forward (SwiGLU, pyre/model.py:128-139)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, register_part


class GatedMLP(Part):
    """down(act(gate(h)) * up(h)) without biases.  The gate and up weights are stacked
    into one [2 I, width] matrix at load, so one product feeds the activation; in bfloat16,
    when I is a multiple of 128, their rows alternate in blocks of 64 features so that one
    output tile of the product holds both halves and the activation runs in its epilogue.
    ``names``: the checkpoint's names of the three projections (default gate_proj, up_proj, down_proj)."""

    DEFAULT_NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the gate/up product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "silu",
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.width, self.intermediate = int(width), int(intermediate)
        if activation != "silu":
            raise ops.UnsupportedSize(f"activation {activation!r}: only silu is implemented")
        self.w_gate_up = self.w_down = None
        self.interleaved = dtype == torch.bfloat16 and self.intermediate % (2 * ops.GATED_BLOCK) == 0

    def tensors(self):
        n = self.names
        return {
            f"{n['gate']}.weight": TensorSpec((self.intermediate, self.width)),
            f"{n['up']}.weight": TensorSpec((self.intermediate, self.width)),
            f"{n['down']}.weight": TensorSpec((self.width, self.intermediate)),
        }

    def load(self, tensors):
        n = self.names
        gate, up = tensors[f"{n['gate']}.weight"], tensors[f"{n['up']}.weight"]
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(gate, up)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[f"{n['down']}.weight"]

    def kernel_libraries(self):
        return ["elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("gate_up"):
            act = ops.gated_linear(h, self.w_gate_up, self.interleaved)
        with lib.section("down"):
            return ops.linear(act, self.w_down, partials_ok=True, deferred_ok="residual")


register_part("ffn", "gated_mlp", GatedMLP)
