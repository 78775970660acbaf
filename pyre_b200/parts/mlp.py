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
    output tile of the product holds both halves and the activation runs in its epilogue."""

    graph_safe = True
    takes_scaled_rows = True      # ``h`` may be ``ops.ScaledRows``: the gate/up product applies the norm's 1/rms itself

    def __init__(self, dtype, device, width: int, intermediate: int, activation: str = "silu"):
        super().__init__(dtype, device)
        self.width, self.intermediate = int(width), int(intermediate)
        if activation != "silu":
            raise ops.UnsupportedSize(f"activation {activation!r}: only silu is implemented")
        self.w_gate_up = self.w_down = None
        self.interleaved = dtype == torch.bfloat16 and self.intermediate % (2 * ops.GATED_BLOCK) == 0

    def tensors(self):
        return {
            "gate_proj.weight": TensorSpec((self.intermediate, self.width)),
            "up_proj.weight": TensorSpec((self.intermediate, self.width)),
            "down_proj.weight": TensorSpec((self.width, self.intermediate)),
        }

    def load(self, tensors):
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        else:
            self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def kernel_libraries(self):
        return ["elementwise"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"])

    def forward(self, ctx, h):
        with lib.section("gate_up"):
            act = ops.gated_linear(h, self.w_gate_up, self.interleaved)
        with lib.section("down"):
            return ops.linear(act, self.w_down, partials_ok=True, deferred_ok=True)


register_part("ffn", "gated_mlp", GatedMLP)
