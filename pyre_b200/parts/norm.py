"""RMSNorm (pyre/model.py:22-38), fused with the residual add that precedes it."""

from __future__ import annotations

from ..kernels import ops
from ..weights.specs import TensorSpec
from .base import Part, register_part


class RMSNorm(Part):
    """h = (v / sqrt(mean(v^2) + eps)) * weight with v = x + delta, all in fp32; ``x`` is
    the fp32 residual stream and receives the sum."""

    graph_safe = True
    fuses_into_product = True     # forward takes ``scaled_ok``: with it, the norm may run as the fix-up of the product
                                  # that ``delta`` stands for and hand its consumer ``ops.ScaledRows``

    def __init__(self, dtype, device, width: int, eps: float):
        super().__init__(dtype, device)
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def tensors(self):
        return {"weight": TensorSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def kernel_libraries(self):
        return ["elementwise"]

    def forward(self, ctx, x, delta=None, rows=None, update_x=True, scaled_ok=False):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, self.dtype, rows=rows, update_x=update_x, scaled_ok=scaled_ok)


register_part("norm", "rms_norm", RMSNorm)
