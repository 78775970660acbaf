"""Token embedding (pyre/model.py:162,196) and the output head (pyre/model.py:172,201)."""

from __future__ import annotations

import torch

from ..kernels import lib, ops
from ..weights.specs import TensorSpec
from .base import Part, PartSpec, make_part, register_part


class TokenEmbedding(Part):
    """x[t] = table[token[t]], widened to the fp32 residual stream."""

    graph_safe = True

    def __init__(self, dtype, device, vocab: int, width: int):
        super().__init__(dtype, device)
        self.vocab, self.width = int(vocab), int(width)
        self.table = None

    def tensors(self):
        return {"weight": TensorSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.table = tensors["weight"]

    def kernel_libraries(self):
        return ["elementwise"]

    def forward(self, ctx):
        return ops.embedding(self.table, ctx.token_ids, err_flag=ctx.error_flag)


class LinearHead(Part):
    """fp32 logits = h W^T for the rows that were asked for.  ``tied_to`` names the
    tensor (full checkpoint name) that stands in when the head's own weight is absent:
    the embedding table of a model with tied embeddings (pyre/loader.py:58-61); the
    storage is then shared, not copied."""

    graph_safe = True

    def __init__(self, dtype, device, vocab: int, width: int, tied_to: "str | None" = None):
        super().__init__(dtype, device)
        self.vocab, self.width, self.tied_to = int(vocab), int(width), tied_to
        self.weight = None

    def tensors(self):
        return {"weight": TensorSpec((self.vocab, self.width), optional_alias=self.tied_to)}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def kernel_libraries(self):
        return ["gemm_f32"] if self.dtype == torch.float32 else ["gemm_tc"]

    def forward(self, ctx, h_rows):
        with lib.section("head"):
            return ops.linear(h_rows, self.weight, out_dtype=torch.float32)


class NormHeadTail(Part):
    """What follows the last block in this architecture (pyre/model.py:199-201): the final norm, applied to the rows
    whose logits are wanted only (the last block's branch output still pending is added on the way), then the head.
    ``names``: the checkpoint prefixes of the two sub-parts' tensors.  An architecture that ends otherwise (no norm,
    a scaled head, several heads) brings a tail of its own; the model's skeleton is embed, the scheduled blocks, tail."""

    graph_safe = True

    DEFAULT_NAMES = {"norm": "model.norm.", "head": "lm_head."}

    def __init__(self, dtype, device, norm: PartSpec, head: PartSpec, names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.norm = make_part("norm", norm, dtype, device)
        self.head = make_part("head", head, dtype, device)

    def children(self):
        return {self.names["norm"]: self.norm, self.names["head"]: self.head}

    def forward(self, ctx, x, pending):
        h = self.norm.forward(ctx, x, delta=pending, rows=ctx.logit_rows)
        return self.head.forward(ctx, h)


register_part("embed", "token_embedding", TokenEmbedding)
register_part("tail", "norm_head", NormHeadTail)
register_part("head", "linear_head", LinearHead)
