"""Arrangement of a layer's parts: the pre-norm residual block (pyre/model.py:142-153)."""

from __future__ import annotations

from .base import Part, PartSpec, make_part, register_part


class PreNormBlock(Part):
    """x = x + mixer(norm1(x)); x = x + ffn(norm2(x)).

    The residual stream ``x`` is fp32.  A branch output is not added at once: it
    travels as ``pending`` to the next norm, whose kernel adds it to x while it
    normalises (one pass over the row instead of three).  The block therefore returns
    (x, pending) with the feed-forward's output still pending.

    ``names`` gives the prefix of each sub-part's tensors inside the layer."""

    graph_safe = True

    DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.",
                     "norm2": "post_attention_layernorm.", "ffn": "mlp."}

    def __init__(self, dtype, device, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec,
                 names: "dict[str, str] | None" = None):
        super().__init__(dtype, device)
        self.names = dict(self.DEFAULT_NAMES, **(names or {}))
        self.norm1 = make_part("norm", norm1, dtype, device)
        self.mixer = make_part("mixer", mixer, dtype, device)
        self.norm2 = make_part("norm", norm2, dtype, device)
        self.ffn = make_part("ffn", ffn, dtype, device)
        # A norm that can run as the fix-up of the product before it hands its consumer activations that still lack
        # the 1/rms factor (``ops.ScaledRows``); it may do so only for a consumer that says it takes them.  Both are
        # opt-in attributes of the parts; parts without them see plain tensors.

        def lazy(norm, consumer):
            ok = getattr(norm, "fuses_into_product", False) and getattr(consumer, "takes_scaled_rows", False)
            return {"scaled_ok": True} if ok else {}
        self._kw1, self._kw2 = lazy(self.norm1, self.mixer), lazy(self.norm2, self.ffn)

    def children(self):
        return {self.names["norm1"]: self.norm1, self.names["mixer"]: self.mixer,
                self.names["norm2"]: self.norm2, self.names["ffn"]: self.ffn}

    def forward(self, ctx, x, pending, call):
        h = self.norm1.forward(ctx, x, delta=pending, **self._kw1)
        a = self.mixer.forward(ctx, h, call)
        h = self.norm2.forward(ctx, x, delta=a, **self._kw2)
        return x, self.ffn.forward(ctx, h)


register_part("block", "prenorm", PreNormBlock)
