"""The host-side plans of the kernels (no GPU needed): every plan the matrix-product planner
and the attention's split rule can return is one the kernels accept, and the choices that
were measured stay as measured."""

import pytest

from pyre_b200.kernels import ops

WIDTHS_ROW_STORE = {128, 160, 192, 208, 224, 256}
WIDTHS_WEIGHT_ROWS = {16, 32, 64, 128, 256}


@pytest.mark.parametrize("pairs", [True, False])
def test_every_product_plan_is_one_the_kernel_takes(monkeypatch, pairs):
    monkeypatch.setattr(ops, "CTA_PAIRS", pairs)
    for M in [1, 2, 7, 8, 16, 17, 33, 64, 65, 127, 128, 129, 200, 256, 257, 511, 512, 777, 1024, 1040, 2048, 2056, 4096, 8192, 40000]:
        for N in [8, 64, 130, 136, 512, 1000, 3584, 4608, 5120, 37888, 152064]:
            for K in [8, 64, 72, 512, 520, 3584, 18944]:
                weights_as_rows, bn, splits = ops.tc_gemm_plan(M, N, K)[:3]
                kb = -(-K // 64)
                assert 1 <= splits <= 16 and splits <= max(kb, 1), (M, N, K, bn, splits)
                if weights_as_rows:
                    assert bn in WIDTHS_WEIGHT_ROWS and (M <= 128 or N % 8), (M, N, K, bn)
                    assert bn >= min(M, 256) or M > 256, (M, N, K, bn)      # the tokens of a tile fit its width
                else:
                    # tokens on the rows: many tokens, or 33 to 128 of them with a split K (tiles of 128 x 128)
                    assert bn in WIDTHS_ROW_STORE and N % 8 == 0 and (M > 128 or (M > 32 and bn == 128 and splits > 1)), (M, N, K, bn)
                if splits > 1:
                    assert kb // splits >= 4, (M, N, K, splits)             # a split keeps a few K blocks


def test_measured_product_choices(monkeypatch):
    """Shapes of the 7B model whose best plan was measured on a B200 (microseconds in the kernel's profile)."""
    monkeypatch.setattr(ops, "CTA_PAIRS", True)
    assert ops.tc_gemm_plan(2048, 4608, 3584)[:3] == (False, 256, 1)          # QKV of a 2,048-token portion
    assert ops.tc_gemm_plan(2048, 3584, 18944)[:3] == (False, 224, 1)         # down: 128 pair tiles of 224
    assert ops.tc_gemm_plan(2048, 37888, 3584)[:3] == (False, 256, 1)         # gate/up: whole 256-wide tiles for the fused activation
    wide, bn, splits = ops.tc_gemm_plan(512, 3584, 18944)[:3]                 # few tiles, long K: wide tiles and a split K
    assert not wide and bn >= 208 and splits == 2
    assert ops.tc_gemm_plan(8, 3584, 18944)[:2] == (True, 16)                 # decode: the weights take the MMA's rows
    assert ops.tc_gemm_plan(64, 37888, 3584)[:3] == (True, 64, 1)
    assert ops.tc_gemm_plan(32, 3584, 18944)[:3] == (True, 32, 5)
    assert ops.tc_gemm_plan(64, 3584, 18944)[:3] == (False, 128, 5)           # 33-128 tokens, split K: tokens on the rows
    assert ops.tc_gemm_plan(128, 4608, 3584)[:3] == (False, 128, 4)
    assert ops.tc_gemm_plan(100, 3584, 18944)[:3] == (False, 128, 5)


def test_attention_splits_stay_in_range():
    for batch in [1, 2, 3, 8, 16, 32, 64, 128, 256]:
        for nh, nkv in [(28, 4), (40, 8), (4, 2), (3, 1), (16, 16), (64, 1)]:
            for ctx in [1, 15, 16, 17, 100, 2048, 8192, 32768, 200000]:
                for window in [None, 64, 4096]:
                    s = ops.attention_splits(batch, batch, nh, nkv, ctx, window)
                    assert 1 <= s <= ops.CLUSTER_MAX_SPLITS or (s % 8 == 0 and 24 <= s <= ops.MAX_SCRATCH_SPLITS), (batch, nh, nkv, ctx, window, s)
                    span = ctx if not window else min(ctx, window + 16)
                    assert s <= max(1, -(-span // 16) + 1), (batch, nh, nkv, ctx, window, s)
    # measured inside whole decode steps of the 7B shape
    assert ops.attention_splits(8, 8, 28, 4, 2100, None) == 7
    assert ops.attention_splits(64, 64, 28, 4, 2100, None) == 1
    assert ops.attention_splits(1, 1, 28, 4, 2100, None) == 16
    assert ops.attention_splits(1, 1, 28, 4, 32768, None) == 64         # one long sequence: many small CTAs through scratch memory
    assert ops.attention_splits(1, 1, 28, 4, 8192, None) == 32 and ops.attention_splits(2, 2, 28, 4, 32768, None) == 32
    assert ops.attention_splits(4, 4, 28, 4, 32768, None) == 24 and ops.attention_splits(8, 8, 28, 4, 32768, None) <= ops.CLUSTER_MAX_SPLITS


def test_launch_keys_come_from_the_parts():
    """The stepper keys its captured decode steps on what the parts say (``Part.launch_key``), not on
    what it knows of attention: a block's key is its mixer's split count, a part of another kind adds its own."""
    import torch

    from pyre_b200.config import config_from_dict
    from pyre_b200.config.registry import architecture_of
    from pyre_b200.models.model import Model
    from pyre_b200.parts.base import Part, collect_launch_keys

    cfg = config_from_dict(dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176,
                                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=512))
    model = Model(architecture_of(cfg).build(cfg), torch.bfloat16, "cpu")
    for rows, context in [(1, 40), (8, 2100), (64, 300)]:
        keys = set()
        for b in model.blocks:
            keys |= collect_launch_keys(b, rows, context)
        assert keys == {(ops.attention_splits(rows, rows, 4, 2, context, None),)}
    assert collect_launch_keys(model.embed, 8, 100) == set() and collect_launch_keys(model.tail, 8, 100) == set()

    class Halves(Part):                     # a part whose launches depend on the longest context in its own way
        def launch_key(self, n_rows, max_context):
            return ("halves", max_context > 1000)

    class Holder(Part):
        def children(self):
            return {"inner.": Halves(torch.float32, torch.device("cpu"))}

    holder = Holder(torch.float32, torch.device("cpu"))
    assert collect_launch_keys(holder, 4, 10) == {("halves", False)}
    assert collect_launch_keys(holder, 4, 5000) == {("halves", True)}


def test_shares_of_the_keys_in_the_prompt_attention(monkeypatch):
    """Shares of the keys only where SMs would stand idle: fewer (query tile, head) items than SMs, and then as many
    as fill two CTAs per SM, each with at least 16 key tiles."""
    from pyre_b200.kernels import ops
    monkeypatch.setattr(ops, "sm_count", lambda: 148)
    assert ops.prefill_key_splits(16 * 28, 17.0, 2048, 28, 128) == 1            # 2,048 fresh tokens
    assert ops.prefill_key_splits(16 * 28, 144.0, 2048, 28, 128) == 1           # 2,048 after 8,192: every SM is busy
    assert ops.prefill_key_splits(8 * 28, 136.0, 1024, 28, 128) == 1            # 224 items
    assert ops.prefill_key_splits(4 * 28, 484.0, 512, 28, 128) == 5             # 512 after 30,720: 112 items, two rounds of 97 tiles
    assert ops.prefill_key_splits(4 * 28, 133.0, 512, 28, 128) == 2             # 512 after 8,192: one round
    assert ops.prefill_key_splits(5 * 28, 262.0, 640, 28, 128) == 2             # 640 after 16,384: two rounds would leave 65 tiles each
    assert ops.prefill_key_splits(4 * 28, 5.0, 512, 28, 128) == 1               # 512 fresh tokens: nothing to share
    assert ops.prefill_key_splits(1 * 28, 481.0, 128, 28, 128) == 8             # one query tile per head
    assert ops.prefill_key_splits(1 * 28, 40.0, 128, 28, 128) == 2              # shares of at least 16 tiles
    assert ops.prefill_key_splits(2 * 28, 484.0, 1 << 18, 28, 128) == 1         # the scratch would not fit
