"""The order in which layers run is data (no GPU needed): binding a schedule to cache groups.  A layer
may run twice, an entry may read the cache layer another entry wrote, layers with different needs
(a window, other head sizes) get groups of their own, and a schedule that cannot work is refused."""

import pytest
import torch

from pyre_b200.config import architecture, config_from_dict
from pyre_b200.models import LayerCall, Model
from pyre_b200.models.model import tensor_table
from pyre_b200.parts import PagedKVSpec, PartSpec

RAW = dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=3,
           num_attention_heads=4, num_key_value_heads=2, vocab_size=512, tie_word_embeddings=True)


def spec_with(schedule=None, windows=(None, None, None)):
    spec = architecture("Qwen2ForCausalLM").build(config_from_dict(RAW))
    for i, w in enumerate(windows):
        b = spec.blocks[i]
        spec.blocks[i] = PartSpec(b.kind, dict(b.params, mixer=PartSpec("attention", dict(b.params["mixer"].params, window=w))))
    if schedule is not None:
        spec.schedule = schedule
    return spec


def bound(spec):
    m = Model(spec, torch.float32, "cpu")
    return m, [(c.block, c.kv_group, c.kv_layer, c.kv_write) for c in m.calls]


def test_default_schedule_is_one_group_one_layer_each():
    m, calls = bound(spec_with())
    assert calls == [(0, 0, 0, True), (1, 0, 1, True), (2, 0, 2, True)]
    assert [(g.spec, g.n_layers) for g in m.kv_groups] == [(PagedKVSpec(2, 16, None), 3)] and m.state_groups == []


def test_a_layer_twice_and_a_shared_cache():
    sched = [LayerCall(0), LayerCall(1, cache="s"), LayerCall(0), LayerCall(2), LayerCall(1, cache="s", write=False)]
    m, calls = bound(spec_with(sched))
    # five entries, four cache layers: the last entry reads what the second one wrote
    assert calls == [(0, 0, 0, True), (1, 0, 1, True), (0, 0, 2, True), (2, 0, 3, True), (1, 0, 1, False)]
    assert m.kv_groups[0].n_layers == 4
    # the weights are those of three blocks, however often they run
    assert len(tensor_table(spec_with(sched))) == len(tensor_table(spec_with()))


def test_layers_with_different_needs_get_groups_of_their_own():
    m, calls = bound(spec_with(windows=(None, 8, 8)))
    assert [(g.spec.window, g.n_layers) for g in m.kv_groups] == [(None, 1), (8, 2)]
    assert calls == [(0, 0, 0, True), (1, 1, 0, True), (2, 1, 1, True)]


def test_schedules_that_cannot_work_are_refused():
    with pytest.raises(ValueError, match="before any entry wrote"):
        bound(spec_with([LayerCall(0, cache="x", write=False), LayerCall(1)]))
    with pytest.raises(ValueError, match="already has a writer"):
        bound(spec_with([LayerCall(0, cache="x"), LayerCall(1, cache="x")]))
    with pytest.raises(ValueError, match="written with"):
        bound(spec_with([LayerCall(0, cache="x"), LayerCall(1, cache="x", write=False)], windows=(None, 8, None)))
    with pytest.raises(ValueError, match="names block 3"):
        spec = architecture("Qwen2ForCausalLM").build(config_from_dict(RAW))
        type(spec)(spec.embed, spec.blocks, spec.final_norm, spec.head, schedule=[LayerCall(3)])


def test_checkpoint_names_of_the_projections_are_parameters():
    """An architecture whose checkpoint calls the projections otherwise sets ``names`` in its builder; the parts stay
    the same classes.  Here layer 0 of the decoder gets other names, layer 1 keeps the defaults."""
    from pyre_b200.config import architecture, config_from_dict
    from pyre_b200.models.model import tensor_table
    from pyre_b200.parts import PartSpec
    import helpers as H
    spec = architecture("Qwen2ForCausalLM").build(config_from_dict(H.TINY_A))
    b = spec.blocks[0]
    mixer = PartSpec("attention", dict(b.params["mixer"].params, names={"q": "wq", "k": "wk", "v": "wv", "o": "wo"}))
    ffn = PartSpec("gated_mlp", dict(b.params["ffn"].params, names={"gate": "w1", "up": "w3", "down": "w2"}))
    spec.blocks[0] = PartSpec(b.kind, dict(b.params, mixer=mixer, ffn=ffn))
    table = tensor_table(spec)
    for name in ("self_attn.wq.weight", "self_attn.wq.bias", "self_attn.wk.weight", "self_attn.wv.bias", "self_attn.wo.weight",
                 "mlp.w1.weight", "mlp.w3.weight", "mlp.w2.weight"):
        assert "model.layers.0." + name in table
    assert "model.layers.0.self_attn.q_proj.weight" not in table and "model.layers.0.self_attn.wo.bias" not in table
    assert "model.layers.1.self_attn.q_proj.weight" in table and "model.layers.1.mlp.down_proj.weight" in table
    assert table["model.layers.0.mlp.w2.weight"].shape == (H.TINY_A["hidden_size"], H.TINY_A["intermediate_size"])
    # the order of a layer's tensors is the checkpoint's: weight then bias per projection, the output projection last
    layer0 = [n for n in table if n.startswith("model.layers.0.self_attn.")]
    assert layer0 == ["model.layers.0.self_attn." + n for n in ("wq.weight", "wq.bias", "wk.weight", "wk.bias", "wv.weight", "wv.bias", "wo.weight")]
