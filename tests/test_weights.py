import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from pyre_b200.config import config_from_dict
from pyre_b200.weights import (WeightsError, expected_tensors, load_tensors, random_state, write_random_model)

import helpers as H


def test_expected_names_are_the_checkpoint_names():
    # pyre/model.py:156-172: 12 tensors per layer + embedding + final norm (+ head)
    a = expected_tensors(config_from_dict(H.TINY_A))
    b = expected_tensors(config_from_dict(H.TINY_B))
    assert len(a) == 2 * 12 + 3 and len(b) == 3 * 12 + 3
    assert a["lm_head.weight"].optional_alias == "model.embed_tokens.weight"      # tied
    assert b["lm_head.weight"].optional_alias is None
    assert b["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert b["model.layers.0.self_attn.q_proj.bias"].shape == (96,)
    assert b["model.layers.1.mlp.down_proj.weight"].shape == (96, 256)
    assert "model.layers.0.self_attn.o_proj.bias" not in b


def test_random_folder_is_reproducible_and_tied_head_is_not_stored(tmp_path):
    cfg = config_from_dict(H.TINY_A)
    write_random_model(tmp_path / "m1", cfg, seed=5)
    write_random_model(tmp_path / "m2", cfg, seed=5)
    write_random_model(tmp_path / "m3", cfg, seed=6)
    s1, s2, s3 = (load_file(str(tmp_path / m / "model.safetensors")) for m in ("m1", "m2", "m3"))
    assert set(s1) == set(s2) and all(torch.equal(s1[k], s2[k]) for k in s1)
    assert not torch.equal(s1["model.embed_tokens.weight"], s3["model.embed_tokens.weight"])
    assert "lm_head.weight" not in s1 and len(s1) == 26
    assert json.loads((tmp_path / "m1" / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    # distributions: matrices N(0, 0.02), norm gains 1 + N(0, 0.1)
    assert abs(s1["model.embed_tokens.weight"].std().item() - 0.02) < 0.002
    assert abs(s1["model.norm.weight"].mean().item() - 1.0) < 0.05


def test_load_roles_and_tied_head_shares_storage(tmp_path):
    cfg = config_from_dict(H.TINY_A)
    write_random_model(tmp_path, cfg, seed=1)
    exp = expected_tensors(cfg)
    t = load_tensors(tmp_path, exp, torch.bfloat16, "cpu")
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32      # vectors stay 32-bit
    assert t["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    assert t["lm_head.weight"].data_ptr() == t["model.embed_tokens.weight"].data_ptr()
    t32 = load_tensors(tmp_path, exp, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    # a folder stored in bf16 loads too; vectors widen exactly
    write_random_model(tmp_path / "bf", cfg, seed=1, store_dtype=torch.bfloat16)
    tb = load_tensors(tmp_path / "bf", exp, torch.bfloat16, "cpu")
    assert tb["model.norm.weight"].dtype == torch.float32
    assert torch.equal(tb["model.norm.weight"], t["model.norm.weight"].to(torch.bfloat16).float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(H.TINY_B)
    state = random_state(cfg, 0)
    del state["model.layers.1.mlp.up_proj.weight"]
    del state["lm_head.weight"]                                   # untied: the head is required
    state["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    state["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 96)
    state["model.norm.weight"] = torch.zeros(95)
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_B))
    save_file(state, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as ei:
        load_tensors(tmp_path, expected_tensors(cfg), torch.float32, "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["model.layers.2.self_attn.k_proj.weight", "model.norm.weight"]
    msg = str(e)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected (32, 96), file has (64, 96)",
                   "model.layers.1.mlp.up_proj.weight"):
        assert needle in msg


def test_no_safetensors_and_shards(tmp_path):
    cfg = config_from_dict(H.TINY_A)
    with pytest.raises(FileNotFoundError, match="no .safetensors"):
        load_tensors(tmp_path, expected_tensors(cfg), torch.float32, "cpu")
    # shards: every *.safetensors of the folder is read (pyre/loader.py:46-52)
    state = random_state(cfg, 2)
    names = sorted(state)
    save_file({k: state[k] for k in names[:10]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: state[k] for k in names[10:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    t = load_tensors(tmp_path, expected_tensors(cfg), torch.float32, "cpu")
    assert all(torch.equal(t[k], state[k]) for k in state)
