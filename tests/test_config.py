import json

import pytest

from pyre_b200.config import (ConfigError, EngineConfig, Qwen2Config, architecture, config_from_dict, load_config,
                              register_architecture, registered_architectures)

RAW = dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, intermediate_size=256, num_hidden_layers=3,
           num_attention_heads=3, vocab_size=1000)


def test_defaults_follow_the_reference():
    # pyre/config.py:45-61
    cfg = config_from_dict(RAW)
    assert isinstance(cfg, Qwen2Config)
    assert cfg.num_key_value_heads == 3 and cfg.head_dim == 32 and cfg.n_rep == 1
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert cfg.tie_word_embeddings is False and cfg.max_position_embeddings == 32768


def test_every_key_is_read():
    raw = dict(RAW, num_key_value_heads=1, head_dim=48, rms_norm_eps=1e-5, rope_theta=1000000,
               tie_word_embeddings=True, max_position_embeddings=512)
    cfg = config_from_dict(raw)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, cfg.rope_theta) == (1, 48, 1e-5, 1e6)
    assert cfg.tie_word_embeddings and cfg.max_position_embeddings == 512 and cfg.n_rep == 3
    assert isinstance(cfg.rope_theta, float)
    # head_dim null or 0 falls back (pyre/config.py:48)
    assert config_from_dict(dict(RAW, head_dim=None)).head_dim == 32
    assert config_from_dict(dict(RAW, head_dim=0)).head_dim == 32


def test_round_trip_through_json(tmp_path):
    cfg = config_from_dict(dict(RAW, num_key_value_heads=1, rope_theta=1e6, tie_word_embeddings=True))
    cfg.to_json(tmp_path / "config.json")
    assert load_config(tmp_path) == cfg
    assert json.loads((tmp_path / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size"])
def test_missing_required_key_is_named(key):
    raw = dict(RAW)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


def test_bad_values_are_refused():
    with pytest.raises(ConfigError, match="multiple of num_key_value_heads"):
        config_from_dict(dict(RAW, num_key_value_heads=2))
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(dict(RAW, rope_scaling={"type": "yarn", "factor": 4}))
    with pytest.raises(ConfigError, match="use_sliding_window"):
        config_from_dict(dict(RAW, use_sliding_window=True, sliding_window=128))
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(dict(RAW, head_dim=31))
    # sliding-window keys that are switched off are accepted, as real checkpoints carry them
    config_from_dict(dict(RAW, use_sliding_window=False, sliding_window=4096, rope_scaling=None))


def test_registry_names_the_unknown_architecture():
    assert "Qwen2ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*registered.*Qwen2ForCausalLM"):
        config_from_dict(dict(RAW, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in RAW.items() if k != "architectures"})
    with pytest.raises(FileNotFoundError):
        load_config("/nonexistent/folder")
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("Qwen2ForCausalLM", Qwen2Config, lambda c: None)
    assert architecture("Qwen2ForCausalLM").config_cls is Qwen2Config


def test_spec_is_built_layer_by_layer_from_the_config():
    cfg = config_from_dict(dict(RAW, num_key_value_heads=1, rms_norm_eps=1e-5, rope_theta=1e6))
    spec = architecture("Qwen2ForCausalLM").build(cfg)
    assert len(spec.blocks) == 3 and [c.block for c in spec.schedule] == [0, 1, 2]
    mixer = spec.blocks[1].params["mixer"]
    assert mixer.kind == "attention" and mixer.params["n_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.params["position"].params == {"head_dim": 32, "theta": 1e6}
    assert spec.blocks[2].params["norm2"].params == {"width": 96, "eps": 1e-5}
    assert spec.blocks[0].params["ffn"].params["intermediate"] == 256
    assert spec.head.params["tied_to"] is None


def test_engine_config():
    ec = EngineConfig(dtype="bf16", page_size=8, max_cache_tokens=100)
    import torch
    assert ec.dtype is torch.bfloat16 and ec.resolve_num_pages(0) == 13
    assert EngineConfig(dtype="float32", num_pages=7).resolve_num_pages(10**6) == 7
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="float16")
