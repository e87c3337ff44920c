"""Configuration: every key of config.json, defaults, errors, the registry."""
import copy
import json

import pytest

import tiny_configs
from gollmgo_b200.config import (ConfigError, EngineConfig, LlamaConfig, known_architectures,
                                 read_config_json, resolve_architecture)
from gollmgo_b200.parts import manifest_for_config


def test_every_key_is_read():
    cfg, *_ = tiny_configs.get("tiny_b")
    c = LlamaConfig.from_dict(cfg)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 128, 4, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 352, 320)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and c.tie_word_embeddings
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (3, 7) and c.max_position_embeddings == 256


def test_defaults():
    c = LlamaConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 64,
                               "num_attention_heads": 4, "intermediate_size": 100,
                               "num_hidden_layers": 1, "vocab_size": 50})
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5
    assert c.rope_scaling is None and not c.tie_word_embeddings and c.eos_token_ids == ()
    assert c.layer_types == ("full_attention",) and c.sliding_window is None


def test_head_dim_need_not_divide_hidden():
    cfg, *_ = tiny_configs.get("tiny_c")
    c = LlamaConfig.from_dict(cfg)
    assert c.head_dim == 48 and c.hidden_size == 120
    assert c.layer_types[0] == "sliding_attention" and c.sliding_window == 24


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_attention_heads": 3, "num_key_value_heads": 2}, "multiple"),
    ({"hidden_size": 66, "head_dim": None}, "head_dim"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": -1}, "positive"),
    ({"num_hidden_layers": "two"}, "integer"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2}}, "lacks"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["sliding_attention", "full_attention"], "sliding_window": None}, "sliding_window"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
])
def test_errors(patch, word):
    cfg, *_ = tiny_configs.get("tiny_a")
    cfg.update(patch)
    cfg = {k: v for k, v in cfg.items() if v is not None or k in ("sliding_window",)}
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(cfg)
    assert word in str(e.value)


def test_registry():
    assert "LlamaForCausalLM" in known_architectures()
    cfg, *_ = tiny_configs.get("tiny_a")
    assert resolve_architecture(cfg).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["GPT2LMHeadModel"]})
    assert "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        resolve_architecture({})


def test_read_config_json(tmp_path):
    cfg, *_ = tiny_configs.get("tiny_a")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert read_config_json(str(tmp_path))["hidden_size"] == 64
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path / "nowhere"))
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(str(tmp_path / "bad"))


def test_manifest_follows_config():
    cfg, *_ = tiny_configs.get("tiny_b")
    m = manifest_for_config(cfg)
    assert m["model.layers.2.self_attn.k_proj.weight"].shape == (32, 128)
    assert m["model.layers.0.mlp.gate_proj.weight"].shape == (352, 128)
    assert m["model.embed_tokens.weight"].shape == (320, 128)
    assert m["lm_head.weight"].optional          # tied
    cfg2, *_ = tiny_configs.get("tiny_a")
    assert not manifest_for_config(cfg2)["lm_head.weight"].optional


def test_engine_config_validation():
    EngineConfig().validate()
    for bad in ({"dtype": "float16"}, {"block_size": 12}, {"max_batch_size": 0},
                {"max_memory_fraction": 1.5}, {"max_token_budget": 0}, {"prefill_chunk_size": -1}):
        with pytest.raises(ValueError):
            EngineConfig(**bad).validate()
    d = EngineConfig()
    # the reference's defaults: internal/config/config.go:63-78
    assert (d.max_batch_size, d.max_token_budget, d.max_queue_depth, d.prefill_chunk_size,
            d.block_size, d.max_memory_fraction) == (64, 4096, 256, 512, 16, 0.9)
