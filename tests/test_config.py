"""Configuration and registry (no GPU)."""
import json

import pytest

from helpers import CONFIGS, config_dict
from rocmforge_b200.config import (ConfigError, InvalidValue, MissingKey, Qwen2Config, UnknownArchitecture,
                                   architecture_for, known_architectures, load_config)


def test_reads_every_key():
    c = Qwen2Config.from_dict(config_dict(CONFIGS["C"]))
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (4, 80, 5, 5)
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads == 16     # explicit head_dim wins
    assert c.intermediate_size == 112 and c.vocab_size == 300
    assert c.rope_theta == 50000.0 and c.rms_norm_eps == 3e-6 and c.tie_word_embeddings is True
    assert c.eos_token_ids == [3, 5]
    assert [c.window_of_layer(i) for i in range(4)] == [None, None, 24, 24]


def test_defaults_follow_the_reference():
    raw = dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=1, hidden_size=32, num_attention_heads=4,
               intermediate_size=48, vocab_size=10)
    c = Qwen2Config.from_dict(raw)
    assert c.num_key_value_heads == 4            # src/config.rs:587
    assert c.head_dim == 8                       # hidden / heads
    assert c.max_position_embeddings == 2048     # src/loader/metadata.rs:98-101
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6      # src/config.rs:422-423
    assert c.tie_word_embeddings is False and c.window_of_layer(0) is None


def test_round_trip_through_config_json(tmp_path):
    c = Qwen2Config.from_dict(config_dict(CONFIGS["B"]))
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    arch, c2 = load_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and c2 == c


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_key_is_named(key):
    raw = config_dict(CONFIGS["A"])
    del raw[key]
    with pytest.raises(MissingKey) as e:
        Qwen2Config.from_dict(raw)
    assert key in str(e.value)


@pytest.mark.parametrize("key,value", [("num_attention_heads", 0), ("hidden_size", -4), ("vocab_size", 1.5),
                                       ("rms_norm_eps", 0.0), ("rope_theta", "x"), ("hidden_act", "gelu"),
                                       ("head_dim", 15), ("tie_word_embeddings", "yes"),
                                       ("rope_scaling", {"type": "yarn"}), ("eos_token_id", 100000)])
def test_invalid_values(key, value):
    raw = config_dict(CONFIGS["A"])
    raw[key] = value
    with pytest.raises(InvalidValue) as e:
        Qwen2Config.from_dict(raw)
    assert key in str(e.value)


def test_heads_must_divide():
    raw = config_dict(CONFIGS["A"])
    raw["num_key_value_heads"] = 3
    with pytest.raises(InvalidValue):
        Qwen2Config.from_dict(raw)


def test_window_needs_a_size():
    raw = config_dict(CONFIGS["A"])
    raw["use_sliding_window"] = True
    with pytest.raises(InvalidValue):
        Qwen2Config.from_dict(raw)


def test_unknown_architecture_is_an_error(tmp_path):
    raw = config_dict(CONFIGS["A"])
    raw["architectures"] = ["LlamaForCausalLM"]
    (tmp_path / "config.json").write_text(json.dumps(raw))
    with pytest.raises(UnknownArchitecture) as e:
        load_config(str(tmp_path))
    assert "LlamaForCausalLM" in str(e.value) and "Qwen2ForCausalLM" in str(e.value)
    assert "Qwen2ForCausalLM" in known_architectures()


def test_bad_files(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{}")
    with pytest.raises(MissingKey):
        load_config(str(tmp_path))


def test_builder_takes_sizes_from_config_only():
    for name, cfg in CONFIGS.items():
        c = Qwen2Config.from_dict(config_dict(cfg))
        spec = architecture_for(c.architecture).build(c)
        specs = spec.param_specs()
        assert specs["model.embed_tokens.weight"].shape == (c.vocab_size, c.hidden_size)
        q = specs["model.layers.0.self_attn.q_proj.weight"].shape
        assert q == (c.num_attention_heads * c.head_dim, c.hidden_size)
        assert specs["model.layers.0.self_attn.k_proj.bias"].shape == (c.num_key_value_heads * c.head_dim,)
        assert "model.layers.0.self_attn.o_proj.bias" not in specs
        assert specs["model.layers.0.mlp.down_proj.weight"].shape == (c.hidden_size, c.intermediate_size)
        assert (specs["lm_head.weight"].tied_to is not None) == c.tie_word_embeddings
        assert len(spec.schedule) == c.num_hidden_layers
        reqs = spec.cache_requests()
        assert [reqs[i].window for i in range(c.num_hidden_layers)] == \
               [c.window_of_layer(i) for i in range(c.num_hidden_layers)]
