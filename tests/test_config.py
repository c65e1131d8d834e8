"""Configuration parsing, validation and the architecture registry (CPU)."""

import json

import pytest

import helpers as H
from servelab_b200.config import (AttentionSpec, ConfigError, Qwen2Config, config_from_dict,
                                  load_config, register_architecture, registered_architectures,
                                  resolve_architecture)


def test_every_key_is_read():
    c = config_from_dict(H.TINY_B)
    assert isinstance(c, Qwen2Config)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (96, 3, 3, 1, 32, 256, 512)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.max_position_embeddings == 512 and c.eos_token_ids == (510, 511)
    assert c.num_query_groups == 3


def test_defaults_follow_the_reference():
    c = config_from_dict({"model_type": "qwen2", "hidden_size": 64, "num_hidden_layers": 1,
                          "num_attention_heads": 4, "intermediate_size": 8, "vocab_size": 10,
                          "rms_norm_eps": 1e-6})
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rope_theta == 1000000.0 and c.max_position_embeddings == 4096
    assert c.tie_word_embeddings is False and c.eos_token_ids == (0,)


def test_round_trip_and_spec():
    c = config_from_dict(H.TINY_C)
    assert config_from_dict(c.to_dict()) == c
    spec = c.to_model_spec()
    assert len(spec.layers) == 4 and [r.layer for r in spec.run_order] == [0, 1, 2, 3]
    windows = [l.mixer.window for l in spec.layers]
    assert windows == [None, None, 24, 24]
    m = spec.layers[0].mixer
    assert isinstance(m, AttentionSpec) and m.qkv_bias and not m.out_bias
    assert m.head_dim == 48 and m.position.theta == 500000.0
    assert spec.layers[0].mixer_norm.eps == 3e-6


def test_missing_and_invalid_keys_are_all_named():
    with pytest.raises(ConfigError) as e:
        config_from_dict({"model_type": "qwen2", "hidden_size": 64})
    for key in ("num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size",
                "rms_norm_eps"):
        assert key in str(e.value)
    bad = dict(H.TINY_A, num_key_value_heads=3)
    with pytest.raises(ConfigError, match="multiple"):
        config_from_dict(bad)
    with pytest.raises(ConfigError, match="hidden_act"):
        config_from_dict(dict(H.TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(dict(H.TINY_A, use_sliding_window=True))


def test_keys_that_change_the_arithmetic_are_refused():
    """A scaled rotation (legal in Qwen2 checkpoints) or any key this class neither reads nor
    knows to be harmless is an error, never silently wrong logits."""
    base = dict(H.TINY_A)
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen2Config.from_dict({**base, "rope_scaling": {"type": "yarn", "factor": 4.0}})
    Qwen2Config.from_dict({**base, "rope_scaling": None})
    with pytest.raises(ConfigError, match="attention_bias"):
        Qwen2Config.from_dict({**base, "attention_bias": False})
    with pytest.raises(ConfigError, match="partial_rotary_factor"):
        Qwen2Config.from_dict({**base, "partial_rotary_factor": 0.5})
    with pytest.raises(ConfigError) as e:
        Qwen2Config.from_dict({**base, "num_experts": 8, "logit_scale": 2.0})
    assert "'logit_scale'" in str(e.value) and "'num_experts'" in str(e.value)
    # keys that change nothing pass
    c = Qwen2Config.from_dict({**base, "attention_dropout": 0.0, "use_cache": True,
                               "bos_token_id": 1, "initializer_range": 0.02,
                               "transformers_version": "x", "sliding_window": 4096})
    assert c.sliding_window is None
    # a per-layer list must agree with the window keys
    win = dict(H.TINY_C)
    kinds = ["full_attention"] * 2 + ["sliding_attention"] * 2
    Qwen2Config.from_dict({**win, "layer_types": kinds})
    with pytest.raises(ConfigError, match="layer_types"):
        Qwen2Config.from_dict({**win, "layer_types": ["full_attention"] * 4})


def test_registry():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve_architecture({"model_type": "qwen2"}) == "Qwen2ForCausalLM"
    with pytest.raises(ValueError, match="unsupported architecture"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ValueError, match="unsupported architecture"):
        resolve_architecture({"model_type": "qwen3"})

    class Toy:
        @classmethod
        def from_dict(cls, d):
            return cls()
    register_architecture("ToyForCausalLM", Toy, model_type="toy")
    assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), Toy)
    assert isinstance(config_from_dict({"model_type": "toy"}), Toy)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_A))
    assert load_config(str(tmp_path)).vocab_size == 256
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nope"))


def test_engine_config_validation():
    from servelab_b200.config import CacheConfig, EngineConfig, SchedulerConfig
    assert CacheConfig().block_size == 16 and SchedulerConfig().max_num_batched_tokens == 2048
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    with pytest.raises(ValueError):
        CacheConfig(block_size=0)
    with pytest.raises(ValueError):
        SchedulerConfig(policy="sjf")
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
