"""Configuration: every key of config.json, the feed-forward sizing rule, refusals, the registry."""

import json

import pytest

import tiny
from akas_b200.config import (ConfigError, EngineConfig, Lfm2Config, architecture_of, architectures, config_from_dict,
                              load_config, register_architecture)


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = config_from_dict(tiny.TINY_A), config_from_dict(tiny.TINY_B)
    for field in ("hidden_size", "feed_forward_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                  "layer_kinds", "vocab_size", "conv_kernel", "conv_bias", "norm_eps", "rope_theta", "tie_embedding"):
        assert getattr(a, field) != getattr(b, field), field
    assert a.layer_kinds == ("conv", "attention", "conv", "attention")
    assert b.layer_kinds == ("attention", "conv", "attention", "conv", "conv", "attention")
    assert (b.feed_forward_size, b.rope_theta, b.head_dim) == (256, 1e6, 32)


@pytest.mark.parametrize("intermediate,expected", [(12288, 8192), (6656, 4608), (10240, 6912)])
def test_feed_forward_rule_gives_the_published_sizes(intermediate, expected):
    data = dict(intermediate_size=intermediate, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
                block_multiple_of=256)
    assert Lfm2Config.feed_forward_width(data) == expected
    assert Lfm2Config.feed_forward_width(dict(block_ff_dim=intermediate)) == intermediate
    assert Lfm2Config.feed_forward_width(dict(intermediate_size=300, block_auto_adjust_ff_dim=True)) == 200


def test_defaults_follow_the_reference():
    c = config_from_dict(dict(model_type="lfm2", hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
                              intermediate_size=64, vocab_size=10, num_hidden_layers=2, full_attn_idxs=[1]))
    assert (c.conv_kernel, c.norm_eps, c.rope_theta, c.max_position_embeddings) == (3, 1e-5, 1e6, 128000)
    assert c.tie_embedding and not c.conv_bias and c.head_dim == 64 and c.layer_kinds == ("conv", "attention")


@pytest.mark.parametrize("change,word", [
    (dict(layer_types=["conv", "mamba", "conv", "conv"]), "unknown kinds"),
    (dict(num_key_value_heads=3), "multiple of num_key_value_heads"),
    (dict(hidden_size=70), "multiple of num_attention_heads"),
    (dict(head_dim=24), "multiple of 16"),
    (dict(rope_scaling={"type": "linear", "factor": 2}), "rope"),
    (dict(rope_parameters={"rope_type": "yarn"}), "rope"),
    (dict(conv_L_cache=1), "conv_L_cache"),
    (dict(block_use_swiglu=False), "block_use_swiglu"),
    (dict(use_pos_enc=False), "use_pos_enc"),
    (dict(norm_eps=0), "norm_eps"),
    (dict(vocab_size=0), "vocab_size"),
    (dict(layer_types=["conv"]), "entries"),
    (dict(model_type="llama"), "model_type"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError, match=word):
        Lfm2Config.from_dict({**tiny.TINY_A, **change})


def test_full_attn_idxs_must_be_layer_indices():
    data = {k: v for k, v in tiny.TINY_A.items() if k != "layer_types"}
    with pytest.raises(ConfigError):
        Lfm2Config.from_dict({**data, "full_attn_idxs": [9]})
    assert Lfm2Config.from_dict({**data, "full_attn_idxs": [0]}).layer_kinds[0] == "attention"


def test_to_dict_reads_back(tmp_path):
    for data in (tiny.TINY_A, tiny.TINY_B):
        c = config_from_dict(data)
        assert config_from_dict(c.to_dict()) == c
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(tmp_path) == c


def test_registry_maps_name_to_configuration():
    assert "Lfm2ForCausalLM" in architectures()
    assert architecture_of({"architectures": ["Lfm2ForCausalLM"]}) == "Lfm2ForCausalLM"
    assert architecture_of({"model_type": "lfm2"}) == "Lfm2ForCausalLM"
    with pytest.raises(KeyError, match="registered"):
        architecture_of({"architectures": ["NoSuchModel"]})

    class Other(Lfm2Config):
        pass

    register_architecture("OtherForCausalLM", Other)
    assert isinstance(config_from_dict({**tiny.TINY_A, "architectures": ["OtherForCausalLM"]}), Other)
    with pytest.raises(TypeError):
        register_architecture("Broken", dict)


def test_model_spec_is_chosen_layer_by_layer():
    spec = config_from_dict(tiny.TINY_B).model_spec()
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["attention", "short_conv", "attention", "short_conv", "short_conv", "attention"]
    assert spec.layers[1].mixer.kernel_size == 4 and spec.layers[1].mixer.bias
    assert spec.layers[0].mixer.position.theta == 1e6 and spec.layers[0].mixer.qk_norm.eps == 1e-6
    assert spec.layers[3].mixer_prefix == "model.layers.3.conv." and spec.head_name == "lm_head.weight"
    assert [e.layer for e in spec.run_order()] == list(range(6))


def test_engine_config_validates():
    with pytest.raises(ValueError):
        EngineConfig(prefill_chunk=0)
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    with pytest.raises(ValueError):
        EngineConfig(prefill_token_budget=0)
    assert EngineConfig(max_requests=2, context=100).pool_tokens == 200
