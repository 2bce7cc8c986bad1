"""Typed configuration and registry: keys, defaults, refusals that name their key."""
import copy

import pytest

import tiny
from xpu_serve_b200 import registry
from xpu_serve_b200.config import ConfigError, Lfm3Config

# the layout of the released checkpoint as the reference's own test writes it
# (tests/unit/model/lfm3_config.cpp:15-28 of the reference)
RELEASED = {
    "model_type": "lfm3", "vocab_size": 128000, "hidden_size": 2048, "intermediate_size": 7680,
    "num_hidden_layers": 24, "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128,
    "norm_eps": 1e-5, "max_position_embeddings": 128000, "sliding_window": 512, "eos_token_id": 7,
    "layer_types": (["conv", "conv", "full_attention", "conv", "sliding_attention", "conv"] * 4),
    "rope_parameters": {"full_attention": {"rope_type": "default", "rope_theta": 1000000.0,
                                           "partial_rotary_factor": 0.5},
                        "sliding_attention": {"rope_type": "default", "rope_theta": 10000.0}},
}


def test_released_layout_and_defaults():
    c = Lfm3Config.from_json(RELEASED)
    assert c.conv_L_cache == 7 and not c.conv_bias and c.use_sandwich_norm and c.tie_word_embeddings
    assert c.attn_head_gate and c.eos_token_id == (7,)
    assert c.rope["full_attention"].pairs(c.head_dim) == 32 and c.rope["sliding_attention"].pairs(c.head_dim) == 64
    spec = c.model_spec()
    assert len(spec.layers) == 24 and [call.layer for call in spec.order] == list(range(24))
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds.count("short_conv") == 16 and kinds.count("attention") == 8
    assert spec.layers[4].mixer.window == 512 and spec.layers[2].mixer.window == 0
    assert spec.layers[2].mixer.position.pairs == 32 and spec.layers[2].mixer.position.theta == 1000000.0
    assert spec.layers[0].sandwich and spec.tied_head


def test_head_dim_defaults_to_hidden_over_heads():
    j = {k: v for k, v in RELEASED.items() if k != "head_dim"}
    assert Lfm3Config.from_json(j).head_dim == 128


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_round_trip(name):
    c = Lfm3Config.from_json(tiny.CONFIGS[name])
    assert Lfm3Config.from_json(c.to_json()) == c


def test_every_size_comes_from_the_json():
    a, b = Lfm3Config.from_json(tiny.CONFIG_A), Lfm3Config.from_json(tiny.CONFIG_B)
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "norm_eps",
                  "num_attention_heads", "num_key_value_heads", "head_dim", "conv_L_cache", "conv_bias",
                  "tie_word_embeddings", "max_position_embeddings", "initializer_range"):
        assert getattr(a, field) != getattr(b, field), field
    sa, sb = a.model_spec(), b.model_spec()
    assert sa.layers[2].mixer.scale == 0.25 and abs(sb.layers[0].mixer.scale - 32 ** -0.5) < 1e-15
    assert sa.layers[2].mixer.position.theta == 10000.0 and sb.layers[0].mixer.position.theta == 500000.0


def test_attn_alias_and_flat_rope_theta():
    c = Lfm3Config.from_json(tiny.CONFIG_A)
    assert c.layer_types == ("conv", "conv", "full_attention", "conv")
    assert c.rope["full_attention"].theta == 10000.0 and c.rope["full_attention"].partial_rotary_factor == 1.0


def test_legacy_tie_key_wins():
    j = dict(tiny.CONFIG_A, tie_embedding=False, tie_word_embeddings=True)
    assert Lfm3Config.from_json(j).tie_word_embeddings is False


def bad(change, match):
    j = copy.deepcopy(RELEASED)
    change(j)
    with pytest.raises(ConfigError, match=match):
        Lfm3Config.from_json(j)


def test_refusals_name_their_key():
    bad(lambda j: j.pop("vocab_size"), "vocab_size")
    bad(lambda j: j.pop("norm_eps"), "norm_eps")
    bad(lambda j: j.pop("max_position_embeddings"), "max_position_embeddings")
    bad(lambda j: j.pop("layer_types"), "layer_types")
    bad(lambda j: j["layer_types"].append("conv"), "25 entries for 24 layers")
    bad(lambda j: j["layer_types"].__setitem__(0, "mamba"), "unknown layer type 'mamba'")
    bad(lambda j: j.__setitem__("num_key_value_heads", 5), "not a multiple")
    bad(lambda j: j.__setitem__("head_dim", 63), "must be even")
    bad(lambda j: j.__setitem__("conv_L_cache", 1), "conv_L_cache")
    bad(lambda j: j.pop("rope_parameters"), "rope_parameters")
    bad(lambda j: j["rope_parameters"].pop("sliding_attention"), "sliding_attention")
    bad(lambda j: j["rope_parameters"]["full_attention"].__setitem__("rope_type", "yarn"), "rope_type 'yarn'")
    bad(lambda j: j["rope_parameters"]["full_attention"].pop("rope_theta"), "rope_theta")
    bad(lambda j: j.pop("sliding_window"), "sliding_window")
    bad(lambda j: j.__setitem__("sliding_window", 0), "sliding_window")
    bad(lambda j: j.__setitem__("hidden_size", "2048"), "hidden_size")
    bad(lambda j: j.__setitem__("conv_bias", "yes"), "conv_bias")


def test_vl_wrapper_reads_text_config():
    j = {"model_type": "lfm3_vl", "text_config": dict(tiny.CONFIG_A)}
    assert Lfm3Config.from_json(j).hidden_size == 64
    with pytest.raises(ConfigError, match="text_config"):
        Lfm3Config.from_json({"model_type": "lfm3_vl"})


def test_registry_dispatch_and_listing():
    assert registry.architecture_for({"model_type": "lfm3"}).config_class is Lfm3Config
    assert registry.architecture_for({"architectures": ["Lfm3ForCausalLM"]}).name == "lfm3"
    with pytest.raises(ConfigError, match=r"'llama'.*supported: lfm3"):
        registry.architecture_for({"model_type": "llama"})


def test_part_registry():
    assert registry.mixer_class("attention").kind == "attention"
    assert registry.mixer_class("short_conv").kind == "short_conv"
    assert registry.ffn_class("swiglu").kind == "swiglu"
    with pytest.raises(KeyError, match="no mixer of kind 'nope'"):
        registry.mixer_class("nope")


def test_order_validation():
    from dataclasses import replace
    from xpu_serve_b200.config.spec import LayerCall
    spec = Lfm3Config.from_json(tiny.CONFIG_A).model_spec()
    replace(spec, order=(LayerCall(0), LayerCall(2), LayerCall(2, cache_of=1), LayerCall(0))).validate()
    with pytest.raises(ValueError, match="does not run before"):
        replace(spec, order=(LayerCall(2, cache_of=1), LayerCall(2))).validate()
    with pytest.raises(ValueError, match="names layer 9"):
        replace(spec, order=(LayerCall(9),)).validate()
