"""Configuration and registry (no GPU)."""
import json

import pytest

import cima_b200
from cima_b200.config import (ConfigError, Qwen2Config, UnknownArchitecture, lookup_architecture,
                              registered_architectures)
from helpers import TINY_A, TINY_B, TINY_C


def test_required_keys_are_named():
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size"):
        raw = dict(TINY_A)
        del raw[key]
        with pytest.raises(ConfigError, match=key):
            Qwen2Config.from_dict(raw)
    raw = dict(TINY_A)
    del raw["model_type"]
    with pytest.raises(ConfigError, match="model_type"):
        Qwen2Config.from_dict(raw)
    with pytest.raises(ConfigError, match="not a number|missing"):
        Qwen2Config.from_dict(dict(TINY_A, hidden_size="128"))


def test_defaults_follow_the_reference():
    raw = dict(model_type="qwen2", hidden_size=64, num_hidden_layers=1, num_attention_heads=4, intermediate_size=32,
               vocab_size=10)
    c = Qwen2Config.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.max_position_embeddings == 4096 and c.tie_word_embeddings is False
    assert c.use_sliding_window is False


def test_explicit_head_dim_and_geometry_checks():
    c = Qwen2Config.from_dict(TINY_C)
    assert c.head_dim == 48 and c.hidden_size != c.num_attention_heads * c.head_dim
    with pytest.raises(ConfigError, match="multiple"):
        Qwen2Config.from_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="even"):
        Qwen2Config.from_dict(dict(TINY_A, head_dim=31))
    with pytest.raises(ConfigError, match="zero attention geometry"):
        Qwen2Config.from_dict(dict(TINY_A, num_attention_heads=0))
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen2Config.from_dict(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen2Config.from_dict(dict(TINY_A, rope_scaling={"type": "yarn", "factor": 4}))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(dict(TINY_A, use_sliding_window=True))


def test_spec_carries_every_size_and_the_window_per_layer():
    c = Qwen2Config.from_dict(TINY_C)
    s = c.model_spec()
    assert s.vocab == 777 and s.hidden == 200 and len(s.layers) == 4 and s.schedule == [0, 1, 2, 3]
    assert [b.mixer.window for b in s.layers] == [0, 0, 40, 40]
    m = s.layers[0].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.qkv_bias, m.out_bias) == (6, 2, 48, True, False)
    assert abs(m.scale - 48 ** -0.5) < 1e-12 and m.position.theta == 50000.0
    assert s.layers[1].mixer_norm.eps == 3e-6 and s.final_norm.eps == 3e-6
    assert s.layers[3].feed_forward.intermediate == 328
    b = Qwen2Config.from_dict(TINY_B).model_spec()
    assert b.tie_head is False and Qwen2Config.from_dict(TINY_A).model_spec().tie_head is True


def test_layer_types_and_the_newer_spelling_of_the_rotary_base():
    raw = dict(TINY_C, layer_types=["sliding_attention", "full_attention", "full_attention", "sliding_attention"])
    c = Qwen2Config.from_dict(raw)
    assert [b.mixer.window for b in c.model_spec().layers] == [40, 0, 0, 40]
    assert Qwen2Config.from_dict(c.to_dict()) == c
    with pytest.raises(ConfigError, match="layer_types"):
        Qwen2Config.from_dict(dict(TINY_C, layer_types=["full_attention"]))
    with pytest.raises(ConfigError, match="layer_types"):
        Qwen2Config.from_dict(dict(TINY_C, layer_types=["full_attention", "linear_attention", "full_attention", "full_attention"]))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(dict(TINY_A, layer_types=["sliding_attention", "full_attention"]))
    raw = {k: v for k, v in TINY_B.items() if k != "rope_theta"}
    c = Qwen2Config.from_dict(dict(raw, rope_parameters={"rope_theta": 250000.0, "rope_type": "default"}))
    assert c.rope_theta == 250000.0 and c.model_spec().layers[0].mixer.position.theta == 250000.0
    assert Qwen2Config.from_dict(dict(TINY_B, rope_scaling={"rope_type": "default"})).rope_theta == TINY_B["rope_theta"]
    with pytest.raises(ConfigError, match="rope_parameters"):
        Qwen2Config.from_dict(dict(raw, rope_parameters={"rope_theta": 1e6, "rope_type": "linear", "factor": 2.0}))


def test_registry_lookup_and_unknown_names():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert lookup_architecture(TINY_A).name == "Qwen2ForCausalLM"
    assert lookup_architecture({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(UnknownArchitecture, match="Qwen2ForCausalLM"):
        lookup_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_config_round_trip_through_a_folder(tmp_path):
    cima_b200.write_random_model(str(tmp_path), TINY_B, seed=3)
    raw = json.load(open(tmp_path / "config.json"))
    assert Qwen2Config.from_dict(raw) == Qwen2Config.from_dict(TINY_B)
    assert Qwen2Config.load(str(tmp_path)) == Qwen2Config.from_dict(TINY_B)
    with pytest.raises(ConfigError, match="cannot read"):
        Qwen2Config.load(str(tmp_path / "nowhere"))


def test_options_table():
    from cima_b200.sampling import GenOptions, OptionError, render_help
    o = GenOptions()
    assert (o.temperature, o.top_k, o.top_p, o.repeat_penalty, o.seed, o.max_tokens) == (0.8, 40, 0.9, 1.1, 0xC0FFEE, 1024)
    o2 = o.set("--temp", "0").set("top-k", "5").set("num_predict", 7).set("n", "9").set("stop", 3).set("stop", "4")
    assert (o2.temperature, o2.top_k, o2.max_tokens, o2.stop) == (0.0, 5, 9, (3, 4))
    assert o.temperature == 0.8                                       # a set makes a copy
    for k, v in [("temperature", "11"), ("top_p", "1.5"), ("repeat_penalty", "0"), ("temperature", "x"),
                 ("ignore_eos", "maybe"), ("nonsense", "1")]:
        with pytest.raises(OptionError):
            o.set(k, v)
    assert o.set("ignore_eos", "true").ignore_eos is True
    assert GenOptions(temperature=0.0, repeat_penalty=1.0).greedy and not GenOptions(temperature=0.0).greedy
    for name in ("temperature", "top-k", "top-p", "repeat-penalty", "seed", "max-tokens", "stop", "ignore-eos"):
        assert "--" + name in render_help()
