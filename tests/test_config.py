"""Configuration and registry (no GPU)."""

import json

import pytest

from somi_inference_b200.config import (ConfigError, Qwen2Config, load_config,
                                        register_architecture, supported_architectures,
                                        unregister_architecture)
from somi_inference_b200.parts import declared_tensors
from tests.tiny import TINY, TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_file():
    c = Qwen2Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (3, 192, 3, 1, 64, 320, 1000)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.max_position_embeddings == 256


def test_from_a_file_or_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert Qwen2Config.from_json(str(tmp_path)) == Qwen2Config.from_json(str(tmp_path / "config.json"))
    assert Qwen2Config.from_json(str(tmp_path)).vocab_size == 1000


def test_head_dim_explicit_wins_over_quotient():
    assert Qwen2Config.from_dict(TINY_C).head_dim == 32       # 80 / 6 is not even an integer
    assert Qwen2Config.from_dict(TINY_A).head_dim == 16


def test_rope_theta_from_rope_parameters():
    d = dict(TINY_A)
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen2Config.from_dict(d).rope_theta == 12345.0


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size",
                                 "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "max_position_embeddings",
                                 "rms_norm_eps", "rope_theta", "tie_word_embeddings"])
def test_missing_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch,msg", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"head_dim": 15}, "even"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"hidden_size": 0}, "positive"),
])
def test_refused_values(patch, msg):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        Qwen2Config.from_dict(d)


def test_window_layers():
    c = Qwen2Config.from_dict(TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [None, 24, 24, 24]
    off = Qwen2Config.from_dict(TINY_A)
    assert all(off.layer_window(i) is None for i in range(2))
    spec = c.to_model_spec()
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 24, 24, 24]


def test_round_trip_and_registry(tmp_path):
    c = Qwen2Config.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    assert "Qwen2ForCausalLM" in supported_architectures()
    bad = dict(TINY_B, architectures=["LlamaForCausalLM"])
    (tmp_path / "config.json").write_text(json.dumps(bad))
    with pytest.raises(ValueError, match="Unsupported architecture.*LlamaForCausalLM"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in bad.items() if k != "architectures"}))
    with pytest.raises(ValueError, match="architectures"):
        load_config(str(tmp_path))


def test_register_another_architecture(tmp_path):
    class Other(Qwen2Config):
        architecture = "OtherForCausalLM"
    register_architecture("OtherForCausalLM", Other)
    try:
        (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["OtherForCausalLM"])))
        assert isinstance(load_config(str(tmp_path)), Other)
    finally:
        unregister_architecture("OtherForCausalLM")


def test_declared_tensors_follow_the_config():
    for name, raw in TINY.items():
        c = Qwen2Config.from_dict(raw)
        d = declared_tensors(c.to_model_spec())
        # the head's matrix is declared for a tied model too, as a copy that is tolerated and ignored
        assert len(d) == 1 + c.num_hidden_layers * 12 + 1 + 1, name
        assert len([x for x in d.values() if not x.ignored]) == \
            1 + c.num_hidden_layers * 12 + 1 + (0 if c.tie_word_embeddings else 1), name
        assert d["model.layers.0.self_attn.k_proj.weight"].shape == (
            c.num_key_value_heads * c.head_dim, c.hidden_size)
        assert d["model.layers.0.mlp.down_proj.weight"].shape == (c.hidden_size, c.intermediate_size)
        assert d["lm_head.weight"].ignored == c.tie_word_embeddings
        assert d["lm_head.weight"].optional == c.tie_word_embeddings


def test_spec_schedule_validation():
    from dataclasses import replace

    from somi_inference_b200.config import RunSpec
    spec = Qwen2Config.from_dict(TINY_A).to_model_spec()
    replace(spec, schedule=(RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(1, cache_of=1))).validate()
    with pytest.raises(ValueError, match="earlier run"):
        replace(spec, schedule=(RunSpec(0, cache_of=1), RunSpec(1))).validate()
    with pytest.raises(ValueError, match="names layer"):
        replace(spec, schedule=(RunSpec(5),)).validate()
    with pytest.raises(ValueError, match="owns no cache"):
        replace(spec, schedule=(RunSpec(0), RunSpec(1, cache_of=0), RunSpec(0, cache_of=1))).validate()
