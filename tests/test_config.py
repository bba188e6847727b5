"""Configuration and registry (no GPU)."""

import json

import pytest

import plain_model
from dryft_flash_infer_b200.config import (ConfigError, Qwen3Config, architecture_named, config_from_dict,
                                           known_architectures, load_config, register_architecture)
from dryft_flash_infer_b200 import models  # noqa: F401
from dryft_flash_infer_b200.engine.model import DecoderModel


def test_reads_the_keys_of_config_json():
    cfg = config_from_dict(plain_model.TINY_B)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 8, 2)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 200, 320)
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False


def test_defaults_follow_the_reference():
    raw = dict(plain_model.TINY_A)
    del raw["head_dim"], raw["rms_norm_eps"]
    cfg = config_from_dict(raw)
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.rms_norm_eps == 1e-6


def test_the_rotation_base_is_read_where_the_file_keeps_it_and_never_guessed():
    raw = dict(plain_model.TINY_A)
    del raw["rope_theta"]
    with pytest.raises(ConfigError, match="rope_theta"):
        config_from_dict(raw)
    newer = dict(raw, rope_parameters={"rope_type": "default", "rope_theta": 123456.0})
    assert config_from_dict(newer).rope_theta == 123456.0
    with pytest.raises(ConfigError, match="rope_type"):
        config_from_dict(dict(raw, rope_parameters={"rope_type": "yarn", "rope_theta": 1e6, "factor": 4.0}))
    assert json.loads(json.dumps(config_from_dict(plain_model.TINY_A).to_dict()))["model_type"] == "qwen3"


def test_round_trip_through_a_folder(tmp_path):
    cfg = config_from_dict(plain_model.TINY_A)
    cfg.save(tmp_path)
    assert load_config(tmp_path) == cfg
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen3ForCausalLM"]


@pytest.mark.parametrize("change, word", [
    ({"architectures": ["NoSuchModel"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"attention_bias": True}, "attention_bias"),
    ({"head_dim": 15}, "head_dim"),
    ({"head_dim": 24}, "head_dim"),
    ({"head_dim": 272}, "head_dim"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
])
def test_bad_configurations_are_named(change, word):
    raw = dict(plain_model.TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(raw)


def test_missing_file(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)


def test_registry_lists_and_takes_new_architectures():
    assert "Qwen3ForCausalLM" in known_architectures()
    entry = architecture_named("Qwen3ForCausalLM")
    register_architecture("ToyForTests", entry.config_class, entry.build)
    assert "ToyForTests" in known_architectures()
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        architecture_named("Nope")


def test_spec_follows_the_configuration_layer_by_layer():
    cfg = config_from_dict(plain_model.TINY_B)
    spec = architecture_named(cfg.architecture).build(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.head_name == "lm_head.weight"
    mixer = spec.layers[0].mixer
    assert mixer.kind == "attention" and mixer.params["head_dim"] == 32 and mixer.params["n_kv_heads"] == 2
    assert mixer.params["position"].params["theta"] == 1e6
    assert spec.layers[0].feed_forward.params["intermediate_size"] == 200
    assert sorted(spec.layers[0].norms) == ["ffn_norm", "mixer_norm"] and spec.layers[0].norms["mixer_norm"].params["eps"] == 1e-5
    model = DecoderModel(spec)
    names = {t.name: t.decl.shape for t in model.expected_tensors()}
    assert names["model.layers.2.self_attn.q_proj.weight"] == (256, 96)
    assert names["model.layers.0.self_attn.k_norm.weight"] == (32,)
    assert names["model.layers.1.mlp.down_proj.weight"] == (96, 200)
    assert names["lm_head.weight"] == (320, 96)
    tied = config_from_dict(plain_model.TINY_A)
    tied_names = [t.name for t in DecoderModel(architecture_named(tied.architecture).build(tied)).expected_tensors()]
    assert "lm_head.weight" not in tied_names
