"""Configuration: keys, defaults, validation, and the architecture registry."""

import copy
import json

import pytest

from ferrisinfer_b200.config import Qwen2Config, get_architecture, registered_architectures, resolve_config
from ferrisinfer_b200.errors import ConfigError, UnsupportedError
from helpers import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_keys():
    cfg = Qwen2Config.from_dict(TINY_B)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers) == (384, 96, 224, 3)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 1, 32)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and not cfg.tie_word_embeddings
    assert [cfg.layer_window(l) for l in range(3)] == [None, 21, 21]


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "rope_theta", "tie_word_embeddings",
                                                      "use_sliding_window", "sliding_window", "max_window_layers")}
    cfg = Qwen2Config.from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings is False
    assert cfg.head_dim == 16 and cfg.rotary_dim == 16
    assert all(cfg.layer_window(l) is None for l in range(cfg.num_hidden_layers))


def test_null_counts_as_absent_for_optional_keys():
    d = dict(TINY_A, rope_theta=None, num_key_value_heads=None, sliding_window=None)
    cfg = Qwen2Config.from_dict(d)
    assert cfg.rope_theta == 10000.0 and cfg.num_key_value_heads == 4


def test_head_dim_key_and_partial_rotation():
    cfg = Qwen2Config.from_dict(TINY_C)
    assert cfg.head_dim == 48 and cfg.q_size == 240 and cfg.rotary_dim == 24


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_attention_heads", "num_hidden_layers",
                                 "vocab_size", "max_position_embeddings", "rms_norm_eps", "hidden_act", "model_type"])
def test_required_keys(key):
    d = copy.deepcopy(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch, error", [
    ({"num_key_value_heads": 3}, ConfigError),
    ({"hidden_size": 66}, ConfigError),
    ({"vocab_size": 0}, ConfigError),
    ({"rms_norm_eps": 0.0}, ConfigError),
    ({"rope_theta": -1.0}, ConfigError),
    ({"partial_rotary_factor": 0.3}, ConfigError),  # 16 * 0.3 rounds to 5: odd
    ({"hidden_act": "gelu"}, UnsupportedError),
    ({"model_type": "llama"}, UnsupportedError),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, UnsupportedError),
    ({"use_sliding_window": True, "sliding_window": None}, ConfigError),
    ({"vocab_size": "many"}, ConfigError),
    ({"tie_word_embeddings": "yes"}, ConfigError),
    ({"rms_norm_eps": float("inf")}, ConfigError),
])
def test_validation(patch, error):
    with pytest.raises(error):
        Qwen2Config.from_dict(dict(TINY_A, **patch))


def test_round_trip_through_config_json(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg.to_dict()))
    arch, again = resolve_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and again == cfg


def test_registry_names_the_model_by_architecture():
    assert "Qwen2ForCausalLM" in registered_architectures()
    arch = get_architecture("Qwen2ForCausalLM")
    plan = arch.plan(Qwen2Config.from_dict(TINY_B))
    assert len(plan.layers) == 3 and [s.layer for s in plan.run_order] == [0, 1, 2]
    assert plan.layers[0].mixer.params["window"] is None and plan.layers[2].mixer.params["window"] == 21
    with pytest.raises(UnsupportedError, match="Qwen2ForCausalLM"):
        get_architecture("SomethingElseForCausalLM")
    with pytest.raises(ConfigError):
        resolve_config({"model_type": "qwen2"})


def test_bad_json(tmp_path):
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        resolve_config(str(tmp_path))
    with pytest.raises(ConfigError):
        resolve_config(str(tmp_path / "nowhere"))
