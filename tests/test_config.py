import json

import pytest

import tiny_configs
from torchlet_b200.config import (EngineConfig, Qwen2Config, config_from_dict, known_architectures, load_config,
                                  register_architecture)


def test_defaults_are_the_references():
    cfg = Qwen2Config.from_dict({k: v for k, v in tiny_configs.TINY_A.items()
                                 if k not in ("rope_theta", "rms_norm_eps", "attention_bias", "tie_word_embeddings",
                                              "num_key_value_heads")})
    assert cfg.rope_theta == 1_000_000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.attention_bias is True and cfg.tie_word_embeddings is False
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == 16


def test_rope_parameters_wins_and_registry_selects():
    raw = dict(tiny_configs.TINY_A, rope_parameters={"rope_theta": 5000.0})
    cfg = config_from_dict(raw)
    assert isinstance(cfg, Qwen2Config) and cfg.rope_theta == 5000.0
    assert "Qwen2ForCausalLM" in known_architectures()


def test_unknown_architecture_lists_known():
    with pytest.raises(KeyError, match="Qwen2ForCausalLM"):
        config_from_dict(dict(tiny_configs.TINY_A, architectures=["NopeForCausalLM"]))
    with pytest.raises(ValueError, match="architectures"):
        config_from_dict({k: v for k, v in tiny_configs.TINY_A.items() if k != "architectures"})


@pytest.mark.parametrize("patch, message", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"num_key_value_heads": 8}, "exceed"),
    ({"hidden_size": 66}, "divisible"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"vocab_size": 0}, "positive"),
])
def test_bad_configs_are_refused(patch, message):
    with pytest.raises(ValueError, match=message):
        Qwen2Config.from_dict(dict(tiny_configs.TINY_A, **patch))


def test_missing_required_keys_are_named():
    raw = {k: v for k, v in tiny_configs.TINY_A.items() if k not in ("vocab_size", "intermediate_size")}
    with pytest.raises(ValueError, match="vocab_size.*intermediate_size|intermediate_size.*vocab_size"):
        Qwen2Config.from_dict(raw)


def test_model_spec_layers_follow_the_config():
    cfg = Qwen2Config.from_dict(tiny_configs.TINY_B)
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    windows = [layer.mixer.params["window"] for layer in spec.layers]
    assert windows == [None, 40, 40]
    mixer = spec.layers[0].mixer.params
    assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (3, 1, 32)
    assert mixer["positions"].params["theta"] == 1e6
    assert spec.layers[0].mixer_norm.params["eps"] == 1e-5 and not spec.tie_word_embeddings
    assert cfg.to_dict()["architectures"] == ["Qwen2ForCausalLM"]
    assert Qwen2Config.from_dict(cfg.to_dict()) == cfg


def test_load_config_and_new_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_C))
    cfg = load_config(tmp_path)
    assert cfg.head_dim == 48 and cfg.attention_bias is False

    @register_architecture("ToyConfigOnly")
    class Toy:
        @classmethod
        def from_dict(cls, raw):
            return cls()

    assert isinstance(config_from_dict({"architectures": ["ToyConfigOnly"]}), Toy)
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")


def test_engine_config():
    cfg = EngineConfig(dtype="bf16", max_decode_slots=3, kv_block_size=8).resolve(100)
    assert cfg.dtype == "bfloat16" and cfg.max_seq_len == 100 and cfg.max_num_blocks == 3 * 13 + 1
    with pytest.raises(ValueError):
        EngineConfig(dtype="fp8")
    with pytest.raises(ValueError):
        EngineConfig(max_seq_len=200).resolve(100)
