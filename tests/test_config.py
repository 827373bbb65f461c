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
    ({"hidden_size": 60, "num_attention_heads": 4}, "even"),  # head_dim 15
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"use_sliding_window": True, "sliding_window": 8, "max_window_layers": 5}, "max_window_layers"),
    ({"rope_parameters": {"rope_theta": 1e4, "rope_type": "yarn"}}, "rope_type"),
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
    assert spec.layers[0].norm("mixer_norm").part.params["eps"] == 1e-5 and not spec.tie_word_embeddings
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


def test_tensor_names_come_from_the_layer_description():
    """The architecture-neutral model spells no tensor name: another architecture names its
    parts' tensors as its checkpoint does, and may give a block one norm or three."""
    import dataclasses

    from torchlet_b200.config import NormSlot, PartSpec
    from torchlet_b200.parts import BLOCKS, Block, LayeredModel, expected_tensors

    spec = Qwen2Config.from_dict(tiny_configs.TINY_A).model_spec()
    names = {t.name for t in expected_tensors(spec)}
    assert "model.layers.1.self_attn.q_proj.weight" in names and "model.layers.0.mlp.down_proj.weight" in names
    assert "model.layers.0.input_layernorm.weight" in names

    @BLOCKS.register("toy_one_norm")
    class OneNorm(Block):
        norm_roles = ("shared",)

    norm = spec.layers[0].norms[0].part
    renamed = tuple(
        dataclasses.replace(layer, prefix=f"h.{i}.", block="toy_one_norm", norms=(NormSlot("shared", norm, "ln_1."),),
                            mixer_prefix="attn.", feed_forward_prefix="ffn.")
        for i, layer in enumerate(spec.layers))
    other = dataclasses.replace(spec, layers=renamed, embedding_name="wte.weight", final_norm_prefix="ln_f.",
                                lm_head_name="head.weight")
    names = {t.name for t in expected_tensors(other)}
    assert {"wte.weight", "h.0.ln_1.weight", "h.1.attn.k_proj.bias", "h.0.ffn.up_proj.weight", "ln_f.weight"} <= names
    assert not any("self_attn" in n or "mlp" in n or "layernorm" in n for n in names)
    model = LayeredModel(other)
    assert list(model.blocks[0].norms) == ["shared"]
    # an arrangement that lacks a norm it needs is refused when the model is put together
    broken = dataclasses.replace(other, layers=(dataclasses.replace(renamed[0], norms=()),) + renamed[1:])
    with pytest.raises(ValueError, match="shared"):
        LayeredModel(broken)
    with pytest.raises(KeyError, match="mixer_norm"):
        renamed[0].norm("mixer_norm")


def test_other_spellings_of_config_keys():
    """``dtype`` beside ``torch_dtype``, a list of eos ids, a window without ``max_window_layers``."""
    cfg = Qwen2Config.from_dict(dict(tiny_configs.TINY_A, dtype="bfloat16", eos_token_id=[7, 9]))
    assert cfg.torch_dtype == "bfloat16" and cfg.eos_token_id == 7
    cfg = Qwen2Config.from_dict(dict(tiny_configs.TINY_A, use_sliding_window=True, sliding_window=8))
    assert [layer.mixer.params["window"] for layer in cfg.model_spec().layers] == [8, 8]


def test_a_model_description_that_cannot_run_is_refused():
    import dataclasses

    from torchlet_b200.config import ScheduleEntry

    spec = Qwen2Config.from_dict(tiny_configs.TINY_A).model_spec()
    spec.validate()
    for change, message in [
        ({"layers": ()}, "at least one layer"),
        ({"schedule": ()}, "schedule is empty"),
        ({"schedule": (ScheduleEntry(0, None), ScheduleEntry(2, None))}, "names layer 2"),
        ({"schedule": (ScheduleEntry(0, 0), ScheduleEntry(1, None))}, "earlier entry"),
        ({"schedule": (ScheduleEntry(0, None), ScheduleEntry(1, 0), ScheduleEntry(0, 1))}, "owns no cache"),
    ]:
        with pytest.raises(ValueError, match=message):
            dataclasses.replace(spec, **change).validate()


def test_a_config_json_with_every_key_a_published_folder_carries():
    """The keys of a Qwen2.5 folder's config.json beyond the ones the reference reads
    (v10_triton_paged_gqa/model/qwen2_5.py:25-36): the window keys with the window switched off,
    token ids, a null rope_scaling, bookkeeping keys of the library that wrote the file.  They are
    accepted, the window stays off, and nothing of them changes a size."""
    raw = {"architectures": ["Qwen2ForCausalLM"], "attention_dropout": 0.0, "bos_token_id": 151643, "eos_token_id": 151645,
           "hidden_act": "silu", "hidden_size": 896, "initializer_range": 0.02, "intermediate_size": 4864,
           "max_position_embeddings": 32768, "max_window_layers": 21, "model_type": "qwen2", "num_attention_heads": 14,
           "num_hidden_layers": 24, "num_key_value_heads": 2, "rms_norm_eps": 1e-06, "rope_theta": 1000000.0,
           "sliding_window": 32768, "tie_word_embeddings": True, "torch_dtype": "bfloat16", "transformers_version": "4.43.1",
           "use_cache": True, "use_sliding_window": False, "vocab_size": 151936, "rope_scaling": None}
    cfg = config_from_dict(raw)
    spec = cfg.model_spec()
    assert isinstance(cfg, Qwen2Config) and cfg.head_dim == 64 and cfg.eos_token_id == 151645
    assert len(spec.layers) == 24 and all(layer.mixer.params["window"] is None for layer in spec.layers)
    assert spec.tie_word_embeddings and spec.vocab_size == 151936
    assert Qwen2Config.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
