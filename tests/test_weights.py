import json

import pytest
import torch

import tiny_configs
from torchlet_b200.config import Qwen2Config, load_config
from torchlet_b200.parts import expected_tensors
from torchlet_b200.weights import (WeightsError, check_and_normalise, load_checkpoint, random_tensors,
                                   write_random_model)


def _expected(cfg_dict):
    return expected_tensors(Qwen2Config.from_dict(cfg_dict).model_spec())


def test_expected_names_are_the_checkpoint_names():
    for cfg, _ in tiny_configs.ALL.values():
        names = {t.name: t.shape for t in _expected(cfg) if not t.optional}
        assert names == {n: s for n, s, _ in tiny_configs.tensor_shapes(cfg)}


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    cfg, init = tiny_configs.ALL["B"]
    weights = tiny_configs.make_weights(cfg, **init)
    del weights["model.layers.1.mlp.up_proj.weight"]
    del weights["lm_head.weight"]
    weights["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5)
    weights["model.layers.9.extra.weight"] = torch.zeros(2)
    with pytest.raises(WeightsError) as info:
        check_and_normalise(weights, _expected(cfg))
    err = info.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "lm_head.weight"}
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape[0][0] == "model.layers.0.self_attn.q_proj.weight"
    text = str(err)
    for piece in ("missing", "unexpected", "wrong shape", "lm_head.weight", "(5, 5)", "(96, 96)"):
        assert piece in text


def test_a_tensor_of_a_type_the_engine_does_not_hold_is_named():
    cfg, init = tiny_configs.ALL["A"]
    weights = tiny_configs.make_weights(cfg, **init)
    name, other = "model.layers.0.mlp.down_proj.weight", "model.layers.1.mlp.down_proj.weight"
    weights[name] = weights[name].to(torch.float8_e4m3fn)  # quantized weights are not taken
    weights[other] = weights[other].to(torch.complex64)
    with pytest.raises(WeightsError) as info:
        check_and_normalise(weights, _expected(cfg))
    assert sorted(info.value.wrong_dtype) == sorted([(name, torch.float8_e4m3fn), (other, torch.complex64)])
    assert "unsupported dtype" in str(info.value)


def test_tied_head_may_be_absent_and_dtypes_are_kept():
    cfg, init = tiny_configs.ALL["A"]
    weights = tiny_configs.make_weights(cfg, dtype=torch.bfloat16, **init)
    weights["model.norm.weight"] = weights["model.norm.weight"].float()
    weights["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)  # ignored buffer
    out = check_and_normalise(weights, _expected(cfg))
    assert "lm_head.weight" not in out
    assert out["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert out["model.norm.weight"].dtype == torch.float32


def test_integer_tables_become_int32():
    from torchlet_b200.parts import TensorSpec

    out = check_and_normalise({"t": torch.arange(4, dtype=torch.int64)}, [TensorSpec("t", (4,))])
    assert out["t"].dtype == torch.int32


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = Qwen2Config.from_dict(tiny_configs.TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=9, std=0.03, norm_std=0.02)
    assert load_config(folder) == Qwen2Config.from_dict(json.loads((folder / "config.json").read_text()))
    tensors = load_checkpoint(folder, _expected(tiny_configs.TINY_B))
    assert all(tensors[name].dtype == torch.bfloat16 for name in tensors)
    again = random_tensors(cfg, seed=9, std=0.03, norm_std=0.02)
    other = random_tensors(cfg, seed=10, std=0.03, norm_std=0.02)
    name = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(tensors[name], again[name]) and not torch.equal(tensors[name], other[name])
    norm = tensors["model.norm.weight"].float()
    assert abs(norm.mean() - 1) < 0.02 and 0.005 < norm.std() < 0.05
    assert abs(tensors[name].float().std() - 0.03) < 0.003


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_checkpoint(tmp_path, [])


def test_sharded_checkpoint_with_an_index_and_errors_found_without_reading(tmp_path):
    """Two shards and the table of contents that names them; a stray file the index does not list
    is not read; shapes are checked from the files' headers, tensors are read one at a time."""
    from safetensors.torch import save_file

    from torchlet_b200.weights import LazyCheckpoint

    cfg, init = tiny_configs.ALL["A"]
    weights = tiny_configs.make_weights(cfg, dtype=torch.bfloat16, **init)
    names = sorted(weights)
    shards = {"model-00001-of-00002.safetensors": names[: len(names) // 2],
              "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for file, part in shards.items():
        save_file({n: weights[n].contiguous() for n in part}, str(tmp_path / file))
    save_file({"stray.tensor": torch.zeros(3)}, str(tmp_path / "leftover.safetensors"))
    index = {"metadata": {}, "weight_map": {n: file for file, part in shards.items() for n in part}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    tensors = load_checkpoint(tmp_path, _expected(cfg))
    assert isinstance(tensors, LazyCheckpoint) and set(tensors) == set(names)
    assert tensors.meta("model.embed_tokens.weight") == ((256, 64), torch.bfloat16)
    assert all(torch.equal(tensors[n], weights[n]) for n in names)
    # without the index every file counts, and the stray tensor is reported
    (tmp_path / "model.safetensors.index.json").unlink()
    with pytest.raises(WeightsError) as info:
        load_checkpoint(tmp_path, _expected(cfg))
    assert info.value.unexpected == ["stray.tensor"]
    # an index that names a file that is not there says so
    index["weight_map"][names[0]] = "model-00003-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(FileNotFoundError, match="00003"):
        load_checkpoint(tmp_path, _expected(cfg))
