"""The safetensors container, binding by name and the loader's one error (no GPU)."""
import json
import shutil

import pytest
import torch

import helpers as H
from vllm_lite_b200.config import plan_from_config_json
from vllm_lite_b200.parts import declare_model
from vllm_lite_b200.weights import (SafetensorsFile, WeightError, load_weights, random_tensors, write_model_dir,
                                    write_safetensors)


def declared(which):
    return declare_model(plan_from_config_json(H.TINY[which]["config"])[1])


def test_written_folder_loads_and_round_trips(tmp_path):
    d = write_model_dir(tmp_path / "m", H.TINY_B, seed=5, std=0.05)
    assert json.loads((d / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    w = load_weights(d, declared("B"), torch.bfloat16, "cpu")
    again = random_tensors(declared("B"), 5, 0.05)
    assert set(w) == set(again)
    for name in w:
        assert w[name].dtype == torch.bfloat16
        assert torch.equal(w[name], again[name]), name
    other = random_tensors(declared("B"), 6, 0.05)
    assert not torch.equal(other["lm_head.weight"], again["lm_head.weight"])
    norm = again["model.layers.1.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.1
    assert abs(float(again["lm_head.weight"].float().std()) - 0.05) < 0.005


def test_float32_mode_widens_and_32bit_tensors_stay_32bit(tmp_path):
    tensors = random_tensors(declared("A"), 0)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4     # stored in 32 bits
    (tmp_path / "config.json").write_text(json.dumps(H.TINY_A))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    w16 = load_weights(tmp_path, declared("A"), torch.bfloat16, "cpu")
    assert w16["model.norm.weight"].dtype == torch.float32
    assert torch.equal(w16["model.norm.weight"], tensors["model.norm.weight"])
    assert w16["model.embed_tokens.weight"].dtype == torch.bfloat16
    w32 = load_weights(tmp_path, declared("A"), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    tensors = random_tensors(declared("B"), 1)
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16, dtype=torch.bfloat16)
    tensors["model.layers.2.self_attn.o_proj.weight"] = torch.ones(96, 96, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.ones(3, dtype=torch.bfloat16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.ones(96, 160, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(tmp_path, declared("B"), torch.bfloat16, "cpu")
    err, msg = e.value, str(e.value)
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.self_attn.q_norm.weight",
                                                 "model.layers.2.self_attn.o_proj.weight"}
    assert [n for n, _ in err.wrong_dtype] == ["model.layers.0.mlp.down_proj.weight"]
    for text in ("missing (2)", "unexpected (1)", "[96, 96]", "expected [96, 256]", "I32"):
        assert text in msg


def test_vision_names_are_skipped_and_shards_are_found(tmp_path):
    tensors = random_tensors(declared("A"), 0)
    names = sorted(tensors)
    half = len(names) // 2
    first = {n: tensors[n] for n in names[:half]}
    first["visual.patch_embed.weight"] = torch.ones(2, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", first)
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half:]})
    w = load_weights(tmp_path, declared("A"), torch.bfloat16, "cpu")
    assert set(w) == set(tensors)
    # the same tensor in two shards is reported
    write_safetensors(tmp_path / "model-00003-of-00003.safetensors", {names[0]: tensors[names[0]]})
    with pytest.raises(WeightError) as e:
        load_weights(tmp_path, declared("A"), torch.bfloat16, "cpu")
    assert "duplicate" in str(e.value)


def test_missing_or_broken_files(tmp_path):
    with pytest.raises(WeightError):
        load_weights(tmp_path, declared("A"), torch.bfloat16, "cpu")
    (tmp_path / "model.safetensors").write_bytes(b"\xff" * 20)
    with pytest.raises(WeightError):
        load_weights(tmp_path, declared("A"), torch.bfloat16, "cpu")


def test_container_reader_keeps_dtypes(tmp_path):
    t = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b": torch.tensor([1.5, -2.0], dtype=torch.bfloat16),
         "c": torch.tensor([1, 2, 3], dtype=torch.int32)}
    write_safetensors(tmp_path / "x.safetensors", t)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    for k in t:
        got = f.read(k)
        assert got.dtype == t[k].dtype and torch.equal(got, t[k])
    f.close()
