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


def test_every_random_element_is_a_function_of_seed_name_and_index():
    """The generator is a counter hash into a table of the normal distribution's inverse CDF: integer
    arithmetic and single float32 roundings only, so any device gives the same bits.  Here the torch
    code is checked against the same recipe in plain Python integers."""
    import numpy as np
    from vllm_lite_b200.weights import random_init as R
    name, seed, n = "model.layers.1.self_attn.k_proj.weight", 11, 70_000
    x = R.standard_normal(seed, name, n)
    points, diffs = R._inverse_cdf_table()
    key = R.tensor_key(seed, name)
    for i in (0, 1, 2, 65_535, 65_536, n - 1):
        z = R._mix_python((i + 1) * R._GOLDEN + key)
        cell, frac = z >> 48, (z >> 24) & 0xFFFFFF
        want = np.float32(points[cell]) + np.float32(np.float32(diffs[cell]) * np.float32(frac * 2.0 ** -24))
        assert float(x[i]) == float(want), i
    # a tensor's values do not depend on what else is generated, nor on how the work is cut into pieces
    saved = R.CHUNK
    try:
        R.CHUNK = 1000
        assert torch.equal(R.standard_normal(seed, name, n), x)
    finally:
        R.CHUNK = saved
    assert not torch.equal(R.standard_normal(seed, name + "x", n), x)
    assert not torch.equal(R.standard_normal(seed + 1, name, n), x)
    both = random_tensors(declared("A"), 3)
    alone = random_tensors({"model.norm.weight": declared("A")["model.norm.weight"]}, 3)
    assert torch.equal(both["model.norm.weight"], alone["model.norm.weight"])
    # and it is the distribution it says
    big = R.standard_normal(1, "t", 2_000_000).double()
    assert abs(float(big.mean())) < 3e-3 and abs(float(big.std()) - 1) < 3e-3
    assert abs(float((big ** 4).mean()) - 3) < 0.05 and float(big.abs().max()) < 4.6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,store", [("bfloat16", torch.bfloat16), ("float32", torch.bfloat16), ("float32", torch.float32)])
def test_one_seed_one_model_with_or_without_a_folder(tmp_path, dtype, store):
    """`random_model` (made on the GPU, no file) and a folder written with the same seed and read back
    hold the same tensors bit for bit."""
    from vllm_lite_b200.engine import load_model_dir, random_model
    d = write_model_dir(tmp_path / "m", H.TINY_B, seed=9, std=0.05, dtype=store)
    _, _, from_folder = load_model_dir(d, dtype, "cuda:0")
    _, _, direct = random_model(H.TINY_B, seed=9, dtype=dtype, device="cuda:0", std=0.05, store_dtype=store)
    assert set(from_folder) == set(direct)
    for name in direct:
        assert direct[name].dtype == from_folder[name].dtype, name
        assert torch.equal(direct[name], from_folder[name]), name
