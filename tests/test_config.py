"""Configuration and the architecture registry (no GPU)."""
import copy

import pytest

import helpers as H
from vllm_lite_b200.config import (ConfigError, InvalidField, MissingField, Qwen3Config, UnknownArchitecture,
                                   plan_from_config_json, register_architecture, registered_architectures,
                                   resolve_architecture, unregister_architecture)
from vllm_lite_b200.parts import cache_needs, declare_model
from vllm_lite_b200.parts.spec import LayerCall, ModelPlan


def test_reads_every_size_from_its_key():
    for which in ("A", "B"):
        src = H.TINY[which]["config"]
        cfg = Qwen3Config.from_dict(src)
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
                    "max_position_embeddings"):
            assert getattr(cfg, key) == src[key], key
        assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_defaults_and_alternate_keys():
    d = copy.deepcopy(H.TINY_A)
    del d["num_key_value_heads"], d["head_dim"], d["rope_theta"]
    d["rotary_base"] = 5000.0
    cfg = Qwen3Config.from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == d["hidden_size"] // d["num_attention_heads"]
    assert cfg.rope_theta == 5000.0
    assert cfg.head_norm_eps == cfg.rms_norm_eps
    d["qk_norm_eps"] = 1e-6
    assert Qwen3Config.from_dict(d).head_norm_eps == 1e-6


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                                 "intermediate_size", "rms_norm_eps", "max_position_embeddings"])
def test_missing_size_is_an_error(key):
    d = copy.deepcopy(H.TINY_B)
    del d[key]
    with pytest.raises(MissingField) as e:
        Qwen3Config.from_dict(d)
    assert key in str(e.value)


@pytest.mark.parametrize("patch", [dict(num_key_value_heads=3), dict(head_dim=15), dict(head_dim=24), dict(head_dim=272),
                                   dict(hidden_size=-4),
                                   dict(vocab_size="many"), dict(attention_bias=True), dict(hidden_act="gelu"),
                                   dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}),
                                   dict(use_sliding_window=True), dict(rms_norm_eps=0.0)])
def test_invalid_values_are_refused(patch):
    d = copy.deepcopy(H.TINY_B)
    d.update(patch)
    with pytest.raises(InvalidField):
        Qwen3Config.from_dict(d)


def test_registry_by_architecture_name():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert resolve_architecture(H.TINY_A).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "Qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(UnknownArchitecture) as e:
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    assert "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(UnknownArchitecture):
        resolve_architecture({})


def test_another_architecture_registers_without_touching_the_framework():
    def plan(cfg):
        base = resolve_architecture(H.TINY_A).plan(cfg)
        return ModelPlan(**{**base.__dict__, "architecture": "ToyTwice",
                            "order": (LayerCall(0), LayerCall(1), LayerCall(1), LayerCall(0, cache_of=0))})
    register_architecture("ToyTwice", Qwen3Config, plan)
    try:
        cfg, p = plan_from_config_json({**H.TINY_A, "architectures": ["ToyTwice"]})
        assert [c.layer for c in p.order] == [0, 1, 1, 0]
        needs = cache_needs(p)
        assert needs[3] is None and needs[0] is not None
        with pytest.raises(KeyError):
            register_architecture("ToyTwice", Qwen3Config, plan)
    finally:
        unregister_architecture("ToyTwice")


def test_plan_holds_the_sizes_and_declares_the_tensors():
    cfg, plan = plan_from_config_json(H.TINY_B)
    block = plan.layers[0]
    assert (block.mixer.num_heads, block.mixer.num_kv_heads, block.mixer.head_dim) == (8, 2, 32)
    assert block.mixer.qk_norm.eps == 1e-5 and block.norm1.eps == 1e-5 and block.mixer.position.theta == 1e6
    assert block.ffn.intermediate_size == 160
    d = declare_model(plan)
    assert d["model.layers.2.self_attn.q_proj.weight"].shape == (256, 96)
    assert d["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert d["lm_head.weight"].shape == (333, 96)
    assert "lm_head.weight" not in declare_model(plan_from_config_json(H.TINY_A)[1])
    assert len(d) == 3 + 3 * 11


def test_order_must_be_consistent():
    _, plan = plan_from_config_json(H.TINY_A)
    bad = ModelPlan(**{**plan.__dict__, "order": (LayerCall(0), LayerCall(5))})
    with pytest.raises(ValueError):
        bad.validate()
    bad = ModelPlan(**{**plan.__dict__, "order": (LayerCall(0, cache_of=0),)})
    with pytest.raises(ValueError):
        bad.validate()
