"""Configuration: keys, defaults, refusals by field name, registry."""
import copy
import json
import os

import pytest

import helpers as H
from aien_sovereign_core_mv_b200 import ConfigError, model_spec_for
from aien_sovereign_core_mv_b200.config import config_from_hf_dict
from aien_sovereign_core_mv_b200 import registry


def test_every_size_comes_from_config():
    for which, raw in H.TINY.items():
        cfg, spec = model_spec_for(raw)
        assert cfg.hidden_size == raw["hidden_size"] and cfg.vocab_size == raw["vocab_size"]
        assert cfg.head_dim == raw["head_dim"] and cfg.num_key_value_heads == raw["num_key_value_heads"]
        assert cfg.qk_norm == (raw["architectures"][0] == "Qwen3ForCausalLM")
        assert len(spec.layers) == raw["num_hidden_layers"] == len(spec.run_list)
        m = spec.layers[0].mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert {slot: n.params["eps"] for slot, n in spec.layers[0].norms.items()} == {"norm_in": raw["rms_norm_eps"], "norm_post": raw["rms_norm_eps"]}
        assert spec.layers[0].position.params["theta"] == raw["rope_theta"]
        assert spec.head.params["tied"] == raw["tie_word_embeddings"]
        assert cfg.to_hf_dict()["intermediate_size"] == raw["intermediate_size"]


def test_defaults():
    raw = dict(H.TINY["A"])
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "tie_word_embeddings", "eos_token_id"):
        raw.pop(k)
    cfg = config_from_hf_dict(raw)
    assert cfg.num_key_value_heads == cfg.num_attention_heads and cfg.head_dim == 16
    assert cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings is False and cfg.eos_token_ids == ()
    gen = {"eos_token_id": [7, 9]}
    assert config_from_hf_dict(raw, gen).eos_token_ids == (7, 9)       # generation_config.json wins


@pytest.mark.parametrize("change,needle", [
    (dict(architectures=["MistralForCausalLM"]), "unsupported architecture"),
    (dict(architectures=["LlamaForCausalLM", "Qwen3ForCausalLM"]), "architectures"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(use_sliding_window=True), "use_sliding_window"),
    (dict(sliding_window=128), "sliding_window"),
    (dict(layer_types=["full_attention", "sliding_attention"]), "layer_types"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0}), "rope_scaling"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 8.0}), "low_freq_factor"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(rms_norm_eps=0), "rms_norm_eps"),
    (dict(vocab_size=-4), "vocab_size"),
])
def test_refusals_name_the_field(change, needle):
    raw = dict(H.TINY["B"])
    raw.update(change)
    with pytest.raises(ConfigError, match=needle):
        model_spec_for(raw)


def test_missing_required_key_and_qwen3_head_dim():
    for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                "rms_norm_eps", "max_position_embeddings"):
        raw = dict(H.TINY["A"]); raw.pop(key)
        with pytest.raises(ConfigError, match=key):
            model_spec_for(raw)
    raw = dict(H.TINY["B"]); raw.pop("head_dim")
    with pytest.raises(ConfigError, match="head_dim"):
        model_spec_for(raw)
    raw = dict(H.TINY["A"]); raw["head_dim"] = 32                 # Llama: heads * head_dim must equal hidden
    with pytest.raises(ConfigError, match="head_dim"):
        model_spec_for(raw)


def test_strict_mode_refuses_unknown_qwen3_keys():
    raw = dict(H.TINY["B"]); raw["mystery_option"] = 1
    model_spec_for(raw)                                           # lenient by default
    with pytest.raises(ConfigError, match="mystery_option"):
        model_spec_for(raw, strict=True)


def test_llama3_scaling_and_rope_parameters_block():
    cfg, spec = model_spec_for(H.TINY["D"])
    assert cfg.rope_scaling.factor == 8.0 and spec.layers[0].position.params["scaling"]["original_max_position_embeddings"] == 64
    raw = dict(H.TINY["A"]); raw.pop("rope_theta"); raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert config_from_hf_dict(raw).rope_theta == 12345.0


def test_registry_is_open():
    assert set(registry.architecture_names()) >= {"LlamaForCausalLM", "Qwen3ForCausalLM"}
    assert "paged_attention" in registry.part_kinds("mixer") and "swiglu" in registry.part_kinds("feed_forward")
    assert "rmsnorm" in registry.part_kinds("norm") and "rotary" in registry.part_kinds("position")
    with pytest.raises(KeyError, match="no mixer part"):
        registry.make_part("mixer", "does-not-exist")

    @registry.register_architecture("ToyForCausalLM")
    def _build(raw, generation_config=None, strict=False):
        base = dict(raw); base["architectures"] = ["LlamaForCausalLM"]
        return model_spec_for(base)

    raw = dict(H.TINY["A"]); raw["architectures"] = ["ToyForCausalLM"]
    cfg, spec = model_spec_for(raw)
    assert spec.hidden_size == 64


def test_run_list_validation():
    from aien_sovereign_core_mv_b200.config import RunEntry
    import dataclasses
    _, spec = model_spec_for(H.TINY["A"])
    ok = dataclasses.replace(spec, run_list=(RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 1, False)))
    ok.validate()                                                  # a layer twice, a run reading another's cache
    for bad in [(RunEntry(0, 0), RunEntry(1, 0)), (RunEntry(0, 1, False),), (RunEntry(5, 0),)]:
        with pytest.raises(ValueError):
            dataclasses.replace(spec, run_list=bad).validate()
