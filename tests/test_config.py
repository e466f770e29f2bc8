"""Configuration and registry (no GPU)."""
import copy

import pytest

from mdma_b200.config import ConfigError, LlamaConfig, load_config
from mdma_b200.registry import ARCHITECTURES, RegistryError
from tiny import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_the_dictionary():
    for raw in (TINY_A, TINY_B, TINY_C):
        arch, cfg = load_config(raw)
        assert cfg.num_hidden_layers == raw["num_hidden_layers"]
        assert cfg.hidden_size == raw["hidden_size"]
        assert cfg.intermediate_size == raw["intermediate_size"]
        assert cfg.num_attention_heads == raw["num_attention_heads"]
        assert cfg.num_key_value_heads == raw["num_key_value_heads"]
        assert cfg.head_dim == raw["head_dim"]
        assert cfg.vocab_size == raw["vocab_size"]
        assert cfg.rms_norm_eps == raw["rms_norm_eps"]
        assert cfg.rope_theta == raw["rope_theta"]
        assert cfg.tie_word_embeddings == raw["tie_word_embeddings"]
        spec = arch.describe(cfg)
        assert len(spec.layers) == raw["num_hidden_layers"]
        assert [e.layer for e in spec.schedule] == list(range(raw["num_hidden_layers"]))


def test_defaults():
    raw = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rope_layout")}
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.num_key_value_heads == raw["num_attention_heads"]      # llama.rs:27-30
    assert cfg.head_dim == raw["hidden_size"] // raw["num_attention_heads"]
    assert cfg.rope_theta == 10000.0                                  # llama.rs:14
    assert cfg.rope_layout == "split_half"
    assert cfg.rope_scaling is None


def test_llama3_scaling_is_typed():
    cfg = LlamaConfig.from_dict(TINY_B)
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size",
                                 "num_attention_heads", "max_position_embeddings", "vocab_size",
                                 "rms_norm_eps"])
def test_required_keys(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(raw)
    raw[key] = 0
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(raw)


@pytest.mark.parametrize("patch,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"sliding_window": 128}, "sliding_window"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "missing"),
    ({"rope_layout": "spiral"}, "rope_layout"),
    ({"qk_norm": True}, "unimplemented configuration keys"),
    ({"rope_theta": float("nan")}, "rope_theta"),
])
def test_rejects_what_is_not_built(patch, match):
    raw = copy.deepcopy(TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(raw)


def test_unknown_architecture_lists_the_registered_ones():
    raw = copy.deepcopy(TINY_A)
    raw["architectures"] = ["MambaForCausalLM"]
    with pytest.raises(RegistryError) as e:
        load_config(raw)
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)


def test_registry_refuses_duplicates():
    with pytest.raises(RegistryError):
        ARCHITECTURES.register("llama", object())
