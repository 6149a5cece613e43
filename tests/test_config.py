"""Configuration and the architecture registry."""

import json

import pytest

from pagedserve_b200.config import (
    ConfigError,
    EngineConfig,
    GPT2Config,
    architecture_names,
    load_model_config,
    resolve_architecture,
)
from pagedserve_b200.config.gpt2 import named_config


def write_config(tmp_path, values):
    (tmp_path / "config.json").write_text(json.dumps(values))
    return str(tmp_path)


def test_reads_architecture_keys(tmp_path):
    values = {"architectures": ["GPT2LMHeadModel"], "n_layer": 3, "n_embd": 96, "n_head": 2, "n_inner": 320,
              "n_positions": 256, "vocab_size": 1000, "layer_norm_epsilon": 1e-6, "activation_function": "gelu",
              "resid_pdrop": 0.1, "bos_token_id": 1}
    config = load_model_config(write_config(tmp_path, values))
    assert isinstance(config, GPT2Config)
    assert (config.n_layer, config.n_embd, config.n_head, config.head_dim) == (3, 96, 2, 48)
    assert config.inner_dim == 320 and config.activation == "gelu_erf"
    assert config.layer_norm_epsilon == 1e-6 and config.max_model_len == 256


def test_defaults_and_null_inner():
    config = GPT2Config.from_dict({"n_embd": 128, "n_head": 4, "n_inner": None})
    assert config.inner_dim == 512 and config.activation == "gelu_tanh" and config.tie_word_embeddings


def test_model_type_fallback_and_unknown(tmp_path):
    name, cls, _ = resolve_architecture({"model_type": "gpt2"})
    assert name == "GPT2LMHeadModel" and cls is GPT2Config
    assert "GPT2LMHeadModel" in architecture_names()
    with pytest.raises(ConfigError, match="unknown architecture"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="names no architecture"):
        resolve_architecture({"hidden_size": 4})
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_config(str(tmp_path))


@pytest.mark.parametrize("bad", [
    {"n_embd": 100, "n_head": 3},
    {"activation_function": "relu"},
    {"add_cross_attention": True},
    {"scale_attn_by_inverse_layer_idx": True},
    {"scale_attn_weights": False},
    {"n_layer": 0},
    {"vocab_size": -1},
    {"n_positions": 64, "n_ctx": 32},
])
def test_refuses_what_it_does_not_compute(bad):
    with pytest.raises(ConfigError):
        GPT2Config.from_dict(bad)


def test_round_trip_and_named():
    config = named_config("tiny-b")
    again = GPT2Config.from_dict(config.to_dict())
    assert again == config
    assert named_config("gpt2-124m").head_dim == 64
    with pytest.raises(ConfigError):
        named_config("gpt5")


def test_engine_config_checks():
    assert EngineConfig().block_size == 16
    for bad in (dict(dtype="float16"), dict(block_size=12), dict(block_size=128), dict(max_num_seqs=0),
                dict(strategy="fifo"), dict(prefill_chunk_size=0), dict(num_blocks=0), dict(kv_cache_memory_mb=0)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)


def test_kv_cache_budget_takes_the_smaller_of_target_and_margin():
    """reference: main.py:48-73 (same arithmetic, same refusals)."""
    from pagedserve_b200.cache.budget import MIB, kv_cache_budget, pages_for_budget

    total, free = 1000 * MIB, 800 * MIB
    # utilisation target: 900 - 200 in use = 700; safety margin: 800 - 50 = 750
    assert kv_cache_budget(free, total, 0.90, 50 * MIB) == int(total * 0.90) - 200 * MIB
    # a large margin decides instead
    assert kv_cache_budget(free, total, 0.90, 300 * MIB) == 500 * MIB
    with pytest.raises(RuntimeError, match="no device memory remains"):
        kv_cache_budget(free, total, 0.90, 800 * MIB)
    with pytest.raises(RuntimeError):
        kv_cache_budget(100 * MIB, total, 0.5, 0)          # already above the target
    for bad in (dict(memory_utilization=0.0), dict(memory_utilization=1.5), dict(safety_memory=-1)):
        with pytest.raises(ValueError):
            kv_cache_budget(free, total, **bad)
    with pytest.raises(ValueError):
        kv_cache_budget(total + 1, total)
    # pages: what the budget affords, but never more than the live requests can hold
    assert pages_for_budget(10 * MIB, 4096, max_num_seqs=4, max_model_len=100, block_size=16) == 4 * 7
    assert pages_for_budget(5 * 4096 + 17, 4096, max_num_seqs=4, max_model_len=100, block_size=16) == 5
    with pytest.raises(ValueError, match="too small"):
        pages_for_budget(4095, 4096, 4, 100, 16)


def test_engine_config_refuses_bad_budget_options():
    for bad in (dict(kv_cache_memory_utilization=0.0), dict(kv_cache_memory_utilization=1.01),
                dict(kv_cache_safety_mb=-1)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)
