"""Configuration and registry (no GPU)."""

import json

import pytest

from jax_vllm_b200 import registry
from jax_vllm_b200.config import EngineConfig, parse_dtype
from jax_vllm_b200.models.qwen3 import Qwen3Config
from tests.util import TINY_A, TINY_B


def test_defaults_follow_reference():
    c = dict(TINY_A)
    cfg = registry.config_from_dict(c)
    assert isinstance(cfg, Qwen3Config)
    assert cfg.head_dim == 64 // 4 and cfg.num_key_value_heads == 2
    c2 = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "rope_theta", "tie_word_embeddings")}
    cfg2 = registry.config_from_dict(c2)
    assert cfg2.num_key_value_heads == 4 and cfg2.rope_theta == 1e6 and cfg2.tie_word_embeddings is False


def test_explicit_head_dim_and_spec():
    cfg = registry.config_from_dict(TINY_B)
    assert cfg.head_dim == 32 and cfg.hidden_size // cfg.num_attention_heads == 16
    spec = cfg.to_spec()
    assert len(spec.layers) == 3 and spec.run_order() == (0, 1, 2)
    m = spec.layers[1].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim) == (6, 1, 32)
    assert abs(m.scale - 32 ** -0.5) < 1e-12 and m.position.theta == 1e6 and m.qk_norm_eps == 1e-5
    assert spec.lm_head_name == "lm_head.weight" and spec.final_norm.eps == 1e-5
    assert registry.config_from_dict(TINY_A).to_spec().lm_head_name is None


def test_missing_keys_and_architecture_errors(tmp_path):
    c = dict(TINY_A); del c["rms_norm_eps"]; del c["vocab_size"]
    with pytest.raises(KeyError) as e:
        registry.config_from_dict(c)
    assert "rms_norm_eps" in str(e.value) and "vocab_size" in str(e.value)
    with pytest.raises(ValueError, match="architectures"):
        registry.config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ValueError, match="unsupported architecture.*Qwen3ForCausalLM"):
        registry.config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(FileNotFoundError):
        registry.config_from_path(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert registry.config_from_path(tmp_path).vocab_size == 384


@pytest.mark.parametrize("extra", [dict(attention_bias=True), dict(rope_scaling={"type": "yarn"}),
                                   dict(use_sliding_window=True), dict(hidden_act="gelu")])
def test_contradicting_keys_are_refused(extra):
    with pytest.raises(ValueError, match="does not do"):
        registry.config_from_dict(dict(TINY_A, **extra))


def test_invalid_sizes():
    with pytest.raises(ValueError, match="multiple"):
        registry.config_from_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ValueError, match="even"):
        registry.config_from_dict(dict(TINY_A, head_dim=15))


def test_round_trip_to_dict():
    cfg = registry.config_from_dict(TINY_B)
    assert registry.config_from_dict(cfg.to_dict()) == cfg


def test_engine_config():
    e = EngineConfig(max_num_seqs=3, max_model_len=100, block_size=16)
    assert e.pages_per_request == 7 and e.pool_pages == 21 and e.prompt_limit == 100
    with pytest.raises(ValueError):
        EngineConfig(max_model_len=64, max_prefill_len=128)
    assert parse_dtype("fp32").is_floating_point and parse_dtype("bfloat16").itemsize == 2
    with pytest.raises(ValueError):
        parse_dtype("fp16")


def test_schedule_and_cache_from_validation():
    from dataclasses import replace
    spec = registry.config_from_dict(TINY_B).to_spec()
    replace(spec, schedule=(0, 1, 1, 2)).validate()
    with pytest.raises(ValueError):
        replace(spec, schedule=(0, 5)).validate()
    layers = list(spec.layers)
    layers[2] = replace(layers[2], cache_from=0)
    replace(spec, layers=tuple(layers)).validate()
    layers[0] = replace(layers[0], cache_from=2)
    with pytest.raises(ValueError):
        replace(spec, layers=tuple(layers)).validate()


def test_pool_sized_by_a_share_of_the_free_memory():
    """With no page count given, `memory_fraction` sizes the pool: what fits into that share of the free memory,
    never more than the worst case, and an error if not even one request of max_model_len would fit."""
    from jax_vllm_b200.config import EngineConfig
    cfg = EngineConfig(max_num_seqs=8, max_model_len=1024, block_size=16, memory_fraction=0.5)
    per_page = 147456 * 16                       # bytes of a 16-token page of the 8B shape
    assert cfg.pages_per_request == 64 and cfg.pool_pages == 512
    assert cfg.pages_for_memory(per_page, 2 * 300 * per_page) == 300
    assert cfg.pages_for_memory(per_page, 1 << 40) == 512                 # capped at the worst case
    with pytest.raises(MemoryError, match="one request of max_model_len needs 64"):
        cfg.pages_for_memory(per_page, 2 * 63 * per_page)
    assert EngineConfig(max_num_seqs=8, max_model_len=1024).pages_for_memory(per_page, 1) == 512    # no fraction: worst case
    with pytest.raises(ValueError, match="memory_fraction"):
        EngineConfig(memory_fraction=1.5)
