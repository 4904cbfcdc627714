"""Configuration and registry: keys, defaults and refusals
(as crates/mrun-engine/src/models/registry.rs:382-430 tests them for the reference)."""
from __future__ import annotations

import json

import pytest

from mrun_b200 import registry
from mrun_b200.config import ConfigError, Qwen3Config, UnsupportedArchitecture
from tiny_models import TINY, tiny_config

BASE = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96,
            num_attention_heads=6, num_key_value_heads=3, head_dim=32, intermediate_size=200, vocab_size=509,
            max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=1e6)


def test_reads_every_key_and_round_trips():
    config = Qwen3Config.from_dict(dict(BASE, tie_word_embeddings=True, eos_token_id=[5, 7]))
    assert (config.num_hidden_layers, config.hidden_size, config.num_attention_heads, config.num_key_value_heads,
            config.head_dim, config.intermediate_size, config.vocab_size, config.max_position_embeddings) == \
        (3, 96, 6, 3, 32, 200, 509, 2048)
    assert config.rms_norm_eps == 1e-5 and config.rope_theta == 1e6 and config.tie_word_embeddings
    assert config.eos_token_id == (5, 7)
    assert Qwen3Config.from_dict(config.to_dict()) == config


def test_defaults():
    cfg = {k: v for k, v in BASE.items() if k != "head_dim"}
    config = Qwen3Config.from_dict(cfg)
    assert config.head_dim == 96 // 6                      # hidden / heads when head_dim is absent
    assert config.tie_word_embeddings is False and config.torch_dtype == "bfloat16"
    nested = dict(cfg, rope_parameters={"rope_theta": 5e5, "rope_type": "default"})
    nested.pop("rope_theta")
    assert Qwen3Config.from_dict(nested).rope_theta == 5e5


@pytest.mark.parametrize("change,key", [
    ({"rope_theta": None}, "rope_theta"),
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": "96"}, "hidden_size"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"num_key_value_heads": 4}, "num_key_value_heads"),
    ({"head_dim": 31}, "head_dim"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"layer_types": ["full_attention", "full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention", "full_attention"]}, "layer_types"),
    ({"torch_dtype": "float8"}, "torch_dtype"),
    ({"quantization": {"bits": 4}}, "quantization"),
    ({"vocab_size": 0}, "vocab_size"),
])
def test_refusals_name_the_key(change, key):
    cfg = dict(BASE)
    for k, v in change.items():
        if v is None:
            cfg.pop(k)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError) as error:
        Qwen3Config.from_dict(cfg)
    assert error.value.key == key and key in str(error.value)


def test_registry_picks_the_model_by_name(tmp_path):
    assert registry.resolve({"architectures": ["Qwen3ForCausalLM"]}) is Qwen3Config
    assert registry.resolve({"model_type": "qwen3"}) is Qwen3Config
    with pytest.raises(UnsupportedArchitecture) as error:
        registry.resolve({"model_type": "llama", "architectures": ["LlamaForCausalLM"]})
    assert "qwen3" in str(error.value) and "llama" in str(error.value)
    with pytest.raises(ConfigError):
        registry.resolve({})
    (tmp_path / "config.json").write_text(json.dumps(BASE))
    assert registry.load_config(str(tmp_path)).hidden_size == 96
    with pytest.raises(FileNotFoundError):
        registry.load_config(str(tmp_path / "missing"))


def test_spec_carries_every_constant():
    for name in TINY:
        config = tiny_config(name)
        spec = config.to_spec()
        spec.validate()
        assert len(spec.layers) == config.num_hidden_layers and spec.vocab_size == config.vocab_size
        attention = spec.layers[0].mixer
        assert (attention.heads, attention.kv_heads, attention.head_dim) == \
            (config.num_attention_heads, config.num_key_value_heads, config.head_dim)
        assert attention.softmax_scale == config.head_dim ** -0.5
        assert attention.qk_norm.eps == config.rms_norm_eps and attention.position.theta == config.rope_theta
        assert attention.window is None
        assert spec.layers[0].feed_forward.intermediate == config.intermediate_size
        assert spec.final_norm.eps == config.rms_norm_eps and spec.tie_embeddings == config.tie_word_embeddings
    # 144 KiB per token for the 8B shape (crates/mrun-engine/src/models/registry.rs:305)
    big = Qwen3Config(36, 4096, 32, 8, 128, 12288, 151936, 40960, 1e-6, 1e6)
    assert big.kv_bytes_per_token(2) == 144 * 1024
    assert abs(big.num_parameters() - 8.19e9) < 0.01e9


def test_schedule_validation():
    from mrun_b200.config import ScheduleEntry
    from dataclasses import replace
    spec = tiny_config("A").to_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_of=0))).validate()
    with pytest.raises(ValueError, match="names layer"):
        replace(spec, schedule=(ScheduleEntry(5),)).validate()
    with pytest.raises(ValueError, match="does not run before"):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=0),)).validate()
    with pytest.raises(ValueError, match="owns none"):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(1, cache_of=1))).validate()
