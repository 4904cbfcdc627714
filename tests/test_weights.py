"""Weights: binding by name, the one error that lists everything wrong, dtype rules, the
random-weights mode."""
from __future__ import annotations

import json
import os

import pytest
import torch

from mrun_b200.weights import (WeightsError, bind_tensors, expected_tensors, load_tensors, random_tensors,
                               write_random_model, write_safetensors)
from mrun_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile
from tiny_models import tiny_config


def test_names_and_shapes_follow_the_reference():
    """crates/mrun-engine/src/models/qwen3.rs:75-105, crates/mrun-engine/src/models/common.rs:119-131,327-333."""
    config = tiny_config("B")
    shapes = {t.name: t.shape for t in expected_tensors(config.to_spec())}
    assert shapes["model.embed_tokens.weight"] == (509, 96) and shapes["lm_head.weight"] == (509, 96)
    assert shapes["model.norm.weight"] == (96,)
    p = "model.layers.2"
    assert shapes[f"{p}.self_attn.q_proj.weight"] == (6 * 32, 96)
    assert shapes[f"{p}.self_attn.k_proj.weight"] == (3 * 32, 96) == shapes[f"{p}.self_attn.v_proj.weight"]
    assert shapes[f"{p}.self_attn.o_proj.weight"] == (96, 6 * 32)
    assert shapes[f"{p}.self_attn.q_norm.weight"] == (32,) == shapes[f"{p}.self_attn.k_norm.weight"]
    assert shapes[f"{p}.mlp.gate_proj.weight"] == (200, 96) == shapes[f"{p}.mlp.up_proj.weight"]
    assert shapes[f"{p}.mlp.down_proj.weight"] == (96, 200)
    assert shapes[f"{p}.input_layernorm.weight"] == (96,) == shapes[f"{p}.post_attention_layernorm.weight"]
    assert len([n for n in shapes if not n.endswith('.bias')]) == 2 + 1 + 3 * 11
    tied = {t.name for t in expected_tensors(tiny_config("A").to_spec())}
    assert "lm_head.weight" not in tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    spec = tiny_config("B").to_spec()
    tensors = dict(random_tensors(spec, seed=1))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.scales"] = torch.zeros(192)
    tensors["model.layers.0.self_attn.o_proj.weight"] = torch.zeros(96, 100)
    with pytest.raises(WeightsError) as error:
        bind_tensors(spec, tensors, "a test")
    e = error.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.scales"]
    assert len(e.wrong_shape) == 1 and "o_proj" in e.wrong_shape[0] and "[96, 100]" in e.wrong_shape[0]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text and "wrong shape (1)" in text and "a test" in text


def test_dropped_and_ignored_tensors():
    """A stored head of a tied model and rotary inv_freq buffers are dropped unread
    (crates/mrun-engine/src/models/common.rs:367-369, crates/mrun-engine/src/models/qwen3.rs:107)."""
    spec = tiny_config("A").to_spec()
    tensors = dict(random_tensors(spec, seed=2))
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    # the vision tower and heads for multi-token prediction, too (crates/mrun-engine/src/load.rs:168-173)
    tensors["vision_tower.blocks.0.attn.qkv.weight"] = torch.zeros(3, 3)
    tensors["model.visual.merger.weight"] = torch.zeros(2)
    tensors["model.layers.1.mtp.proj.weight"] = torch.zeros(4, 4)
    bound = bind_tensors(spec, tensors)
    required = [t for t in expected_tensors(spec) if not t.optional]
    assert "lm_head.weight" not in bound and sorted(bound) == sorted(t.name for t in required)


def test_ignored_tensors_are_never_read(tmp_path):
    spec = tiny_config("A").to_spec()
    tensors = dict(random_tensors(spec, seed=2))
    tensors["vision_tower.huge.weight"] = torch.zeros(5, 5)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    read = []
    original = SafetensorsFile.tensor
    def spy(self, name):
        read.append(name)
        return original(self, name)
    SafetensorsFile.tensor = spy
    try:
        load_tensors(str(tmp_path), spec)
    finally:
        SafetensorsFile.tensor = original
    assert "vision_tower.huge.weight" not in read and "model.norm.weight" in read


def test_an_optional_bias_is_bound_when_the_file_has_it():
    """crates/mrun-engine/src/load.rs:281: a linear layer takes ``<path>.bias`` if it is there."""
    spec = tiny_config("B").to_spec()
    tensors = dict(random_tensors(spec, seed=1))
    assert not any(name.endswith(".bias") for name in tensors)            # the random mode makes none
    assert not any(name.endswith(".bias") for name in bind_tensors(spec, tensors))
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
    tensors["model.layers.2.mlp.down_proj.bias"] = torch.ones(96)
    bound = bind_tensors(spec, tensors)
    assert torch.equal(bound["model.layers.2.mlp.down_proj.bias"], torch.ones(96))
    assert "model.layers.0.self_attn.q_proj.bias" in bound and "model.layers.0.self_attn.k_proj.bias" not in bound
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(191)
    with pytest.raises(WeightsError) as error:
        bind_tensors(spec, tensors)
    assert "q_proj.bias" in error.value.wrong_shape[0] and not error.value.missing


def test_storage_dtypes_are_kept(tmp_path):
    spec = tiny_config("A").to_spec()
    tensors = dict(random_tensors(spec, seed=3, dtype=torch.bfloat16))
    name32 = "model.layers.0.input_layernorm.weight"
    name16 = "model.layers.1.mlp.down_proj.weight"
    tensors[name32] = tensors[name32].to(torch.float32)
    tensors[name16] = tensors[name16].to(torch.float16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    loaded = load_tensors(str(tmp_path), spec)
    assert loaded[name32].dtype == torch.float32                 # stored in 32-bit, stays so
    # float16 is widened to 32-bit, exactly: a 32-bit run computes with the stored values, a
    # bfloat16 run narrows the matrix when it goes to the device
    assert loaded[name16].dtype == torch.float32 and torch.equal(loaded[name16], tensors[name16].float())
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert torch.equal(loaded["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"])


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    config = tiny_config("B")
    folder = write_random_model(config, str(tmp_path / "m"), seed=5, std=0.05, norm_noise=0.1)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    cfg = json.load(open(os.path.join(folder, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["hidden_size"] == 96
    from mrun_b200 import registry
    assert registry.load_config(folder) == config
    loaded = load_tensors(folder, config.to_spec())
    again = dict(random_tensors(config.to_spec(), seed=5, std=0.05, norm_noise=0.1))
    other = dict(random_tensors(config.to_spec(), seed=6, std=0.05, norm_noise=0.1))
    for name, tensor in loaded.items():
        assert torch.equal(tensor, again[name]), name             # a seed fixes every value
    assert not torch.equal(loaded["lm_head.weight"], other["lm_head.weight"])
    q = loaded["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(q.std()) - 0.05) < 0.005
    norm = loaded["model.norm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.1 and 0.03 < float(norm.std()) < 0.2
    ones = dict(random_tensors(config.to_spec(), seed=5))["model.norm.weight"]
    assert torch.equal(ones.float(), torch.ones(96))
    # the safetensors package reads what this writer wrote
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(folder, "model.safetensors"))
    assert set(theirs) == set(loaded) and torch.equal(theirs["lm_head.weight"], loaded["lm_head.weight"])


def test_bad_files(tmp_path):
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_tensors(str(tmp_path), tiny_config("A").to_spec())
    bad = tmp_path / "x.safetensors"
    bad.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(bad))
    bad.write_bytes(b"\xff\xff\xff\xff\x00\x00\x00\x00{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(bad))
