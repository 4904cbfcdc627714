"""The plain implementation checked against itself and against hand-worked values: it is the
yardstick of every GPU test, so its parts are pinned here on the CPU."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from mrun_b200.sampling import draw_key, mix64
from tiny_models import TINY, make_folder, random_tokens


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    got = plain.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(got, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]]))
    assert torch.allclose(plain.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-6), torch.zeros(1, 4))


def test_rope_by_hand_and_properties():
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0]]])               # one token, one head, D = 4: pairs (0,2), (1,3)
    out = plain.rope(x, torch.tensor([1]), theta=100.0)
    a0, a1 = 1.0, 1.0 * 100.0 ** (-2 / 4)
    want = [math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1)]
    assert torch.allclose(out[0, 0], torch.tensor(want), atol=1e-6)
    assert torch.equal(plain.rope(x, torch.tensor([0]), 100.0), x)          # position 0 is the identity
    # scores depend on the distance only
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 16, generator=g), torch.randn(1, 1, 16, generator=g)
    dot = lambda pq, pk: float((plain.rope(q, torch.tensor([pq]), 1e4) * plain.rope(k, torch.tensor([pk]), 1e4)).sum())
    assert abs(dot(5, 2) - dot(105, 102)) < 1e-4
    # partial rotation leaves the tail alone
    part = plain.rope(torch.ones(1, 1, 8), torch.tensor([3]), 1e4, rotary_dim=4)
    assert torch.equal(part[0, 0, 4:], torch.ones(4))


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    L, nh, nkv, D = 6, 4, 2, 8
    q, k, v = torch.randn(L, nh, D, generator=g), torch.randn(L, nkv, D, generator=g), torch.randn(L, nkv, D, generator=g)
    pos = torch.arange(L)
    out = plain.attention_scores_softmax_values(q, k, v, D ** -0.5, pos)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])    # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0
    again = plain.attention_scores_softmax_values(q, k2, v2, D ** -0.5, pos)
    assert torch.allclose(out[:4], again[:4])                               # later keys do not matter
    v3 = v.clone()
    v3[:, 1] += 1.0
    moved = plain.attention_scores_softmax_values(q, k, v3, D ** -0.5, pos)
    assert torch.allclose(moved[:, :2], out[:, :2]) and torch.allclose(moved[:, 2:], out[:, 2:] + 1.0, atol=1e-5)
    windowed = plain.attention_scores_softmax_values(q, k, v, D ** -0.5, pos, window=1)
    assert torch.allclose(windowed[:, 0], v[:, 0])                          # a window of one: the token itself
    assert torch.allclose(plain.attention_scores_softmax_values(q, k, v, D ** -0.5, pos, window=100), out)


def test_swiglu_by_hand():
    w = {"m.gate_proj.weight": torch.tensor([[1.0]]), "m.up_proj.weight": torch.tensor([[2.0]]),
         "m.down_proj.weight": torch.tensor([[3.0]])}
    got = plain.swiglu_mlp(torch.tensor([[0.5]]), w, "m")
    silu = 0.5 / (1 + math.exp(-0.5))
    assert abs(float(got) - silu * 1.0 * 3.0) < 1e-6


@pytest.mark.parametrize("name", sorted(TINY))
def test_forward_is_causal_and_deterministic(name, tmp_path):
    folder = make_folder(name, str(tmp_path / name))
    cfg, weights = plain.load_folder(folder)
    assert cfg["hidden_size"] == TINY[name]["config"]["hidden_size"]
    tokens = random_tokens(cfg["vocab_size"], 24, seed=3)
    full = plain.forward(cfg, weights, tokens)
    assert full.shape == (24, cfg["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(plain.forward(cfg, weights, tokens[:10]), full[:10], atol=2e-5)
    changed = tokens[:]
    changed[20] = (changed[20] + 1) % cfg["vocab_size"]
    assert torch.allclose(plain.forward(cfg, weights, changed)[:20], full[:20], atol=2e-5)
    assert not torch.allclose(plain.forward(cfg, weights, changed)[20:], full[20:], atol=1e-3)
    # logits have a scale at which errors of a few percent are visible
    assert 0.05 < float(full.abs().max()) < 50


def test_sampling_generator_and_filters():
    assert plain.mix64(0) == mix64(0) and plain.mix64(12345) == mix64(12345)
    assert mix64(0) == 0xE220A8397B1DCDAF                                  # SplitMix64's first output for seed 0
    assert plain.draw_key(7, 3) == draw_key(7, 3) and draw_key(7, 3) != draw_key(7, 4)
    noise = plain.gumbel_noise(draw_key(1, 1), 20000)
    assert abs(float(noise.mean()) - 0.5772) < 0.03 and abs(float(noise.var()) - math.pi ** 2 / 6) < 0.08
    logits = np.log(np.array([0.5, 0.2, 0.15, 0.1, 0.05], dtype=np.float32))
    assert plain.filter_threshold(logits, top_p=0.6).tolist() == [True, True, False, False, False]
    assert plain.filter_threshold(logits, top_p=0.5).tolist() == [True, False, False, False, False]
    assert plain.filter_threshold(logits, top_k=3).tolist() == [True, True, True, False, False]
    assert plain.filter_threshold(logits, min_p=0.25).tolist() == [True, True, True, False, False]
    assert plain.sample_token(logits, 0.0) == 0
    counts = np.bincount([plain.sample_token(logits, 1.0, draw_key(9, n)) for n in range(1, 4001)], minlength=5)
    assert np.allclose(counts / 4000, [0.5, 0.2, 0.15, 0.1, 0.05], atol=0.03)
    penalised = plain.apply_repetition_penalty(np.array([2.0, -2.0, 1.0], dtype=np.float32), [0, 1, 1], 2.0)
    assert penalised.tolist() == [1.0, -4.0, 1.0]
