"""The Qwen3-8B layer sizes (hidden 4096, 32/8 heads of 128, intermediate 12288, vocabulary 151936)
with four layers and random weights: the bfloat16 engine against the engine's true 32-bit path on
the same weights, whole, in portions, token by token through the captured step, and mixed.  The
32-bit path itself is pinned to the plain implementation by the tiny-model tests; here it carries
that yardstick to shapes the plain implementation is too slow for."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engines():
    from mrun_b200.config import Qwen3Config
    from mrun_b200.engine import Executor
    from mrun_b200.weights import random_tensors
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2 ** 30:
        pytest.skip("needs about 40 GB of device memory")
    config = Qwen3Config(num_hidden_layers=4, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                         head_dim=128, intermediate_size=12288, vocab_size=151936, max_position_embeddings=8192,
                         rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    spec = config.to_spec()
    tensors = dict(random_tensors(spec, seed=1, std=0.02, norm_noise=0.1, dtype=torch.bfloat16, device="cuda:0"))
    half = Executor(spec, tensors, dtype="bfloat16", page_size=16, num_pages=256, max_requests=8)
    full = Executor(spec, tensors, dtype="float32", page_size=16, num_pages=256, max_requests=8)
    del tensors
    return config, half, full


def test_bfloat16_follows_the_32_bit_path_under_every_cutting(engines):
    from mrun_b200.engine import StepEntry
    config, half, full = engines
    rng = np.random.default_rng(3)
    seqs = {name: rng.integers(0, config.vocab_size, size=n).tolist() for name, n in (("a", 300), ("b", 97), ("c", 40))}

    # the yardstick: each sequence whole through the 32-bit path, logits at a spread of positions
    places = {name: sorted(set(list(range(0, len(t), 13)) + list(range(len(t) - 34, len(t))))) for name, t in seqs.items()}
    want = {}
    for name, tokens in seqs.items():
        r = full.admit(name)
        want[name] = dict(zip(places[name], full.step([StepEntry(r, tokens, places[name])]).cpu().numpy()))
        full.release(r)
    scale = max(float(np.abs(v).max()) for rows in want.values() for v in rows.values())

    def check(name, start, positions, logits, tolerance=4e-2):
        got = logits.float().cpu().numpy()
        for row, p in enumerate(positions):
            if start + p in want[name]:
                error = float(np.abs(got[row] - want[name][start + p]).max()) / scale
                assert error <= tolerance, (name, start + p, error)

    # 32-bit path against itself in portions: bit-equal rows would be too strict across kernels, 2e-5 is not
    r = full.admit("a-portions")
    at = 0
    for n in (64, 3, 129, 2, 60, 42):
        check("a", at, range(n), full.step([StepEntry(r, seqs["a"][at:at + n], range(n))]), tolerance=2e-5)
        at += n
    full.release(r)

    # bfloat16: whole
    for name, tokens in seqs.items():
        r = half.admit(name)
        check(name, 0, places[name], half.step([StepEntry(r, tokens, places[name])]))
        half.release(r)
    # bfloat16: most of it in one step, the last 32 tokens one by one through the captured step
    r = half.admit("a-tail")
    head = len(seqs["a"]) - 32
    check("a", 0, range(head), half.step([StepEntry(r, seqs["a"][:head], range(head))]))
    for i in range(head, len(seqs["a"])):
        half.decode_step([StepEntry(r, [seqs["a"][i]], [0])])
        check("a", i, [0], half.decode_logits([None]))
    half.release(r)
    # bfloat16: mixed, three live requests, portions beside single tokens
    live = {name: half.admit(name + "-mixed") for name in seqs}
    fed = {name: 0 for name in seqs}
    plan = {"a": [200, 1, 1, 50, 1, 47], "b": [1, 90, 1, 1, 4], "c": [7, 1, 1, 30, 1]}
    for turn in range(6):
        entries, names = [], []
        for name in seqs:
            if turn < len(plan[name]):
                n = plan[name][turn]
                entries.append(StepEntry(live[name], seqs[name][fed[name]:fed[name] + n], range(n)))
                names.append((name, fed[name], n))
                fed[name] += n
        logits = half.step(entries)
        row = 0
        for name, start, n in names:
            check(name, start, range(n), logits[row:row + n])
            row += n
    assert fed == {name: len(t) for name, t in seqs.items()}
    for r in live.values():
        half.release(r)
    half.cache.check_invariants()


def test_greedy_tokens_agree_between_the_precisions(engines):
    """Batched greedy decoding through the pipelined captured step in bfloat16 picks the tokens the
    32-bit path picks, except at near-ties."""
    from mrun_b200.engine.engine import Engine
    config, half, full = engines
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, config.vocab_size, size=n).tolist() for n in (33, 120, 64, 17, 250, 9)]
    a = Engine(half, max_batch_tokens=256).generate(prompts, max_tokens=12, ignore_eos=True)
    b = Engine(full, max_batch_tokens=256).generate(prompts, max_tokens=12, ignore_eos=True)
    assert half._graphs and all(len(x.tokens) == 12 for x in a + b)
    agree = sum(x.tokens[0] == y.tokens[0] for x, y in zip(a, b))
    assert agree >= len(prompts) - 1, [(x.tokens[:3], y.tokens[:3]) for x, y in zip(a, b)]


OTHER_SHAPES = {
    # Qwen3-4B: heads x head size (4096) is not the width (2560), tied head
    "4b": dict(num_hidden_layers=2, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=9728, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
               rope_theta=1e6, tie_word_embeddings=True),
    # Qwen3-32B: eight query heads per kv head (the attention kernels' 16-token tiles and two-stage ring)
    "32b": dict(num_hidden_layers=2, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
                rope_theta=1e6, tie_word_embeddings=False),
}


@pytest.mark.parametrize("shape", sorted(OTHER_SHAPES))
def test_other_layer_shapes_follow_the_32_bit_path(shape):
    """Two layers of the Qwen3-4B and Qwen3-32B shapes: a prompt whole, then tokens one by one
    through the captured step, then a mixed step, bfloat16 against the engine's 32-bit path."""
    from mrun_b200.config import Qwen3Config
    from mrun_b200.engine import Executor, StepEntry
    from mrun_b200.weights import random_tensors
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2 ** 30:
        pytest.skip("needs about 20 GB of device memory")
    config = Qwen3Config(**OTHER_SHAPES[shape])
    spec = config.to_spec()
    tensors = dict(random_tensors(spec, seed=2, std=0.02, norm_noise=0.1, dtype=torch.bfloat16, device="cuda:0"))
    half = Executor(spec, tensors, dtype="bfloat16", page_size=16, num_pages=128, max_requests=4)
    full = Executor(spec, tensors, dtype="float32", page_size=16, num_pages=128, max_requests=4)
    del tensors
    rng = np.random.default_rng(6)
    tokens = rng.integers(0, config.vocab_size, size=330).tolist()
    other = rng.integers(0, config.vocab_size, size=90).tolist()
    head = 300

    def run(ex, captured):
        rows = []
        r = ex.admit("a")
        rows.append(ex.step([StepEntry(r, tokens[:head], [0, 17, head - 1])]).float().cpu().numpy())
        for i in range(head, head + 8):                               # token by token
            if captured:
                ex.decode_step([StepEntry(r, [tokens[i]], [0])])
                rows.append(ex.decode_logits([None]).float().cpu().numpy())
            else:
                rows.append(ex.step([StepEntry(r, [tokens[i]], [0])]).float().cpu().numpy())
        s = ex.admit("b")                                             # a portion beside a single token
        rows.append(ex.step([StepEntry(s, other, [0, 89]), StepEntry(r, [tokens[head + 8]], [0])]).float().cpu().numpy())
        ex.release(r)
        ex.release(s)
        return np.concatenate(rows)

    want, got = run(full, False), run(half, True)
    assert half._graphs
    from mrun_b200.kernels import ops
    ops.tc5_check()
    assert got.shape == want.shape == (3 + 8 + 3, config.vocab_size)
    error = np.abs(got - want).max() / np.abs(want).max()
    assert error <= 4e-2, error
