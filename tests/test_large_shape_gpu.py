"""Real layer sizes against the plain implementation: two layers of the Qwen3-8B, Qwen3-4B and
Qwen3-32B shapes (heads of 128, the full vocabulary of 151,936) with random weights, in 32-bit and
in bfloat16, each sequence whole, most of it in one step and the last 32 tokens one by one through
the captured decode step, and mixed (portions of some requests beside single tokens of others).
The yardstick is ``plain_qwen3`` on the CPU with the same weights, not another path of the engine."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

SHAPES = {
    "8b": dict(num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
               rope_theta=1e6, tie_word_embeddings=False),
    # heads x head size (4096) is not the width (2560), tied head
    "4b": dict(num_hidden_layers=2, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=9728, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
               rope_theta=1e6, tie_word_embeddings=True),
    # eight query heads per kv head (the attention kernels' 16-token tiles and two-stage ring)
    "32b": dict(num_hidden_layers=2, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, vocab_size=151936, max_position_embeddings=8192, rms_norm_eps=1e-6,
                rope_theta=1e6, tie_word_embeddings=False),
}
TOLERANCE = {"float32": 2e-5, "bfloat16": 4e-2}


def plain_rows(cfg, weights, tokens, places):
    """The plain implementation's logits at ``places`` only: the layers over the whole sequence,
    the final norm and the head at the wanted rows (the head over 300 rows of this vocabulary would
    be most of the work)."""
    positions = torch.arange(len(tokens))
    x = weights["model.embed_tokens.weight"][torch.tensor(tokens)]
    for i in range(cfg["num_hidden_layers"]):
        x = plain.decoder_layer(x, weights, i, cfg, positions)
    h = plain.rms_norm(x[torch.tensor(places)], weights["model.norm.weight"], cfg["rms_norm_eps"])
    head = weights["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else weights["lm_head.weight"]
    return (h @ head.T).numpy()


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request):
    """(config, tensors on the device in bfloat16, plain config, plain weights in 32-bit on the host)."""
    from mrun_b200.config import Qwen3Config
    from mrun_b200.weights import random_tensors
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2 ** 30:
        pytest.skip("needs about 30 GB of device memory")
    config = Qwen3Config(**SHAPES[request.param])
    tensors = dict(random_tensors(config.to_spec(), seed=1, std=0.02, norm_noise=0.1, dtype=torch.bfloat16,
                                  device="cuda:0"))
    weights = {name: t.to("cpu", torch.float32) for name, t in tensors.items()}
    yield request.param, config, tensors, config.to_dict(), weights
    del tensors, weights
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_at_real_layer_sizes_matches_plain(shape, dtype):
    from mrun_b200.engine import Executor, StepEntry
    from mrun_b200.kernels import ops
    name, config, tensors, cfg, weights = shape
    ex = Executor(config.to_spec(), tensors, dtype=dtype, page_size=16, num_pages=96, max_requests=8)
    rng = np.random.default_rng(3)
    seqs = {rid: rng.integers(0, config.vocab_size, size=n).tolist() for rid, n in (("a", 300), ("b", 97), ("c", 40))}
    places = {rid: sorted(set(list(range(0, len(t), 29)) + list(range(len(t) - 33, len(t))))) for rid, t in seqs.items()}
    want = {rid: dict(zip(places[rid], plain_rows(cfg, weights, tokens, places[rid]))) for rid, tokens in seqs.items()}
    scale = max(float(np.abs(v).max()) for rows in want.values() for v in rows.values())
    worst = {}

    def check(label, rid, start, positions, logits):
        got = logits.float().cpu().numpy()
        for row, p in enumerate(positions):
            if start + p in want[rid]:
                error = float(np.abs(got[row] - want[rid][start + p]).max()) / scale
                worst[label] = max(worst.get(label, 0.0), error)
                assert error <= TOLERANCE[dtype], (name, dtype, label, rid, start + p, error)

    # whole
    for rid, tokens in seqs.items():
        r = ex.admit(rid)
        check("whole", rid, 0, places[rid], ex.step([StepEntry(r, tokens, places[rid])]))
        ex.release(r)
    # most of it in one step, the last 32 tokens one by one through the captured step
    r = ex.admit("a-tail")
    head = len(seqs["a"]) - 32
    check("tail", "a", 0, range(head), ex.step([StepEntry(r, seqs["a"][:head], range(head))]))
    for i in range(head, len(seqs["a"])):
        entries = [StepEntry(r, [seqs["a"][i]], [0])]
        ex.decode_step(entries)
        check("tail", "a", i, [0], ex.decode_logits(entries))
    ex.release(r)
    assert ex._graphs
    # mixed: three live requests, portions beside single tokens, down to two tokens
    live = {rid: ex.admit(rid + "-mixed") for rid in seqs}
    fed = {rid: 0 for rid in seqs}
    plan = {"a": [200, 1, 1, 50, 1, 47], "b": [1, 90, 1, 1, 4], "c": [7, 1, 2, 29, 1]}
    for turn in range(6):
        entries, names = [], []
        for rid in seqs:
            if turn < len(plan[rid]):
                n = plan[rid][turn]
                entries.append(StepEntry(live[rid], seqs[rid][fed[rid]:fed[rid] + n], range(n)))
                names.append((rid, fed[rid], n))
                fed[rid] += n
        logits = ex.step(entries)
        row = 0
        for rid, start, n in names:
            check("mixed", rid, start, range(n), logits[row:row + n])
            row += n
    assert fed == {rid: len(t) for rid, t in seqs.items()}
    for r in live.values():
        ex.release(r)
    ex.cache.check_invariants()
    ops.tc5_check()
    print(name, dtype, {k: f"{v:.2e}" for k, v in worst.items()})
    assert set(worst) == {"whole", "tail", "mixed"}


def test_batched_greedy_decoding_at_real_layer_sizes_follows_plain(shape):
    """Six prompts through ``Engine.generate`` in bfloat16 (prompt portions, then the pipelined
    captured decode step at batch 6): every token is the plain implementation's, except at
    near-ties (the reference's rule, crates/mrun-engine/tests/conformance.rs:26-27,162-190)."""
    from mrun_b200.engine import Executor
    from mrun_b200.engine.engine import Engine
    name, config, tensors, cfg, weights = shape
    if name != "8b":
        pytest.skip("one shape is enough for the scheduler's path")
    ex = Executor(config.to_spec(), tensors, dtype="bfloat16", page_size=16, num_pages=128, max_requests=8)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, config.vocab_size, size=n).tolist() for n in (33, 120, 64, 17, 250, 9)]
    runs = Engine(ex, max_batch_tokens=256).generate(prompts, max_tokens=8, ignore_eos=True)
    assert ex._graphs and all(len(r.tokens) == 8 for r in runs)
    differing = 0
    for prompt, run in zip(prompts, runs):
        tokens = list(prompt)
        for token in run.tokens:
            logits = plain_rows(cfg, weights, tokens, [len(tokens) - 1])[0]
            best = int(np.argmax(logits))
            if token != best:
                differing += 1
                top2 = np.sort(logits)[-2:]
                assert top2[1] - top2[0] < 0.05 * float(np.abs(logits).max()) and logits[token] >= top2[0], \
                    (name, len(tokens), token, best, float(top2[1] - top2[0]))
            tokens.append(token)
    print("tokens that differ from plain at near-ties:", differing, "of", 8 * len(prompts))
