"""Replays the same requests through bin/trace_run cut in every way and compares all logits with
the plain implementation: each request whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; and mixed, up to four live requests, with so
few pages that they are used again.  In 32-bit and in bfloat16, on both tiny configurations."""
from __future__ import annotations

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_models import TOLERANCE, random_tokens
from trace_tools import TraceBuilder, TraceRunner, cut_decode_tail, cut_mixed, cut_portions, cut_whole

LENGTHS = [70, 133, 45, 260, 97, 38, 161]
SIZES = [2, 7, 3, 16, 5, 2, 33, 9, 64, 4]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_matches_plain(tiny, dtype, tmp_path):
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    vocab = cfg["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS)}
    want = {rid: plain.forward(cfg, weights, tokens).numpy() for rid, tokens in requests.items()}

    cuts = {}
    b = TraceBuilder()
    def section(label):
        cuts[label] = len(b.where)
    section("whole")
    for rid in ("r0", "r1", "r3"):
        cut_whole(b, rid, requests[rid])
    section("decode_tail")
    for rid in ("r0", "r3"):
        cut_decode_tail(b, rid, requests[rid])
    section("portions")
    for k, rid in enumerate(("r1", "r2", "r3")):
        cut_portions(b, rid, requests[rid], SIZES[k:] + SIZES[:k])
    section("mixed")
    cut_mixed(b, requests, SIZES, live=4, seed=5)
    section("end")

    # four live requests, each rounded up to 64 tokens: the four longest could be live together
    rounded = sorted((-(-n // 64) * 64 for n in LENGTHS), reverse=True)
    max_tokens = sum(rounded[:4])
    runner = TraceRunner(folder, dtype, str(tmp_path / "out"), max_tokens, settings["page_size"])
    try:
        runner.run(b.steps)
    finally:
        assert runner.close() == 0

    tolerance = TOLERANCE[dtype]
    scale = max(float(np.max(np.abs(w))) for w in want.values())
    files = {}
    worst = {}
    first_seen = {}
    labels = list(cuts)
    for index, (step, row, rid, position) in enumerate(b.where):
        if step not in files:
            files[step] = runner.logits(step, vocab)
        got = files[step][row]
        if dtype == "float32":
            # 32-bit: every reduction runs in an order that depends on the row only, so a
            # position's logits are the same bits however the work was cut and batched
            # (the reference's bar, crates/mrun-engine/tests/lanes.rs:68-112)
            seen = first_seen.setdefault((rid, position), (got, step))
            assert np.array_equal(seen[0], got), (f"{name}: request {rid}, position {position}: steps {seen[1]} "
                                                  f"and {step} differ in bits")
        error = float(np.max(np.abs(got - want[rid][position]))) / scale
        label = [l for l in labels[:-1] if cuts[l] <= index][-1]
        if error > worst.get(label, (0.0,))[0]:
            worst[label] = (error, step, rid, position)
    print({k: f"{v[0]:.2e}" for k, v in worst.items()})
    for label, (error, step, rid, position) in worst.items():
        assert error <= tolerance, (f"{name}/{dtype}/{label}: error {error:.3e} at step {step}, "
                                    f"request {rid}, position {position}")
    assert set(worst) == {"whole", "decode_tail", "portions", "mixed"}
