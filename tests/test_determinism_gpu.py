"""Bits, not tolerances: the same trace replayed twice in one process and once more in another
process writes the same bytes, in both precisions (crates/mrun-engine/tests/determinism.rs:1-11);
and how far a request's bfloat16 logits move with the requests beside it, reported and bounded,
with the near-tie rule on its greedy tokens (crates/mrun-engine/tests/lanes.rs:68-112 holds the
reference to bit equality there; this engine's bfloat16 kernels are chosen by the step's shape)."""
from __future__ import annotations

import os

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_models import TINY, TOLERANCE, make_folder, random_tokens
from trace_tools import TraceBuilder, TraceRunner, cut_mixed

pytestmark = pytest.mark.gpu


def renamed(steps, suffix, first_step):
    """The same steps for requests with other names, numbered from ``first_step``."""
    out = []
    for i, step in enumerate(steps):
        out.append({"step": first_step + i,
                    "entries": [dict(e, id=e["id"] + suffix) for e in step["entries"]],
                    "end": [rid + suffix for rid in step["end"]]})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "E"])
def test_a_trace_writes_the_same_bytes_twice_and_in_another_process(name, dtype, tmp_path):
    settings = TINY[name]
    folder = make_folder(name, str(tmp_path / "model"))
    vocab = settings["config"]["vocab_size"]
    requests = {f"r{i}": random_tokens(vocab, n, seed=60 + i) for i, n in enumerate([90, 41, 150, 66, 23, 118])}
    b = TraceBuilder()
    cut_mixed(b, requests, [2, 19, 5, 64, 3, 33], live=4, seed=9)
    n = len(b.steps)
    max_tokens = 4 * 192
    first = TraceRunner(folder, dtype, str(tmp_path / "one"), max_tokens, settings["page_size"])
    try:
        first.run(b.steps)
        first.run(renamed(b.steps, "-again", n))          # pages come back in another order the second time
    finally:
        assert first.close() == 0
    second = TraceRunner(folder, dtype, str(tmp_path / "two"), max_tokens, settings["page_size"])
    try:
        second.run(b.steps)
    finally:
        assert second.close() == 0
    compared = 0
    for step in range(n):
        path = os.path.join(str(tmp_path / "one"), f"{step}.f32")
        if not os.path.exists(path):
            continue
        data = open(path, "rb").read()
        assert data == open(os.path.join(str(tmp_path / "one"), f"{step + n}.f32"), "rb").read(), \
            f"{name}/{dtype}: step {step} differs when replayed in the same process"
        assert data == open(os.path.join(str(tmp_path / "two"), f"{step}.f32"), "rb").read(), \
            f"{name}/{dtype}: step {step} differs in a second process"
        compared += 1
    assert compared > 20


@pytest.mark.parametrize("name", ["C", "E"])
def test_bfloat16_logits_beside_other_requests(name, tmp_path):
    """One request decoded alone and beside 1, 7 and 63 others, the same tokens fed every time:
    the largest difference of its logits is reported and stays inside the bfloat16 bound, every
    run is within that bound of the plain implementation, and its greedy token changes only at a
    near-tie of the plain logits."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    settings = TINY[name]
    folder = make_folder(name, str(tmp_path / "model"))
    cfg, weights = plain.load_folder(folder)
    vocab = cfg["vocab_size"]
    target = random_tokens(vocab, 200 + 24, seed=1)
    want = plain.forward(cfg, weights, target).numpy()[200:]
    scale = float(np.abs(want).max())
    others = [random_tokens(vocab, 20 + (37 * i) % 260, seed=100 + i) for i in range(63)]
    ex = executor_from_folder(folder, dtype="bfloat16", page_size=settings["page_size"], num_pages=64 * 24,
                              max_requests=64)

    def run(beside: int) -> np.ndarray:
        live = [ex.admit(("t", beside))] + [ex.admit(("o", beside, i)) for i in range(beside)]
        ex.step([StepEntry(live[0], target[:200], [])])               # its prompt alone, the same every time
        for r, tokens in zip(live[1:], others):
            ex.step([StepEntry(r, tokens[:-1], [])])
        rows = []
        for i in range(24):
            entries = [StepEntry(live[0], [target[200 + i]], [0])]
            entries += [StepEntry(r, [tokens[-1] if i == 0 else 1 + i], [0]) for r, tokens in zip(live[1:], others)]
            ex.decode_step(entries)
            rows.append(ex.decode_logits(entries)[0].float().cpu().numpy())
        for r in live:
            ex.release(r)
        ex.cache.check_invariants()
        return np.stack(rows)

    alone = run(0)
    report = {}
    for beside in (1, 7, 63):
        got = run(beside)
        report[beside] = float(np.abs(got - alone).max()) / scale
        assert float(np.abs(got - want).max()) / scale <= TOLERANCE["bfloat16"], (name, beside)
        for row in range(24):
            if int(np.argmax(got[row])) != int(np.argmax(alone[row])):
                top2 = np.sort(want[row])[-2:]
                assert top2[1] - top2[0] < 0.05 * scale, (name, beside, row, float(top2[1] - top2[0]))
    print(f"{name}: largest change of a request's bfloat16 logits (relative to the largest logit) beside "
          f"1 / 7 / 63 others: {report[1]:.2e} / {report[7]:.2e} / {report[63]:.2e}")
    assert float(np.abs(alone - want).max()) / scale <= TOLERANCE["bfloat16"]
    assert max(report.values()) <= TOLERANCE["bfloat16"]
    assert np.array_equal(run(0), alone)                              # and alone twice: the same bits
