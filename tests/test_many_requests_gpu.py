"""Steps with many live requests against the plain implementation: decode steps of 17, 33, 40 and
64 requests (above the rows the decode GEMM takes, through the 32- and 64-row captured steps and
with the decode attention's tiles dealt across pairs), and mixed steps with more than 16 single
tokens beside a prompt portion, through ``bin/trace_run`` and through ``Executor.decode_step``, in
both precisions (crates/mrun-engine/tests/lanes.rs:68-186, crates/mrun/tests/admission.rs)."""
from __future__ import annotations

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_models import TINY, TOLERANCE, make_folder, random_tokens
from trace_tools import TraceBuilder, TraceRunner

pytestmark = pytest.mark.gpu


def lengths_for(n: int):
    return [12 + (53 * i) % 150 for i in range(n)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E"])
def test_traces_with_up_to_64_live_requests(name, dtype, tmp_path):
    settings = TINY[name]
    folder = make_folder(name, str(tmp_path / "model"))
    cfg, weights = plain.load_folder(folder)
    vocab = cfg["vocab_size"]
    tail = 12                                          # tokens every request decodes one by one
    b = TraceBuilder()
    wanted = {}
    most = 0
    for live in (17, 33, 40, 64):
        requests = {f"n{live}-{i}": random_tokens(vocab, n + tail, seed=1000 * live + i)
                    for i, n in enumerate(lengths_for(live))}
        wanted.update(requests)
        most = max(most, sum(-(-len(t) // 64) * 64 for t in requests.values()))
        ids = list(requests)
        fed = {rid: 0 for rid in ids}

        def one_token(rid):
            at = fed[rid]
            fed[rid] += 1
            return (rid, requests[rid][at:at + 1], [0])

        # prompts in groups of seven a step; the requests that already have their prompt decode
        # beside them: up to 57 single tokens next to seven portions in one step
        for start in range(0, live, 7):
            entries = [one_token(rid) for rid in ids[:start]]
            for rid in ids[start:start + 7]:
                n = len(requests[rid]) - tail
                entries.append((rid, requests[rid][:n], [n - 1]))
                fed[rid] = n
            b.step(entries)
        # then everyone decodes side by side; a request that has fed its last token drops out
        while True:
            left = [rid for rid in ids if fed[rid] < len(requests[rid])]
            if not left:
                break
            last = all(fed[rid] + 1 == len(requests[rid]) for rid in left)
            b.step([one_token(rid) for rid in left], end=ids if last else [])
    runner = TraceRunner(folder, dtype, str(tmp_path / "out"), most, settings["page_size"], max_requests=64)
    try:
        runner.run(b.steps)
    finally:
        assert runner.close() == 0
    want = {rid: plain.forward(cfg, weights, tokens).numpy() for rid, tokens in wanted.items()}
    scale = max(float(np.abs(w).max()) for w in want.values())
    files, worst = {}, (0.0, None)
    for step, row, rid, position in b.where:
        if step not in files:
            files[step] = runner.logits(step, vocab)
        error = float(np.max(np.abs(files[step][row] - want[rid][position]))) / scale
        if error > worst[0]:
            worst = (error, (step, rid, position))
    print(f"{name}/{dtype}: worst {worst[0]:.2e} at {worst[1]} over {len(b.where)} rows")
    assert worst[0] <= TOLERANCE[dtype], worst
    assert len(b.where) >= (17 + 33 + 40 + 64) * (tail + 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E"])
@pytest.mark.parametrize("live", [17, 33, 64])
@pytest.mark.parametrize("gemm", ["vendor", "tcgen05"])
def test_captured_decode_steps_of_many_requests(name, dtype, live, gemm, tmp_path, monkeypatch):
    """``decode_step`` (the captured 32- and 64-row steps, sampling inside) with 17, 33 and 64
    requests of different lengths: greedy tokens and logits against the plain implementation;
    with the vendor library's products and with the tcgen05 GEMM (residual sum and norms in its
    epilogues) switched on."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    from mrun_b200.kernels import ops
    if gemm == "tcgen05":
        if dtype != "bfloat16" or name != "E":
            pytest.skip("the tcgen05 GEMM takes bfloat16 products whose k is a multiple of 64")
        monkeypatch.setattr(ops, "TC5_GEMM", True)
    settings = TINY[name]
    folder = make_folder(name, str(tmp_path / "model"))
    cfg, weights = plain.load_folder(folder)
    vocab = cfg["vocab_size"]
    steps = 4
    seqs = [random_tokens(vocab, n + steps, seed=7000 + live * 100 + i) for i, n in enumerate(lengths_for(live))]
    ex = executor_from_folder(folder, dtype=dtype, page_size=settings["page_size"], num_pages=64 * 12,
                              max_requests=64)
    requests = [ex.admit(i) for i in range(live)]
    for start in range(0, live, 9):
        ex.step([StepEntry(r, t[:-steps], []) for r, t in zip(requests[start:start + 9], seqs[start:start + 9])])
    want = [plain.forward(cfg, weights, t).numpy() for t in seqs]
    scale = max(float(np.abs(w).max()) for w in want)
    worst = 0.0
    for s in range(steps):
        entries = [StepEntry(r, [t[len(t) - steps + s]], [0]) for r, t in zip(requests, seqs)]
        tokens = ex.decode_step(entries).tolist()
        logits = ex.decode_logits(entries).float().cpu().numpy()
        for i, t in enumerate(seqs):
            row = want[i][len(t) - steps + s]
            error = float(np.abs(logits[i] - row).max()) / scale
            worst = max(worst, error)
            assert error <= TOLERANCE[dtype], (name, dtype, live, s, i, error)
            if tokens[i] != int(np.argmax(row)):
                top2 = np.sort(row)[-2:]
                assert top2[1] - top2[0] < (1e-3 if dtype == "float32" else 0.05 * scale), (i, s)
    assert ex._graphs and max(ex._graphs) >= (32 if live <= 32 else 64)
    for r in requests:
        ex.release(r)
    ex.cache.check_invariants()
    print(f"{name}/{dtype}/{live}: worst {worst:.2e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forty_requests_through_the_entry_point(dtype, tmp_path):
    """``Engine.generate`` with 40 prompts live at once: prompt portions beside up to 39 decoding
    requests, then the pipelined 64-row captured step; every request's tokens are the plain
    implementation's (bfloat16: up to near-ties), and everything is given back."""
    from mrun_b200 import Engine
    from test_engine_gpu import plain_tokens_match
    name = "E"
    settings = TINY[name]
    folder = make_folder(name, str(tmp_path / "model"))
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=9000 + i) for i, n in enumerate(lengths_for(40))]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=40 * 192,
                                max_batch_tokens=96, max_requests=64)
    runs = engine.generate(prompts, max_tokens=48, ignore_eos=True)      # long enough for all 40 to decode side by side
    assert max(engine.executor._graphs) == 64
    for prompt, run in zip(prompts, runs):
        assert run.finish_reason == "length" and len(run.tokens) == 48
        plain_tokens_match(cfg, weights, prompt, run.tokens, margin=1e-3 if dtype == "float32" else 0.05)
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live and engine.executor.cache.free_pages() == engine.executor.cache.num_pages
