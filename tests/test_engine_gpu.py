"""Generation through the Python entry point against the plain implementation: greedy and
temperature sampling, captured decode steps beside eager mixed steps, the first tokens of a
sequence, long decoding."""
from __future__ import annotations

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_models import TOLERANCE, random_tokens, rel_error

pytestmark = pytest.mark.gpu


def plain_tokens_match(cfg, weights, prompt, got, temperature=0.0, seed=0, margin=1e-3):
    """Follows the engine's tokens with the plain implementation; a difference is accepted only at
    a near-tie: the plain score of the engine's token is within ``margin`` of the best plain score
    (the reference's rule for its own comparisons is a top-2 margin below 1e-3,
    crates/mrun-engine/tests/conformance.rs:26-27,162-190; with three candidates inside the margin
    any of them may win)."""
    tokens = list(prompt)
    for n, token in enumerate(got, start=1):
        logits = plain.forward(cfg, weights, tokens)[-1].numpy()
        if temperature == 0.0:
            score = logits
        else:
            score = logits * np.float32(1.0 / temperature) + plain.gumbel_noise(plain.draw_key(seed, n), len(logits))
        want = int(np.argmax(score))
        if token != want:
            assert score[want] - score[token] < margin, \
                f"token {n}: engine {token}, plain {want}, behind by {score[want] - score[token]:.4f}"
        tokens.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(tiny, dtype):
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=n) for n in (1, 9, 40, 71)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=1024,
                                max_batch_tokens=7, max_requests=4)
    streamed = {i: [] for i in range(len(prompts))}
    results = engine.generate(prompts, max_tokens=12, ignore_eos=True,
                              on_token=lambda i, token: streamed[i].append(token))
    assert engine.executor._graphs, "decode steps should have gone through a captured graph"
    assert [streamed[i] for i in range(len(prompts))] == [r.tokens for r in results]
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and len(result.tokens) == 12
        margin = 1e-3 if dtype == "float32" else 0.05
        plain_tokens_match(cfg, weights, prompt, result.tokens, margin=margin)
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live


def test_temperature_sampling_matches_plain_draws(tiny):
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=50 + n) for n in (5, 17, 33)]
    engine = Engine.from_folder(folder, dtype="float32", page_size=settings["page_size"], context=512,
                                max_batch_tokens=16, max_requests=4)
    first = engine.generate(prompts, max_tokens=12, temperature=0.8, seed=1234, ignore_eos=True)
    again = engine.generate(prompts, max_tokens=12, temperature=0.8, seed=1234, ignore_eos=True)
    other = engine.generate(prompts, max_tokens=12, temperature=0.8, seed=99, ignore_eos=True)
    assert [r.tokens for r in first] == [r.tokens for r in again]
    assert [r.tokens for r in first] != [r.tokens for r in other]
    for i, (prompt, result) in enumerate(zip(prompts, first)):
        plain_tokens_match(cfg, weights, prompt, result.tokens, temperature=0.8, seed=1234 + i)


def test_long_decoding_stays_on_the_plain_logits(tiny):
    """300 decode steps one by one (captured graph), logits checked against whole-sequence plain."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    tokens = random_tokens(cfg["vocab_size"], 330, seed=77)
    want = plain.forward(cfg, weights, tokens).numpy()
    for dtype in ("float32", "bfloat16"):
        ex = executor_from_folder(folder, dtype=dtype, page_size=settings["page_size"], num_pages=max(64, 352 // settings["page_size"]),
                                  max_requests=2)
        request = ex.admit("long")
        first = ex.step([StepEntry(request, tokens[:30], [0, 1, 2, 29])]).cpu().numpy()
        assert rel_error(first, want[[0, 1, 2, 29]]) <= TOLERANCE[dtype]       # the first tokens of a sequence
        worst = 0.0
        for i in range(30, 330):
            ex.decode_step([StepEntry(request, [tokens[i]], [0])])
            got = ex.decode_logits([None])[0].cpu().numpy()
            worst = max(worst, float(np.max(np.abs(got - want[i])) / np.max(np.abs(want))))
        assert worst <= TOLERANCE[dtype], (dtype, worst)
        ex.release(request)
        ex.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_end_tokens_stop_requests_in_the_middle_of_pipelined_decoding(tiny, dtype):
    """Decode steps are launched before the tokens of the step before them are read.  A request
    that samples an end token has then already been given a row in the next step: that row's
    token must be dropped, the other requests must go on unchanged, and everything must be freed.
    The end token itself is not part of the output."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=200 + n) for n in (6, 11, 19, 25, 3)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=1024,
                                max_batch_tokens=64, max_requests=8)
    free = engine.generate(prompts, max_tokens=40, ignore_eos=True)
    assert all(len(r.tokens) == 40 for r in free)
    # an end token that stops some requests early and at different steps
    counts = {}
    for r in free:
        for t in set(r.tokens[3:30]):
            counts[t] = counts.get(t, 0) + 1
    eos = max(counts, key=lambda t: (counts[t], t))
    engine.eos_token_ids = (eos,)
    stopped = engine.generate(prompts, max_tokens=40)
    reasons = set()
    for prompt, before, after in zip(prompts, free, stopped):
        assert eos not in after.tokens
        if dtype == "float32":                      # 32-bit logits do not depend on the batch: the same tokens
            if eos in before.tokens:
                cut = before.tokens.index(eos)
                assert after.tokens == before.tokens[:cut] and after.finish_reason == "stop"
            else:
                assert after.tokens == before.tokens and after.finish_reason == "length"
        else:                                       # bfloat16: the plain tokens up to near-ties, the end token last
            ended = [eos] if after.finish_reason == "stop" else []
            plain_tokens_match(cfg, weights, prompt, after.tokens + ended, margin=0.05)
            assert after.finish_reason == "stop" or len(after.tokens) == 40
        reasons.add(after.finish_reason)
    assert "stop" in reasons
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live and engine.executor.cache.free_pages() == engine.executor.cache.num_pages
    # different output limits: each request leaves the pipeline at its own step
    limits = engine.generate(prompts[:3], max_tokens=7, ignore_eos=True) + engine.generate(prompts[3:], max_tokens=1, ignore_eos=True)
    for prompt, before, after in zip(prompts, free, limits):
        if dtype == "float32":
            assert after.tokens == before.tokens[:len(after.tokens)]
        else:
            plain_tokens_match(cfg, weights, prompt, after.tokens, margin=0.05)
        assert after.finish_reason == "length"
    assert [len(r.tokens) for r in limits] == [7, 7, 7, 1, 1]


def test_cancelling_one_request_leaves_the_others_as_they_were(tiny):
    """``on_token`` returning False cancels that prompt in the middle of pipelined decoding: it
    keeps what it had, the token in flight for it is dropped, and the other prompts' tokens are
    those of an undisturbed run (crates/mrun-engine/tests/tiny_qwen3.rs:193-211)."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=600 + n) for n in (14, 5, 30)]
    engine = Engine.from_folder(folder, dtype="float32", page_size=settings["page_size"], context=512,
                                max_batch_tokens=32, max_requests=4)
    free = engine.generate(prompts, max_tokens=20, ignore_eos=True)
    seen = []
    def on_token(i, token):
        seen.append((i, token))
        return not (i == 1 and sum(1 for j, _ in seen if j == 1) == 6)
    cut = engine.generate(prompts, max_tokens=20, ignore_eos=True, on_token=on_token)
    assert cut[1].finish_reason == "cancelled" and cut[1].tokens == free[1].tokens[:6]
    assert cut[0].tokens == free[0].tokens and cut[2].tokens == free[2].tokens
    assert cut[0].finish_reason == cut[2].finish_reason == "length"
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live and engine.executor.cache.free_pages() == engine.executor.cache.num_pages


def test_stop_sequences_end_requests_in_the_middle_of_pipelined_decoding(tiny):
    """``stop=`` through ``Engine.generate``: each prompt ends where its own free-running output
    would contain a stop sequence (taken from those outputs), without the sequence; the token in
    flight for it is dropped, the others go on unchanged, what was held back reaches ``on_token``
    in order, and everything is given back (the reference's ``--stop``, on token ids:
    crates/mrun/src/chat/stop.rs:24-85)."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=700 + n) for n in (9, 21, 4)]
    engine = Engine.from_folder(folder, dtype="float32", page_size=settings["page_size"], context=512,
                                max_batch_tokens=32, max_requests=4)
    free = engine.generate(prompts, max_tokens=24, ignore_eos=True)
    stops = [free[0].tokens[7:10], free[1].tokens[15:16]]
    def first_end(tokens):
        ends = [(i + len(s), s) for s in stops for i in range(len(tokens) - len(s) + 1) if tokens[i:i + len(s)] == s]
        return min(ends, key=lambda e: (e[0], -len(e[1]))) if ends else None
    seen = {0: [], 1: [], 2: []}
    cut = engine.generate(prompts, max_tokens=24, ignore_eos=True, stop=stops, on_token=lambda i, t: seen[i].append(t))
    stopped = 0
    for i, (a, b) in enumerate(zip(free, cut)):
        end = first_end(a.tokens)
        if end is None:
            assert b.tokens == a.tokens and b.finish_reason == "length" and b.stop_sequence is None
        else:
            stopped += 1
            assert b.finish_reason == "stop" and b.stop_sequence == end[1]
            assert b.tokens == a.tokens[:end[0] - len(end[1])]
        assert seen[i] == b.tokens and len(b.token_times) == len(b.tokens)
    assert stopped >= 2
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live and engine.executor.cache.free_pages() == engine.executor.cache.num_pages
    with pytest.raises(ValueError, match="at most 4 stop sequences"):
        engine.generate(prompts, max_tokens=2, stop=[[1]] * 5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_cut_back_goes_on_as_if_it_had_never_been_longer(tiny, dtype):
    """``Executor.trim``: 40 tokens fed, the request cut back to 17 (and once to a page's edge),
    another continuation fed in portions and decoded: the logits equal the plain implementation
    on the first tokens + the continuation, and in 32-bit they are the bits of a fresh request
    that was fed the same tokens in the same steps; the pages beyond the cut went back and are
    used again meanwhile (crates/mrun-engine/tests/tiny_qwen3.rs:213-245, trim exact)."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.loading import executor_from_folder
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    vocab, page = cfg["vocab_size"], settings["page_size"]
    ex = executor_from_folder(folder, dtype=dtype, page_size=page, num_pages=-(-256 // page), max_requests=4)
    first = random_tokens(vocab, 40, seed=31)
    other = random_tokens(vocab, 21, seed=32)
    for cut in (17, 2 * page):
        a = ex.admit(("cut", cut))
        ex.step([StepEntry(a, first, [])])
        free_before = ex.cache.free_pages()
        ex.trim(a, cut)
        assert a.length == cut and ex.cache.free_pages() == free_before + (-(-40 // page)) - (-(-cut // page))
        filler = ex.admit(("filler", cut))                       # takes the pages that came back
        ex.step([StepEntry(filler, random_tokens(vocab, 3 * page, seed=33), [])])
        b = ex.admit(("fresh", cut))
        ex.step([StepEntry(b, first[:cut], [])])
        got_a, got_b = [], []
        for lo, hi in ((0, 9), (9, 11), (11, 20), (20, 21)):
            want_rows = list(range(hi - lo))
            out = ex.step([StepEntry(a, other[lo:hi], want_rows), StepEntry(b, other[lo:hi], want_rows)])
            rows = out.float().cpu().numpy()
            got_a.append(rows[:hi - lo]); got_b.append(rows[hi - lo:])
        got_a, got_b = np.concatenate(got_a), np.concatenate(got_b)
        want = plain.forward(cfg, weights, first[:cut] + other).numpy()[cut:]
        scale = float(np.abs(want).max())
        assert float(np.abs(got_a - want).max()) / scale <= TOLERANCE[dtype]
        if dtype == "float32":
            assert np.array_equal(got_a, got_b)
        else:
            assert float(np.abs(got_a - got_b).max()) / scale <= TOLERANCE[dtype]
        for r in (a, b, filler):
            ex.release(r)
        ex.cache.check_invariants()
        assert ex.cache.free_pages() == ex.cache.num_pages


def test_constrained_decoding_with_token_masks(tiny):
    """``allowed_tokens`` through ``Engine.generate``: a prompt that decodes under a mask that
    changes with every token (beside an unconstrained one in the same batch) gives the tokens of
    a host-side replay on the plain logits, greedy and drawn; the unconstrained prompt is as it
    was; a mask that allows nothing, and one wider than the logits, end their prompt with the
    reference's messages (crates/mrun-engine/src/sample.rs:88-116, engine.rs:571-576)."""
    from mrun_b200 import Engine, TokenMask
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    vocab = cfg["vocab_size"]
    prompts = [random_tokens(vocab, n, seed=800 + n) for n in (11, 6)]
    engine = Engine.from_folder(folder, dtype="float32", page_size=settings["page_size"], context=512,
                                max_batch_tokens=32, max_requests=4)
    def allowed(n):                       # the tokens allowed for the n-th output token: a moving window plus one far token
        return sorted({(7 * n + j) % vocab for j in range(9)} | {vocab - 1 - n})
    calls = []
    def constraint(i, output):
        calls.append((i, len(output)))
        if i != 0:
            return None
        return TokenMask.of(allowed(len(output)), vocab) if len(output) % 2 else allowed(len(output))
    free = engine.generate(prompts, max_tokens=10, ignore_eos=True)
    for temperature, seed in ((0.0, None), (0.9, 4)):
        runs = engine.generate(prompts, max_tokens=10, ignore_eos=True, temperature=temperature, seed=seed,
                               top_p=0.95 if temperature else 1.0, allowed_tokens=constraint)
        tokens = list(prompts[0])
        for n, token in enumerate(runs[0].tokens):
            logits = plain.apply_token_mask(plain.forward(cfg, weights, tokens)[-1].numpy(), allowed(n))
            want = plain.sample_token(logits, temperature, plain.draw_key(seed or 0, n + 1), top_p=0.95 if temperature else 1.0)
            assert token == want and token in allowed(n), (temperature, n, token, want)
            tokens.append(token)
        assert len(runs[0].tokens) == 10 and runs[0].finish_reason == "length"
        if temperature == 0.0:
            assert runs[1].tokens == free[1].tokens
    assert (0, 0) in calls and (0, 9) in calls and (1, 3) in calls
    # masks that cannot be used
    nothing = engine.generate(prompts, max_tokens=6, ignore_eos=True,
                              allowed_tokens=lambda i, output: TokenMask.none_allowed(vocab) if i == 0 and len(output) == 3 else None)
    assert nothing[0].finish_reason == "invalid" and nothing[0].message == "the token mask allows no token"
    assert nothing[0].tokens == free[0].tokens[:3] and nothing[1].tokens == free[1].tokens[:6]
    wide = engine.generate(prompts[:1], max_tokens=6, ignore_eos=True,
                           allowed_tokens=lambda i, output: TokenMask.of([1], vocab + 1))
    assert wide[0].finish_reason == "invalid" and f"wider than the model's {vocab} logits" in wide[0].message
    engine.executor.cache.check_invariants()
    assert not engine.executor.cache.live and engine.executor.cache.free_pages() == engine.executor.cache.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repetition_penalty_and_filters_through_generate(tiny, dtype):
    """Sampling settings that need the token history (the penalty) keep decoding correct: the
    tokens equal a host-side replay of the same rule on the plain logits, for a request that
    decodes beside an unpenalised greedy one in the same batch.  bfloat16: a token may differ
    where the plain scores of the two candidates are within the bfloat16 bound of each other."""
    from mrun_b200 import Engine, SamplingParams
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    prompt = random_tokens(cfg["vocab_size"], 12, seed=5)
    other = random_tokens(cfg["vocab_size"], 7, seed=6)
    engine = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=256, max_requests=2)
    params = SamplingParams(temperature=0.9, top_k=12, top_p=0.95, min_p=0.01, seed=77, repetition_penalty=1.4)
    runs = engine.generate([prompt, other], max_tokens=10, sampling=[params, SamplingParams()], ignore_eos=True)
    tokens = list(prompt)
    for n, token in enumerate(runs[0].tokens, start=1):
        logits = plain.forward(cfg, weights, tokens)[-1].numpy()
        logits = plain.apply_repetition_penalty(logits, tokens[-20:], 1.4)
        want = plain.sample_token(logits, 0.9, plain.draw_key(77, n), top_p=0.95, top_k=12, min_p=0.01)
        if dtype == "float32":
            assert token == want, (n, token, want)
        elif token != want:
            score = logits / np.float32(0.9) + plain.gumbel_noise(plain.draw_key(77, n), len(logits))
            assert abs(float(score[token] - score[want])) < 0.05 * float(np.abs(logits).max()) / 0.9, (n, token, want)
        tokens.append(token)
    plain_tokens_match(cfg, weights, other, runs[1].tokens, margin=1e-3 if dtype == "float32" else 0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_through_few_slots_and_few_pages(tiny, dtype):
    """Continuous batching under pressure: more requests than state slots, a pool so small that
    pages are reused many times, and (without reservations) requests that are preempted and fed
    again.  Greedy tokens must not depend on any of it: in 32-bit they are the same tokens, in
    bfloat16 the plain implementation's up to near-ties."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    exact = dtype == "float32"
    lengths = [3, 47, 12, 80, 5, 33, 64, 9, 21, 70, 2, 55]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=300 + i) for i, n in enumerate(lengths)]
    roomy = Engine.from_folder(folder, dtype=dtype, page_size=settings["page_size"], context=4096,
                               max_batch_tokens=64, max_requests=16)
    want = [r.tokens for r in roomy.generate(prompts, max_tokens=10, ignore_eos=True)]
    for prompt, tokens in list(zip(prompts, want))[:3]:
        if exact:
            assert tokens == plain.generate(cfg, weights, prompt, 10)
        else:
            plain_tokens_match(cfg, weights, prompt, tokens, margin=0.05)

    def same(got, expected, their_prompts):
        if exact:
            assert [r.tokens for r in got] == expected
        else:
            for prompt, run in zip(their_prompts, got):
                assert len(run.tokens) == len(expected[0])
                plain_tokens_match(cfg, weights, prompt, run.tokens, margin=0.05)

    page = settings["page_size"]
    tight = Engine.from_folder(folder, dtype=dtype, page_size=page, num_pages=-(-200 // page),
                               max_batch_tokens=24, max_requests=3)
    got = tight.generate(prompts, max_tokens=10, ignore_eos=True)
    same(got, want, prompts)
    assert all(r.finish_reason == "length" for r in got)
    tight.executor.cache.check_invariants()
    assert tight.executor.cache.free_pages() == tight.executor.cache.num_pages

    # without reservations: four requests are admitted on what their prompts need, then grow by
    # 40 tokens each until the pool of 160 tokens runs out
    growing = [random_tokens(cfg["vocab_size"], n, seed=400 + n) for n in (20, 25, 30, 18)]
    want_long = [r.tokens for r in roomy.generate(growing, max_tokens=40, ignore_eos=True)]
    greedy_pool = Engine.from_folder(folder, dtype=dtype, page_size=page, num_pages=-(-160 // page),
                                     max_batch_tokens=32, max_requests=4, reserve=False)
    got = greedy_pool.generate(growing, max_tokens=40, ignore_eos=True)
    same(got, want_long, growing)
    assert greedy_pool.stats.preemptions > 0 and sum(r.preemptions for r in got) == greedy_pool.stats.preemptions, \
        "the pool was meant to run out"
    greedy_pool.executor.cache.check_invariants()
    assert greedy_pool.executor.cache.free_pages() == greedy_pool.executor.cache.num_pages

    too_long = tight.generate([random_tokens(cfg["vocab_size"], 400, seed=1)], max_tokens=4)[0]
    assert too_long.finish_reason == "too_long" and too_long.tokens == []


def test_preempted_requests_keep_their_draws(tiny):
    """Temperature sampling with a seed through a pool that runs out: a request that is preempted
    and fed again goes on with the draw it had reached, so its tokens are the plain
    implementation's draws (the draw counter is the number of output tokens, not of steps)."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    page = settings["page_size"]
    prompts = [random_tokens(cfg["vocab_size"], n, seed=500 + n) for n in (20, 25, 30, 18)]
    pool = Engine.from_folder(folder, dtype="float32", page_size=page, num_pages=-(-160 // page),
                              max_batch_tokens=32, max_requests=4, reserve=False)
    got = pool.generate(prompts, max_tokens=40, temperature=0.8, seed=4321, ignore_eos=True)
    assert pool.stats.preemptions > 0, "the pool was meant to run out"
    for i, (prompt, run) in enumerate(zip(prompts, got)):
        assert run.finish_reason == "length" and len(run.tokens) == 40
        plain_tokens_match(cfg, weights, prompt, run.tokens, temperature=0.8, seed=4321 + i)
    assert any(r.preemptions for r in got)
    pool.executor.cache.check_invariants()
    assert pool.executor.cache.free_pages() == pool.executor.cache.num_pages


def test_top_logprobs_beside_every_output_token(tiny):
    """``logprobs=n`` reports the n most likely tokens at every generated place: the same ids and
    values as the plain implementation, the chosen (greedy) token first, and the tokens unchanged."""
    from mrun_b200 import Engine
    name, folder, settings = tiny
    cfg, weights = plain.load_folder(folder)
    engine = Engine.from_folder(folder, dtype="float32", page_size=settings["page_size"], num_pages=64, max_requests=4)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=40 + n) for n in (5, 19)]
    plain_runs = engine.generate(prompts, max_tokens=6, ignore_eos=True)
    runs = engine.generate(prompts, max_tokens=6, ignore_eos=True, logprobs=3)
    for prompt, run, base in zip(prompts, runs, plain_runs):
        assert run.tokens == base.tokens and len(run.top_logprobs) == len(run.tokens) and not base.top_logprobs
        tokens = list(prompt)
        for token, top in zip(run.tokens, run.top_logprobs):
            want = plain.top_logprobs(plain.forward(cfg, weights, tokens)[-1].numpy(), 3)
            assert [i for i, _ in top] == [i for i, _ in want] and top[0][0] == token
            assert max(abs(a - b) for (_, a), (_, b) in zip(top, want)) <= 1e-4
            tokens.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_the_reach_of_a_captured_step(dtype, tmp_path):
    """Captured decode steps are made for contexts up to 4,096, up to 16,384 or up to the model's
    positions, and the host takes the smallest that covers the step.  A request whose context
    crosses 4,096 tokens in the middle of pipelined decoding changes graphs there; its token still
    comes from the step before, on the device, and the tokens stay the plain implementation's."""
    from mrun_b200 import Engine
    from mrun_b200.config import Qwen3Config
    from mrun_b200.weights import write_random_model
    from tiny_models import TINY
    t = TINY["C"]
    config = Qwen3Config(**dict(t["config"], max_position_embeddings=8192))
    folder = write_random_model(config, str(tmp_path / "model"), seed=t["seed"], std=t["std"], norm_noise=t["norm_noise"])
    cfg, weights = plain.load_folder(folder)
    prompts = [random_tokens(cfg["vocab_size"], n, seed=70 + n) for n in (4090, 37)]
    engine = Engine.from_folder(folder, dtype=dtype, page_size=16, context=2 * 4224, max_batch_tokens=1024, max_requests=2)
    runs = engine.generate(prompts, max_tokens=14, ignore_eos=True)
    graphs = engine.executor._graphs[2]
    assert sorted(graphs) == [4096, 8192], sorted(graphs)
    for prompt, run in zip(prompts, runs):
        assert len(run.tokens) == 14
        plain_tokens_match(cfg, weights, prompt, run.tokens, margin=1e-3 if dtype == "float32" else 0.05)
