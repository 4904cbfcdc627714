"""The scheduler's decisions, on the host with a scripted model in place of the GPU
(as the reference tests its runtime on a scripted engine, crates/mrun/src/runtime/scripted.rs,
crates/mrun/tests/admission.rs): refusals, admission with reservations, portions under the token
budget, finishing, and what happens when pages run out."""
from __future__ import annotations

import pytest

from mrun_b200.cache import CacheManager, OutOfPages, PagedKV
from mrun_b200.engine.scheduler import Request, Scheduler, chunk_len, looping
from mrun_b200.sampling import SamplingParams


def cache(pages=64, page_size=4, requests=4):
    return CacheManager([PagedKV(1, 8)], [None], page_size, pages, requests)


def drive(scheduler, next_token=lambda r: len(r.output) + 100, max_steps=10000, on_plan=None):
    """Runs plans against the cache manager the way the engine does; returns the plans."""
    plans = []
    for _ in range(max_steps):
        if not scheduler.has_work():
            break
        plan = scheduler.schedule()
        assert plan is not None
        try:
            append = scheduler.cache.plan_append([(e.request.cache, len(e.tokens)) for e in plan.entries])
        except OutOfPages:
            assert scheduler.preempt_newest() is not None
            continue
        scheduler.cache.commit(append)
        scheduler.cache.check_invariants()
        plans.append(plan)
        if on_plan:
            on_plan(plan)
        scheduler.launched(plan)
        scheduler.complete(plan, [next_token(r) for r in plan.sampled])
    assert not scheduler.has_work() and not scheduler.unsettled()
    return plans


def test_chunk_len_follows_the_reference_table():
    """crates/mrun-engine/src/engine.rs:481-486: clamp(2048 * 16384 / depth, 128, 2048)."""
    assert chunk_len(0) == 2048 and chunk_len(16384) == 2048 and chunk_len(32768) == 1024
    assert chunk_len(10 ** 7) == 128 and chunk_len(0, budget=64) == 64 and chunk_len(10 ** 7, budget=64) == 64


def test_loop_guard():
    assert not looping([1, 2, 3] * 100)
    assert looping([1, 2, 3] * 171)                      # 513 tokens repeating with period 3
    assert not looping(list(range(600)))
    assert looping(list(range(256)) * 2)                 # the longest period still caught
    assert not looping(list(range(257)) * 2)


def test_refusals():
    s = Scheduler(cache(pages=8, page_size=4), max_queue=1)
    cases = [
        (Request("empty", []), "invalid", "empty"),
        (Request("zero", [1], max_tokens=0), "invalid", "at least 1"),
        (Request("temp", [1], sampling=SamplingParams(temperature=-1.0)), "invalid", "temperature"),
        (Request("topp", [1], sampling=SamplingParams(top_p=0.0)), "invalid", "top_p"),
        (Request("long", list(range(32))), "too_long", "32 tokens"),
    ]
    for request, reason, text in cases:
        assert s.submit(request) == reason
        assert request.state == "finished" and request.finish_reason == reason and text in request.message
    assert s.submit(Request("fits", list(range(31)), max_tokens=100)) is None
    assert s.waiting[0].limit == 1                       # clamped to the room the prompt leaves
    assert s.submit(Request("second", [1])) == "queue_full"


def test_admission_reserves_prompt_plus_output():
    s = Scheduler(cache(pages=10, page_size=4, requests=4), max_batch_tokens=64)
    a = Request("a", list(range(10)), max_tokens=6)      # 16 tokens = 4 pages
    b = Request("b", list(range(9)), max_tokens=8)       # 17 tokens = 5 pages
    c = Request("c", list(range(3)), max_tokens=2)       # 5 tokens = 2 pages: does not fit beside a and b
    for r in (a, b, c):
        s.submit(r)
    plan = s.schedule()
    assert [e.request.request_id for e in plan.entries] == ["b", "a"]      # fewest prompt tokens left first
    assert c.state == "waiting" and a.state == b.state == "running"
    drive_rest = drive(s)
    assert c.finish_reason == "length" and len(c.output) == 2
    assert all(r.finish_reason == "length" for r in (a, b)) and s.preemptions == 0
    assert s.cache.free_pages() == 10 and s.cache.free_slots == 4


def test_portions_under_the_token_budget_beside_decodes():
    s = Scheduler(cache(pages=256, page_size=4, requests=4), max_batch_tokens=16)
    short = Request("short", list(range(5)), max_tokens=30)
    long = Request("long", list(range(50)), max_tokens=3)
    s.submit(short)
    s.submit(long)
    plans = drive(s)
    sizes = [[(e.request.request_id, len(e.tokens), e.wants_logits) for e in p.entries] for p in plans]
    assert sizes[0] == [("short", 5, True), ("long", 11, False)]           # shortest first, budget 16
    assert sizes[1] == [("short", 1, True), ("long", 15, False)]           # a decode beside a portion
    assert sizes[2] == [("short", 1, True), ("long", 15, False)]
    assert sizes[3] == [("short", 1, True), ("long", 9, True)]             # the last portion wants logits
    assert sizes[4] == [("short", 1, True), ("long", 1, True)]
    assert all(sum(n for _, n, _ in step) <= 16 for step in sizes)
    fed = {}
    for p in plans:
        for e in p.entries:
            fed.setdefault(e.request.request_id, []).extend(e.tokens)
    assert fed["long"] == long.prompt + long.output[:-1]                     # every token fed once, in order
    assert fed["short"] == short.prompt + short.output[:-1]


def test_finishing_reasons_and_eos():
    s = Scheduler(cache(), eos_token_ids=[7], max_batch_tokens=8)
    stop = Request("stop", [1, 2, 3], max_tokens=50)
    ignore = Request("ignore", [1, 2, 3], max_tokens=5, ignore_eos=True)
    s.submit(stop)
    s.submit(ignore)
    drive(s, next_token=lambda r: 7 if len(r.output) == 2 else 9)
    # the end token is not part of the output (crates/mrun/src/runtime/generate.rs:868-874)
    assert stop.finish_reason == "stop" and stop.output == [9, 9]
    assert ignore.finish_reason == "length" and ignore.output == [9, 9, 7, 9, 9]
    s = Scheduler(cache(pages=512), max_batch_tokens=8)
    loop = Request("loop", [1], max_tokens=2000)
    s.submit(loop)
    drive(s, next_token=lambda r: len(r.output) % 5)
    assert loop.finish_reason == "repetition" and len(loop.output) == 512
    # a run of a forced length goes to its limit however it repeats
    # (crates/mrun/src/runtime/generate.rs:908-913)
    s = Scheduler(cache(pages=512), max_batch_tokens=8)
    forced = Request("forced", [1], max_tokens=700, ignore_eos=True)
    s.submit(forced)
    drive(s, next_token=lambda r: len(r.output) % 5)
    assert forced.finish_reason == "length" and len(forced.output) == 700


def test_cancelling_from_the_token_callback_and_from_outside():
    """on_token returning False ends that request at once with what it has; the others go on
    (crates/mrun-engine/src/engine.rs:463-479, crates/mrun-engine/tests/tiny_qwen3.rs:193-211)."""
    s = Scheduler(cache(pages=64), max_batch_tokens=16)
    seen = []
    def stop_after_three(request, token):
        seen.append(token)
        return len(request.output) < 3
    a = Request("a", [1, 2, 3], max_tokens=20, on_token=stop_after_three)
    b = Request("b", [4, 5], max_tokens=6, on_token=lambda r, t: None)         # None is no cancellation
    c = Request("c", [6], max_tokens=20)
    for r in (a, b, c):
        s.submit(r)
    def tokens(r):
        if r is c and len(c.output) == 4:
            c.cancel_requested = True                     # asked from outside: it ends with its next token
        return 100 + len(r.output)
    drive(s, next_token=tokens)
    assert a.finish_reason == "cancelled" and a.output == [100, 101, 102] and seen == a.output
    assert b.finish_reason == "length" and b.output == [100 + i for i in range(6)]
    assert c.finish_reason == "cancelled" and c.output == [100 + i for i in range(5)]
    assert s.cache.free_pages() == 64 and s.cache.free_slots == 4
    s.cache.check_invariants()


def test_whose_turn_it_is_to_start():
    """crates/mrun/src/runtime/handle.rs:563-587: the oldest side request first, else the oldest
    request of another member than the one started last, else the oldest; a request cancelled
    while it waited never reaches the engine (:533-549)."""
    s = Scheduler(cache(requests=4), max_running=1)
    made = {}
    def request(name, **kw):
        made[name] = Request(name, [1, 2, 3], max_tokens=2, **kw)
        assert s.submit(made[name]) is None
    request("a1", turn="a"); request("a2", turn="a"); request("a3", turn="a")
    request("b1", turn="b"); request("side", auxiliary=True); request("gone", turn="c")
    made["gone"].cancel_requested = True
    drive(s)
    started = sorted((r for r in made.values() if r.order >= 0), key=lambda r: r.order)
    # the side request first; it names no member, so the oldest that names one is next (a1); then
    # another member than a (b1); then another than b (a2); then "gone" of member c, which is
    # dropped when its turn comes; a3 is left
    assert [r.request_id for r in started] == ["side", "a1", "b1", "a2", "a3"]
    assert made["gone"].finish_reason == "cancelled" and made["gone"].order == -1 and made["gone"].output == []
    assert made["gone"].cache is None and s.cancelled_waiting == [made["gone"]]
    assert all(r.finish_reason == "length" for r in started)
    # the native rule by itself
    from mrun_b200.cache import native
    lib, ia = native.library(), native.int_array
    assert lib.mrun_sched_next_turn(0, ia([]), ia([]), ia([]), 0, -1) == -1
    assert lib.mrun_sched_next_turn(3, ia([0, 0, 0]), ia([5, 5, 6]), ia([0, 0, 0]), 1, 5) == 2
    assert lib.mrun_sched_next_turn(3, ia([0, 0, 0]), ia([5, 5, 5]), ia([0, 0, 0]), 1, 5) == 0
    assert lib.mrun_sched_next_turn(3, ia([0, 0, 1]), ia([5, 6, 5]), ia([0, 0, 0]), 1, 5) == 2
    assert lib.mrun_sched_next_turn(3, ia([0, 0, 1]), ia([5, 6, 5]), ia([0, 1, 0]), 1, 5) == 1      # a preempted request before all


def test_stop_sequences_of_token_ids():
    """The reference's stop strings on token ids (crates/mrun/src/chat/stop.rs:24-85 and its tests
    at :95-130): a sequence split over steps is found and left out; a false start is shown later;
    the longest of several that end at one token wins; held tokens are shown when the request
    ends for another reason; more than four or an empty one are refused."""
    def run(stream, stop, max_tokens=20, eos=()):
        s = Scheduler(cache(), eos_token_ids=eos)
        seen = []
        r = Request("r", [1, 2, 3], max_tokens=max_tokens, stop=stop, on_token=lambda request, t: seen.append(t))
        assert s.submit(r) is None
        drive(s, next_token=lambda request: stream[len(request.output) + (len(request.stop_sequence or []))])
        return r, seen

    stream = [10, 11, 7, 8, 9, 12, 13, 14] + [0] * 40
    r, seen = run(stream, [[7, 8, 9]])
    assert r.finish_reason == "stop" and r.stop_sequence == [7, 8, 9] and r.output == [10, 11] and seen == [10, 11]
    assert len(r.token_times) == 2
    # a false start is released once it cannot be a stop sequence any more
    r, seen = run([7, 8, 5, 7, 8, 9] + [0] * 40, [[7, 8, 9]])
    assert r.output == [7, 8, 5] and seen == [7, 8, 5] and r.finish_reason == "stop"
    # the longest of the sequences that end at the same token began earliest
    r, _ = run(stream, [[9], [8, 9], [30, 31]])
    assert r.stop_sequence == [8, 9] and r.output == [10, 11, 7]
    # ... and a sequence that ends earlier wins over a longer one that would end later
    r, _ = run(stream, [[7, 8, 9, 12], [8]])
    assert r.stop_sequence == [8] and r.output == [10, 11, 7]
    # what was held back is shown when the limit ends the request
    order = []
    s = Scheduler(cache())
    r = Request("r", [1, 2, 3], max_tokens=4, stop=[[7, 8, 9]], on_token=lambda request, t: order.append((len(request.output), t)))
    assert s.submit(r) is None
    drive(s, next_token=lambda request: [10, 11, 7, 8][len(request.output)])
    assert r.finish_reason == "length" and r.output == [10, 11, 7, 8] and r.stop_sequence is None
    assert order == [(1, 10), (2, 11), (4, 7), (4, 8)]            # 7 and 8 only once the request had ended
    # an end token ends it as before, and shows what was held
    r, seen = run([10, 7, 99], [[7, 8]], eos=(99,))
    assert r.finish_reason == "stop" and r.stop_sequence is None and r.output == [10, 7] and seen == [10, 7]
    # refusals
    for bad, message in (([[1]] * 5, "at most 4 stop sequences"), ([[]], "1..=64 tokens"), ([list(range(65))], "1..=64 tokens")):
        s = Scheduler(cache())
        r = Request("r", [1, 2, 3], stop=bad)
        assert s.submit(r) == "invalid" and message in r.message


def test_out_of_pages_preempts_the_newest_and_recomputes():
    """Without reservations the pool runs out in mid-run: the request admitted last gives
    everything back, waits at the head of the queue, and later feeds prompt + output again."""
    s = Scheduler(cache(pages=12, page_size=4, requests=3), max_batch_tokens=32, reserve=False)
    a = Request("a", list(range(12)), max_tokens=20)
    b = Request("b", list(range(12)), max_tokens=20)
    s.submit(a)
    s.submit(b)
    refed = []
    def watch(plan):
        for e in plan.entries:
            if e.request is b and b.preemptions and e.request.fed == 0:
                refed.append(list(e.tokens))
    drive(s, on_plan=watch)
    assert a.preemptions == 0 and b.preemptions >= 1 and s.preemptions == b.preemptions
    assert a.finish_reason == b.finish_reason == "length" and len(a.output) == len(b.output) == 20
    assert refed and refed[0][:12] == b.prompt and refed[0][12:] == b.output[:len(refed[0]) - 12]
    assert s.cache.free_pages() == 12 and s.cache.free_slots == 3


def test_a_lone_request_is_never_preempted():
    s = Scheduler(cache(pages=4, page_size=4, requests=2), reserve=False)
    only = Request("only", list(range(10)), max_tokens=100)
    s.submit(only)
    drive(s)
    assert only.finish_reason == "length" and len(only.output) == 6 and only.preemptions == 0
    assert s.preempt_newest() is None


def test_abort_frees_everything():
    s = Scheduler(cache())
    r = Request("r", list(range(9)), max_tokens=5)
    s.submit(r)
    plan = s.schedule()
    s.cache.commit(s.cache.plan_append([(r.cache, 9)]))
    s.abort(r, "cancelled")
    assert r.finish_reason == "aborted" and s.cache.free_pages() == 64 and not s.has_work()


def test_seeds():
    s = Scheduler(cache())
    seeded = Request("s", [1], sampling=SamplingParams(temperature=1.0, seed=42))
    free1, free2 = Request("f1", [1], sampling=SamplingParams(temperature=1.0)), Request("f2", [1])
    for r in (seeded, free1, free2):
        s.submit(r)
    assert seeded.seed == 42 and free1.seed != free2.seed


def test_steps_in_flight():
    """A step may be planned while the tokens of the step before are unread: the request counts
    its unread token, leaves out requests whose unread token is their last, and a request that
    turns out to have ended keeps its pages until the step in flight has been read."""
    s = Scheduler(cache(pages=64, page_size=4, requests=4), eos_token_ids=[7], max_batch_tokens=32)
    a, b = Request("a", [1, 2, 3], max_tokens=3), Request("b", [4, 5], max_tokens=10)
    s.submit(a)
    s.submit(b)
    def launch():
        plan = s.schedule()
        s.cache.commit(s.cache.plan_append([(e.request.cache, len(e.tokens)) for e in plan.entries]))
        s.launched(plan)
        return plan
    def read(plan, tokens):                            # tokens by request id, in the plan's row order
        return s.complete(plan, [tokens[e.request.request_id] for e in plan.entries if e.wants_logits])
    first = launch()                                   # both prompts, logits wanted
    assert a.inflight == b.inflight == 1 and a.fed == 3 and b.fed == 2
    second = launch()                                  # planned before the first step is read
    assert sorted((e.request.request_id, e.from_device) for e in second.entries) == [("a", True), ("b", True)]
    assert a.inflight == 2 and a.remaining == 1          # the second unread token is still to be fed
    read(first, {"a": 9, "b": 7})                    # b sampled an end token: it is in the second step already
    assert b.finish_reason == "stop" and b.retiring and b.cache is not None and b.output == []
    third = launch()                                   # a's third token will be its last: one more row, b is gone
    assert [e.request.request_id for e in third.entries] == ["a"]
    assert not s.has_work() and s.unsettled()          # nothing more to plan, tokens still on the way
    read(second, {"a": 9, "b": 1})                   # b's token is dropped and b gives its pages back
    assert b.output == [] and b.cache is None and not b.retiring
    read(third, {"a": 9})
    assert a.finish_reason == "length" and a.output == [9, 9, 9] and not s.unsettled()
    assert s.cache.free_pages() == 64 and s.cache.free_slots == 4
    s.cache.check_invariants()


def test_native_plan_follows_the_rule_under_random_states():
    """The step the host library plans (csrc/host/sched_core.cpp) against the rule restated here:
    one token for every request past its prompt (while the budget lasts), then portions, fewest
    tokens left first, ties by admission order, each at most chunk_len(depth) and the budget."""
    import random
    from mrun_b200.cache import native
    core = native.library()
    rng = random.Random(5)
    for _ in range(300):
        n = rng.randint(1, 12)
        budget_all = rng.choice([1, 3, 16, 64, 2048])
        prompt = [rng.randint(1, 5000) for _ in range(n)]
        out = [rng.choice([0, 0, 1, 7]) for _ in range(n)]
        limit = [o + rng.choice([0, 1, 5]) for o in out]
        inflight = [rng.choice([0, 0, 1]) if o > 0 or rng.random() < 0.2 else 0 for o in out]
        retiring = [1 if rng.random() < 0.1 else 0 for _ in range(n)]
        order = rng.sample(range(100), n)
        seq = [p + o for p, o in zip(prompt, out)]
        fed = []
        for i in range(n):
            if inflight[i]:
                fed.append(seq[i])                        # everything read so far is in the cache
            elif out[i] > 0:
                fed.append(seq[i] - 1)                    # the last token read is still to be fed
            else:
                fed.append(rng.choice([0, rng.randint(0, prompt[i] - 1)]))
        # the rule
        want, budget = [], budget_all
        active = [i for i in range(n) if not retiring[i] and out[i] + inflight[i] < limit[i]]
        decoding = [i for i in active if seq[i] + inflight[i] - fed[i] == 1 and fed[i] > 0]
        for i in decoding[:budget]:
            want.append((i, 1, 1, 1 if inflight[i] else 0))
        budget -= len(want)
        readers = sorted((i for i in active if i not in decoding and not inflight[i]),
                         key=lambda i: (seq[i] - fed[i], order[i]))
        for i in readers:
            if budget < 1:
                break
            take = min(seq[i] - fed[i], budget, chunk_len(fed[i], budget_all))
            want.append((i, take, 1 if take == seq[i] - fed[i] else 0, 0))
            budget -= take
        which, tokens = native.int_array([0] * n), native.int_array([0] * n)
        wants, from_device = native.int_array([0] * n), native.int_array([0] * n)
        made = core.mrun_sched_plan(n, native.long_array(seq), native.long_array(fed), native.int_array(inflight),
                                    native.long_array(out), native.long_array(limit), native.int_array(retiring),
                                    native.long_array(order), budget_all, which, tokens, wants, from_device)
        got = [(which[e], tokens[e], wants[e], from_device[e]) for e in range(made)]
        assert got == want
        assert sum(t for _, t, _, _ in got) <= budget_all


def test_native_end_reason_and_victim():
    from mrun_b200.cache import native
    core = native.library()
    assert core.mrun_sched_end_reason(1, 0, 3, 10, None, 0) == 1 and core.mrun_sched_end_reason(1, 1, 3, 10, None, 0) == 0
    assert core.mrun_sched_end_reason(0, 0, 10, 10, None, 0) == 2 and core.mrun_sched_end_reason(1, 1, 10, 10, None, 0) == 2
    loop = native.int_array([4, 9] * 256)
    assert core.mrun_sched_end_reason(0, 0, 512, 9999, loop, 512) == 3
    assert core.mrun_sched_end_reason(0, 0, 513, 9999, loop, 512) == 0          # not a multiple of the interval
    assert core.mrun_sched_end_reason(0, 1, 512, 9999, loop, 512) == 0          # the guard is off with ignore_eos
    assert core.mrun_sched_preemption_victim(3, native.int_array([0, 0, 0]), native.long_array([5, 9, 2])) == 1
    assert core.mrun_sched_preemption_victim(3, native.int_array([0, 1, 0]), native.long_array([5, 9, 2])) == 0
    assert core.mrun_sched_preemption_victim(2, native.int_array([0, 1]), native.long_array([5, 9])) == -1
