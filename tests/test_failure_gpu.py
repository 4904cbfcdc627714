"""Failures made on the host in the middle of a step: a part whose ``forward`` raises at a chosen
layer on a chosen call, a sampler that raises after the model ran, a settings callback that raises
inside the captured decode step.  After each, every request is as it was before the step (length,
block row, free pages, state slots), and the same step run again gives bit-identical 32-bit
logits to an executor that was never disturbed
(crates/mrun-engine/tests/failure.rs:20-96, crates/mrun-engine/src/nuvec_engine.rs:78-92).
Nothing faults on the device: the exception is a Python ``raise`` between two kernel launches."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, ClassVar

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_models import TINY, random_tokens, tiny_config

pytestmark = pytest.mark.gpu


class Injected(RuntimeError):
    pass


class Trigger:
    """Raises on the n-th forward of the feed-forward of one layer, once."""

    def __init__(self):
        self.layer, self.countdown, self.fired = None, 0, 0

    def arm(self, layer: int, nth: int = 1) -> None:
        self.layer, self.countdown = layer, nth

    def visit(self, layer: int) -> None:
        if self.layer == layer and self.countdown > 0:
            self.countdown -= 1
            if self.countdown == 0:
                self.layer = None
                self.fired += 1
                raise Injected(f"injected at the feed-forward of layer {layer}")


TRIGGER = Trigger()


@dataclass(frozen=True)
class FailingMLPSpec:
    kind: ClassVar[str] = "failing_mlp"
    inner: Any
    layer: int


def register_failing():
    from mrun_b200.parts import FEED_FORWARDS, register_feed_forward
    if "failing_mlp" in FEED_FORWARDS.kinds():
        return
    GatedMLP = FEED_FORWARDS.get("gated_mlp")

    @register_feed_forward("failing_mlp")
    class FailingMLP(GatedMLP):
        @staticmethod
        def tensor_specs(spec, prefix):
            return GatedMLP.tensor_specs(spec.inner, prefix)

        def __init__(self, spec, tensors, runtime):
            super().__init__(spec.inner, tensors, runtime)
            self.layer = spec.layer

        def forward(self, x, ctx, defer_output=False):
            TRIGGER.visit(self.layer)
            return super().forward(x, ctx, defer_output=defer_output)


def executors(name: str, dtype: str, pages: int, requests: int = 4):
    """(executor with the failing feed-forward in every layer, undisturbed executor), same weights."""
    from mrun_b200.engine.executor import Executor
    from mrun_b200.weights import random_tensors
    register_failing()
    t = TINY[name]
    spec = tiny_config(name).to_spec()
    tensors = dict(random_tensors(spec, t["seed"], t["std"], t["norm_noise"], torch.float32))
    failing = replace(spec, layers=tuple(replace(layer, feed_forward=FailingMLPSpec(layer.feed_forward, i))
                                         for i, layer in enumerate(spec.layers)))
    make = lambda s: Executor(s, tensors, dtype=dtype, page_size=t["page_size"], num_pages=pages, max_requests=requests)
    return make(failing), make(spec)


def books(executor):
    """Everything the cache manager knows, as plain values."""
    cache = executor.cache
    cache.check_invariants()
    return {
        "free_pages": {key: cache.free_pages(key) for key in cache.groups},
        "free_slots": cache.free_slots,
        "requests": {r.request_id: (r.slot, r.length, r.pending,
                                    {key: list(r.pages_held(key)) for key in cache.groups})
                     for r in cache.live},
    }


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("layer", [0, 1])
def test_a_part_that_raises_in_mid_step_changes_nothing(name, layer):
    from mrun_b200.engine import StepEntry
    hurt, calm = executors(name, "float32", pages=96)
    vocab = tiny_config(name).vocab_size
    prompts = {rid: random_tokens(vocab, n, seed=700 + n) for rid, n in (("a", 37), ("b", 21), ("c", 9))}

    def run(executor, inject):
        """A prompt portion, then a mixed step, then a single-token step; with ``inject`` each of
        them fails once first (a different call of the layer's feed-forward each time)."""
        out = []
        live = {rid: executor.admit(rid) for rid in prompts}
        steps = [
            [("a", prompts["a"][:30], [29])],
            [("a", prompts["a"][30:31], [0]), ("b", prompts["b"][:17], [3, 16]), ("c", prompts["c"], [8])],
            [("a", prompts["a"][31:32], [0]), ("b", prompts["b"][17:18], [0])],
        ]
        for number, step in enumerate(steps):
            entries = [StepEntry(live[rid], tokens, want) for rid, tokens, want in step]
            if inject:
                before = books(executor)
                TRIGGER.arm(layer)
                with pytest.raises(Injected):
                    executor.step(entries)
                assert books(executor) == before, f"step {number} left something behind"
            out.append(executor.step(entries).clone())
        assert [live[rid].length for rid in ("a", "b", "c")] == [32, 18, 9]
        for request in live.values():
            executor.release(request)
        executor.cache.check_invariants()
        assert executor.cache.free_pages() == executor.cache.num_pages
        return out

    fired = TRIGGER.fired
    got, want = run(hurt, True), run(calm, False)
    assert TRIGGER.fired == fired + 3
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # and both are the plain implementation's logits
    cfg, weights = plain_model(name)
    logits = plain.forward(cfg, weights, prompts["a"][:32])
    scale = float(logits.abs().max())
    assert float((want[0][0].cpu() - logits[29]).abs().max()) <= 2e-5 * scale
    assert float((want[2][0].cpu() - logits[31]).abs().max()) <= 2e-5 * scale


def plain_model(name):
    from mrun_b200.weights import random_tensors
    t = TINY[name]
    config = tiny_config(name)
    weights = {k: v.float() for k, v in random_tensors(config.to_spec(), t["seed"], t["std"], t["norm_noise"], torch.float32)}
    return config.to_dict(), weights


def test_a_failure_inside_the_captured_decode_step_rolls_back():
    """``decode_step`` takes the pages for its tokens, lays the step out and replays its graph; a
    failure after the pages were taken (here: the callback that writes the sampling settings)
    gives them back, and the step run again gives the undisturbed tokens and logits."""
    from mrun_b200.engine import StepEntry
    hurt, calm = executors("C", "float32", pages=64)
    vocab = tiny_config("C").vocab_size
    prompts = [random_tokens(vocab, n, seed=800 + n) for n in (16, 31, 5)]     # 16: the next token opens a page

    def run(executor, inject):
        live = [executor.admit(i) for i in range(len(prompts))]
        executor.step([StepEntry(r, p[:-1], []) for r, p in zip(live, prompts)])
        last = [p[-1] for p in prompts]
        tokens, logits = [], []
        for step in range(6):
            entries = [StepEntry(r, [t], [0]) for r, t in zip(live, last)]
            if inject and step in (0, 3):
                before = books(executor)
                def broken(host, where):
                    raise Injected("injected while the step was laid out")
                with pytest.raises(Injected):
                    executor.decode_step(entries, sampling=broken)
                assert books(executor) == before
            last = executor.decode_step(entries).tolist()
            tokens.append(last)
            logits.append(executor.decode_logits(entries).clone())
        for r in live:
            executor.release(r)
        executor.cache.check_invariants()
        return tokens, logits

    got, want = run(hurt, True), run(calm, False)
    assert got[0] == want[0]
    for a, b in zip(got[1], want[1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("where", ["model", "sampler"])
def test_generation_that_fails_frees_everything_and_the_next_one_is_unchanged(where, monkeypatch):
    """Through the entry point: a step that raises (in a part, or in the sampler after the model
    ran and the step was committed) ends the call with that exception; every request's pages and
    slot are given back, and the same call afterwards returns the undisturbed tokens."""
    from mrun_b200.engine.engine import Engine
    hurt, calm = executors("A", "float32", pages=96)
    vocab = tiny_config("A").vocab_size
    prompts = [random_tokens(vocab, n, seed=900 + n) for n in (12, 40, 3)]
    want = [g.tokens for g in Engine(calm, max_batch_tokens=16).generate(prompts, max_tokens=9, ignore_eos=True)]
    engine = Engine(hurt, max_batch_tokens=16)
    if where == "model":
        TRIGGER.arm(1, nth=3)                                # the third step of the prompts
    else:
        original, calls = engine.sampler.sample, []
        def failing_sample(*args, **kwargs):
            calls.append(1)
            if len(calls) == 2:
                raise Injected("injected in the sampler")
            return original(*args, **kwargs)
        monkeypatch.setattr(engine.sampler, "sample", failing_sample)
    with pytest.raises(Injected):
        engine.generate(prompts, max_tokens=9, ignore_eos=True)
    hurt.cache.check_invariants()
    assert not hurt.cache.live and hurt.cache.free_pages() == hurt.cache.num_pages
    assert hurt.cache.free_slots == hurt.cache.max_requests
    got = [g.tokens for g in engine.generate(prompts, max_tokens=9, ignore_eos=True)]
    assert got == want


def test_the_other_requests_of_a_failed_step_finish_with_unchanged_tokens():
    """Scheduler and step function driven by hand, as the engine's loop does: a mixed step fails,
    nothing was recorded as launched, the scheduler plans the same step again, and every request
    ends with the tokens of an undisturbed run."""
    from mrun_b200.engine import StepEntry
    from mrun_b200.engine.scheduler import Request, Scheduler
    hurt, calm = executors("B", "float32", pages=128)
    vocab = tiny_config("B").vocab_size
    prompts = [random_tokens(vocab, n, seed=950 + n) for n in (33, 4, 18)]

    def run(executor, fail_at):
        scheduler = Scheduler(executor.cache, max_batch_tokens=12, max_positions=executor.spec.max_positions)
        requests = [Request(i, list(p), max_tokens=7, ignore_eos=True) for i, p in enumerate(prompts)]
        for r in requests:
            scheduler.submit(r)
        step, failures = 0, 0
        while scheduler.has_work():
            plan = scheduler.schedule()
            entries = [StepEntry(e.request.cache, e.tokens, [len(e.tokens) - 1] if e.wants_logits else [])
                       for e in plan.entries]
            if step in fail_at:
                fail_at = fail_at - {step}
                before = books(executor)
                TRIGGER.arm(2)
                with pytest.raises(Injected):
                    executor.step(entries)
                assert books(executor) == before
                failures += 1
                continue                                   # plan again: the same step comes back
            logits = executor.step(entries)
            scheduler.launched(plan)
            tokens = logits.argmax(-1).tolist() if logits is not None else []
            scheduler.complete(plan, tokens)
            step += 1
        executor.cache.check_invariants()
        assert executor.cache.free_pages() == executor.cache.num_pages
        return [r.output for r in requests], failures

    got, failures = run(hurt, {1, 4, 6})
    want, _ = run(calm, set())
    assert failures == 3 and got == want
    cfg, weights = plain_model("B")
    assert want[1] == plain.generate(cfg, weights, prompts[1], 7)
