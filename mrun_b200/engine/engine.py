"""The Python entry point: ``Engine(...).generate(prompts, ...)``, token ids in, token ids out.

The reference has no Python API; its token-ids-in program is
``generate <model-dir> <ids> [max-tokens]`` (crates/mrun-engine/examples/generate.rs:1-13) and
its sampling options are those of ``mrun run`` (crates/mrun/src/cli/run.rs:27-79).  This class
follows both: the same option names and meanings, the same finish reasons.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.manager import token_bytes
from ..cache.pages import OutOfPages
from ..sampling.mask import TokenMask
from ..sampling.params import REPETITION_CONTEXT, SamplingParams, draw_key
from ..sampling.sampler import Sampler
from . import budget
from .batch import RECENT, StepEntry
from .budget import MemoryBudget
from .executor import Executor
from .loading import executor_from_config, executor_from_folder
from .scheduler import Request, Scheduler, StepPlan, checked_stops


@dataclass
class Generation:
    tokens: List[int]
    finish_reason: str
    message: str = ""
    prompt_tokens: int = 0
    time_to_first_token_s: float = 0.0
    total_s: float = 0.0
    preemptions: int = 0
    first_token_time: float = 0.0                 # host clock (perf_counter) readings
    finished_time: float = 0.0
    token_times: List[float] = field(default_factory=list)
    # with ``logprobs=n``: per output token the n most likely tokens at that place as
    # (id, log-probability), most likely first (crates/mrun-engine/src/engine.rs:740-741)
    top_logprobs: List[list] = field(default_factory=list)
    stop_sequence: Optional[List[int]] = None     # the stop sequence that ended it (finish reason ``stop``), else None


@dataclass
class _Flying:
    """A captured decode step whose tokens the host has not read yet."""
    plan: StepPlan
    rows: dict                     # id(request) -> row of the step
    bucket: int
    pinned: torch.Tensor           # where its tokens land on the host
    event: torch.cuda.Event


@dataclass
class EngineStats:
    steps: int = 0
    tokens_in: int = 0
    tokens_out: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    h2d_mask_bytes: int = 0        # token masks of constrained requests copied to the device
    preemptions: int = 0


class Engine:
    def __init__(self, executor: Executor, max_batch_tokens: int = 2048, reserve: bool = True,
                 max_queue: Optional[int] = None):
        self.executor = executor
        self.max_batch_tokens = max_batch_tokens
        self.reserve = reserve
        self.max_queue = max_queue
        self.sampler = Sampler(executor.device)
        self.eos_token_ids = tuple(executor.spec.eos_token_ids)
        self.stats = EngineStats()
        self._next_id = 0
        rows = max(1, 2 * executor.cache.max_requests)
        self._token_buffers = [torch.empty(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._token_turn = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, model_dir: str, dtype: str = "bfloat16", page_size: int = 16,
                    num_pages: Optional[int] = None, context: Optional[int] = None,
                    max_requests: int = 64, max_batch_tokens: int = 2048, reserve: bool = True,
                    device: str = "cuda:0", memory: Optional[MemoryBudget] = None, **kw) -> "Engine":
        """``num_pages`` or ``context`` size the cache directly.  With ``memory`` (a budget from
        :func:`mrun_b200.engine.budget.plan`) the cache is what the budget leaves beside the
        weights and the step's scratch, or exactly ``context`` tokens if that fits."""
        sizing = None
        if memory is not None and num_pages is None:
            sizing = _sizing(memory, context, page_size, max_requests, max_batch_tokens)
        pages = _pages_for(num_pages, context, page_size)
        executor = executor_from_folder(model_dir, dtype=dtype, page_size=page_size, num_pages=pages,
                                        max_requests=max_requests, device=device, sizing=sizing)
        return cls(executor, max_batch_tokens=max_batch_tokens, reserve=reserve, **kw)

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype: str = "bfloat16", std: float = 0.02,
                    norm_noise: float = 0.0, page_size: int = 16, num_pages: Optional[int] = None,
                    context: Optional[int] = None, max_requests: int = 64, max_batch_tokens: int = 2048,
                    reserve: bool = True, device: str = "cuda:0", memory: Optional[MemoryBudget] = None,
                    **kw) -> "Engine":
        sizing = None
        if memory is not None and num_pages is None:
            sizing = _sizing(memory, context, page_size, max_requests, max_batch_tokens)
        pages = _pages_for(num_pages, context, page_size)
        executor = executor_from_config(config, seed, dtype=dtype, std=std, norm_noise=norm_noise,
                                        page_size=page_size, num_pages=pages, max_requests=max_requests,
                                        device=device, sizing=sizing)
        return cls(executor, max_batch_tokens=max_batch_tokens, reserve=reserve, **kw)

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 2048, temperature: float = 0.0,
                 top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0, seed: Optional[int] = None,
                 repetition_penalty: float = 1.0, ignore_eos: bool = False,
                 sampling: Optional[Sequence[SamplingParams]] = None, logprobs: int = 0,
                 on_token=None, stop: Optional[Sequence[Sequence[int]]] = None,
                 allowed_tokens=None) -> List[Generation]:
        """Generates for every prompt (lists of token ids) and returns the results in order.
        ``sampling`` gives each prompt settings of its own; otherwise all share the keyword
        values, prompt i drawing with ``seed + i`` when a seed is given.  ``logprobs`` = n > 0
        also reports, for every output token, the n most likely tokens at its place with their
        log-probabilities (of the logits as the model gave them, before any penalty); such
        requests are read back step by step, not pipelined.  ``on_token(i, token)`` is called as
        each output token of prompt i reaches the host (with pipelined decoding one step after it
        was sampled), the way the reference streams a generation to its client; when it returns
        False, prompt i is cancelled: it ends with finish reason ``cancelled`` and the tokens read
        so far, and the other prompts go on unchanged (the reference's cancel flag,
        crates/mrun-engine/src/engine.rs:463-479).  An end token finishes a prompt with ``stop``
        and is itself not part of the output (crates/mrun/src/runtime/generate.rs:868-874).
        ``stop``: up to 4 stop sequences of token ids (the reference's ``--stop`` on ids instead of
        text): a prompt ends with ``stop`` where its output would end with one of them, the
        sequence left out and named in ``Generation.stop_sequence``; tokens that may begin one are
        held back from ``on_token`` until they cannot (crates/mrun/src/chat/stop.rs:24-85).
        ``allowed_tokens(i, output)``: constrained decoding; called before each token of prompt i
        is sampled with the tokens generated so far, it returns the tokens allowed next as a
        ``TokenMask`` or an iterable of ids, or None for no constraint (the reference's token mask,
        crates/mrun-engine/src/sample.rs:88-116); such prompts are read back step by step."""
        if not 0 <= logprobs <= 1024:
            raise ValueError(f"logprobs must be 0 .. 1024, got {logprobs}")
        stops = checked_stops(stop)
        requests = []
        for i, prompt in enumerate(prompts):
            if sampling is not None:
                params = sampling[i]
            else:
                params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                                        seed=None if seed is None else seed + i,
                                        repetition_penalty=repetition_penalty)
            requests.append(Request(request_id=("gen", self._next_id), prompt=list(map(int, prompt)),
                                    max_tokens=max_tokens, sampling=params, ignore_eos=ignore_eos,
                                    logprobs=logprobs, stop=[list(sequence) for sequence in stops],
                                    allowed_tokens=None if allowed_tokens is None
                                    else (lambda r, i=i: allowed_tokens(i, list(r.output))),
                                    on_token=None if on_token is None else (lambda r, t, i=i: on_token(i, t))))
            self._next_id += 1
        self.run(requests)
        return [Generation(tokens=r.output, finish_reason=r.finish_reason, message=r.message,
                           prompt_tokens=len(r.prompt),
                           time_to_first_token_s=max(0.0, r.first_token_at - r.submitted_at) if r.output else 0.0,
                           total_s=r.finished_at - r.submitted_at, preemptions=r.preemptions,
                           first_token_time=r.first_token_at, finished_time=r.finished_at,
                           token_times=r.token_times, top_logprobs=r.top_logprobs, stop_sequence=r.stop_sequence)
                for r in requests]

    def run(self, requests: Sequence[Request]) -> None:
        """Runs the requests to their end through the scheduler and the step function.

        Pure decode steps are pipelined: step n+1 is launched with the tokens of step n taken on
        the device, and only then are step n's tokens read back, so the host's work for a step
        overlaps the device's work for the step before (the reference pipelines its decode the
        same way, crates/mrun-engine/src/nuvec_engine.rs:1489-1517)."""
        scheduler = Scheduler(self.executor.cache, eos_token_ids=self.eos_token_ids,
                              max_batch_tokens=self.max_batch_tokens, reserve=self.reserve,
                              max_queue=self.max_queue, max_positions=self.executor.spec.max_positions)
        for request in requests:
            scheduler.submit(request)
        flying: Optional[_Flying] = None
        try:
            while scheduler.has_work() or flying is not None:
                plan = scheduler.schedule() if scheduler.has_work() else None
                if plan is not None and self._pipelinable(plan, flying):
                    launched = self._launch_captured(scheduler, plan, flying)
                    if launched is not None:
                        if flying is not None:
                            self._deliver(scheduler, flying)
                        flying = launched
                        continue
                if flying is not None:          # read what is in flight, then plan with everything known
                    self._deliver(scheduler, flying)
                    flying = None
                    continue
                if plan is None:
                    raise RuntimeError("the scheduler has waiting requests and nothing to run")
                self._run_plan(scheduler, plan)
            if scheduler.unsettled():
                raise RuntimeError("requests are left without a step to run")
        finally:
            if flying is not None:
                flying.event.synchronize()
            for request in list(scheduler.running):
                request.inflight = 0
                scheduler.abort(request, "generation was interrupted")
        self.stats.preemptions += scheduler.preemptions
        from ..kernels import ops
        ops.tc5_check(self.executor.device)

    # ------------------------------------------------------------------ pipelined decode steps
    def _pipelinable(self, plan: StepPlan, flying: Optional["_Flying"]) -> bool:
        """A plan of single decode tokens that a captured step takes, whose unread tokens all sit
        in the step in flight, and that needs no token history for a repetition penalty."""
        if not all(len(e.tokens) == 1 and e.wants_logits for e in plan.entries):
            return False
        if any(e.request.logprobs or e.request.allowed_tokens is not None for e in plan.entries):
            return False                    # the logits themselves are wanted on the host side, or a mask comes from it
        bucket = self.executor.decode_bucket(len(plan.entries))
        if bucket is None:
            return False
        if any(e.request.sampling.repetition_penalty != 1.0 for e in plan.entries):
            return flying is None and not any(e.from_device for e in plan.entries)
        for entry in plan.entries:
            if entry.from_device and (flying is None or flying.bucket != bucket
                                      or id(entry.request) not in flying.rows):
                return False
        return True

    def _launch_captured(self, scheduler: Scheduler, plan: StepPlan,
                         flying: Optional["_Flying"]) -> Optional["_Flying"]:
        sampled = plan.sampled
        entries = [StepEntry(e.request.cache, e.tokens, [0]) for e in plan.entries]
        sources = [flying.rows[id(e.request)] if e.from_device else -1 for e in plan.entries]
        try:
            tokens = self.executor.decode_step(
                entries, lambda host, where: _fill_sampling(host, where, sampled), sources)
        except OutOfPages:
            return None                     # settle what is in flight, then the slow path decides
        pinned = self._token_buffers[self._token_turn]
        self._token_turn ^= 1
        pinned[:len(entries)].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        scheduler.launched(plan)
        self.stats.steps += 1
        self.stats.tokens_in += plan.num_tokens
        return _Flying(plan, {id(e.request): row for row, e in enumerate(plan.entries)},
                       self.executor.decode_bucket(len(entries)), pinned, event)

    def _deliver(self, scheduler: Scheduler, flying: "_Flying") -> None:
        flying.event.synchronize()
        host = flying.pinned[:len(flying.plan.entries)].tolist()
        self.stats.tokens_out += len(host)
        self.stats.d2h_bytes += 4 * len(host)
        scheduler.complete(flying.plan, host)

    def _run_plan(self, scheduler: Scheduler, plan: StepPlan) -> None:
        """A step with prompt portions in it (or one no captured step takes): run and read at once."""
        entries = [StepEntry(e.request.cache, e.tokens, [len(e.tokens) - 1] if e.wants_logits else [])
                   for e in plan.entries]
        sampled = plan.sampled
        try:
            logits = self.executor.step(entries)
        except OutOfPages:
            if scheduler.preempt_newest() is None:
                raise
            return                          # plan again without the preempted request
        scheduler.launched(plan)
        self.stats.steps += 1
        self.stats.tokens_in += plan.num_tokens
        if not sampled:
            scheduler.complete(plan, [])
            return
        wanted = [(row, r) for row, r in enumerate(sampled) if r.logprobs]
        if wanted:                          # before the sampler, which applies penalties in place
            ids, values = self.sampler.top_logprobs(logits, max(r.logprobs for _, r in wanted))
            ids, values = ids.to("cpu").tolist(), values.to("cpu").tolist()
            for row, r in wanted:
                r.top_logprobs.append(list(zip(ids[row][:r.logprobs], values[row][:r.logprobs])))
        refused = self._apply_token_masks(logits, sampled)
        tokens = self.sampler.sample(
            logits, [r.sampling for r in sampled], [r.seed for r in sampled],
            [len(r.output) + 1 for r in sampled],
            [r.recent(REPETITION_CONTEXT) for r in sampled])
        host = tokens.to("cpu").tolist()
        for row in refused:
            host[row] = None
        if plan.num_tokens > len(plan.entries):          # a step with prompt portions: its kernels wait on one another
            self.executor.check()
        self.stats.tokens_out += len(host)
        self.stats.d2h_bytes += 4 * len(host)
        scheduler.complete(plan, host)

    def _apply_token_masks(self, logits: torch.Tensor, sampled: Sequence[Request]) -> List[int]:
        """Asks the requests that decode under a constraint for their masks and sets the logits
        of the tokens they do not allow to -inf.  Returns the rows whose mask cannot be used
        (their requests' messages say why: crates/mrun-engine/src/engine.rs:571-576)."""
        from ..kernels import ops
        vocab = logits.shape[1]
        words_a_mask = -(-vocab // 32)
        rows, words, widths, refused = [], [], [], []
        for row, request in enumerate(sampled):
            if request.allowed_tokens is None:
                continue
            mask = request.allowed_tokens(request)
            if mask is None:
                continue
            if not isinstance(mask, TokenMask):
                mask = TokenMask.of(mask, vocab)
            if mask.vocab > vocab:
                request.message = f"a token mask over {mask.vocab} tokens is wider than the model's {vocab} logits"
                refused.append(row)
            elif mask.is_none():
                request.message = "the token mask allows no token"
                refused.append(row)
            else:
                padded = np.zeros(words_a_mask, dtype=np.uint32)
                padded[:len(mask.words)] = mask.words
                rows.append(row); words.append(padded); widths.append(mask.vocab)
        if rows:
            device = logits.device
            ops.apply_token_mask(logits, torch.tensor(rows, dtype=torch.int32).to(device),
                                 torch.from_numpy(np.stack(words).view(np.int32)).to(device),
                                 torch.tensor(widths, dtype=torch.int32).to(device))
            self.stats.h2d_mask_bytes += 4 * words_a_mask * len(rows)
        return refused

    # ------------------------------------------------------------------ direct stepping
    def step(self, entries: Sequence[StepEntry]):
        """The step function itself, for callers that schedule on their own."""
        return self.executor.step(entries)

    def info(self) -> dict:
        ex = self.executor
        return {
            "architecture": ex.spec.architecture,
            "dtype": ex.precision.name,
            "weights_bytes": ex.model.weight_bytes(),
            "page_size": ex.cache.page_size,
            "num_pages": ex.cache.num_pages,
            "cache_bytes": ex.cache.bytes_per_page() * ex.cache.num_pages,
            "capacity_tokens": ex.cache.num_pages * ex.cache.page_size,
            "max_requests": ex.cache.max_requests,
            "max_batch_tokens": self.max_batch_tokens,
            "eos_token_ids": list(self.eos_token_ids),
            "memory": ex.memory.breakdown() if ex.memory is not None else None,
        }


def _fill_sampling(host, where, requests: Sequence[Request]) -> None:
    """Writes the rows' sampling settings into a captured step's input buffer."""
    n = len(requests)
    as_bits = lambda values: np.asarray(values, dtype=np.float32).view(np.int32)
    temperature = host[where["temperature"]]; top_p = host[where["top_p"]]
    min_p = host[where["min_p"]]; penalty = host[where["penalty"]]
    top_p[:] = as_bits([1.0])[0]
    penalty[:] = as_bits([1.0])[0]
    temperature[:n] = as_bits([r.sampling.temperature for r in requests])
    top_p[:n] = as_bits([r.sampling.top_p for r in requests])
    min_p[:n] = as_bits([r.sampling.min_p for r in requests])
    penalty[:n] = as_bits([r.sampling.repetition_penalty for r in requests])
    host[where["top_k"]][:n] = [r.sampling.top_k for r in requests]
    recent = host[where["recent"]].reshape(-1, RECENT)
    recent[:] = -1
    keys = np.zeros(len(temperature), dtype=np.uint64)
    for i, r in enumerate(requests):
        if not r.sampling.greedy:
            keys[i] = draw_key(r.seed, len(r.output) + r.inflight + 1)
        if r.sampling.repetition_penalty != 1.0:
            ids = r.recent(RECENT)
            recent[i, :len(ids)] = ids
    host[where["keys"]] = keys.view(np.int32)


def _sizing(memory: MemoryBudget, context: Optional[int], page_size: int, max_requests: int,
            max_batch_tokens: int):
    """The executor's page count from a memory budget, once the model is on the device."""
    def sizing(model):
        spec, precision = model.spec, model.runtime.precision
        element = 2 if precision.act == torch.bfloat16 else 4
        per_token, per_slot = token_bytes(model.cache_needs(), model.cache_shares(), element)
        scratch = budget.scratch_estimate(spec.hidden_size, model.activation_elements(), spec.vocab_size,
                                          max_batch_tokens, max_requests, element)
        weights = model.weight_bytes()
        most = spec.max_positions * max_requests
        if context is not None:
            done = budget.for_context(memory, context, weights, scratch, max(1, per_token), most,
                                      per_slot * max_requests)
        else:
            done = budget.with_capacity(memory, weights, scratch, max(1, per_token), most,
                                        per_slot * max_requests)
        return max(1, -(-done.capacity_tokens // page_size)), done
    return sizing


def _pages_for(num_pages: Optional[int], context: Optional[int], page_size: int) -> int:
    if num_pages is not None:
        return num_pages
    if context is not None:
        return -(-context // page_size)
    return -(-32768 // page_size)
