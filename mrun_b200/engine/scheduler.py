"""The scheduler: admits requests, cuts prompts into portions under a token budget, lets every
running request decode, finishes requests and frees what they hold.  Host-side only; it decides,
the executor computes.  The decisions themselves (refusal and clamped limit at submission, the
admission test, what a step holds, the length of a portion, why a request ends, who gives way when
pages run out) are computed by the host runtime library (``csrc/host/sched_core.cpp``, C++); this
class keeps the request objects and the queues and hands their numbers over.

Decisions, with the reference's where it has one
------------------------------------------------
* **Refusals** at submission: empty prompt, ``max_tokens`` 0, invalid sampling → ``invalid``; a
  prompt that leaves no room for one output token in the cache → ``too_long``; the output limit is
  clamped to what remains (crates/mrun/src/runtime/generate.rs:522-532, 600-636).  A full waiting
  queue refuses with ``queue_full`` (crates/mrun/src/runtime/queue.rs:80-91).
* **Admission** is first come, first served: a request starts when a state slot is free and, with
  ``reserve`` on, when the pages for its prompt plus its clamped output limit fit beside what the
  running requests have reserved (crates/mrun/src/runtime/handle.rs:497-559).  With reservations
  a running request never runs out of pages.
* **A step** holds one token of every running request that has finished its prompt, plus prompt
  portions while the token budget lasts, the request with the fewest prompt tokens left first,
  ties by admission order (crates/mrun/src/runtime/lanes.rs:187-196).  A portion is at most
  ``chunk_len(depth)`` = clamp(budget · 16384 / depth, 128, budget) tokens
  (crates/mrun-engine/src/engine.rs:481-486).  The portion that ends a prompt asks for the logits
  of its last token.  Unlike the reference, portions and decoded tokens share one batch.
* **When pages run out** (only with ``reserve`` off): the running request admitted last gives
  everything back and returns to the head of the queue; when it is admitted again it feeds its
  prompt and what it had generated as one prompt.  Requests admitted earlier are never touched,
  and a request that runs alone always fits because of the refusal above.
* **Steps in flight**: a decode step may be launched before the tokens of the step before it have
  been read back (they are taken from the device).  The scheduler then plans with
  ``Request.inflight`` unread tokens; a request whose unread token will reach its output limit
  is left out, and a request that turns out to have ended (an end token) while a later step was
  already launched is marked ``retiring``: that step's token for it is dropped and its pages are
  freed when the step is read.
* **Finishing**: an end token (unless ``ignore_eos``) → ``stop``, the end token itself being left
  out of the output; the output limit → ``length``; the last 512 output tokens repeating with a
  period of at most 256, checked every 16 tokens and never with ``ignore_eos`` → ``repetition``
  (crates/mrun/src/runtime/generate.rs:27-33, 420-426, 866-919).
* **Whose turn** (crates/mrun/src/runtime/handle.rs:497-587): among the waiting requests the
  oldest side request (``Request.auxiliary``) starts first, else the oldest request of another
  member (``Request.turn``) than the one started last, else the oldest; a request that was
  preempted goes before all of them.  If the one whose turn it is does not fit, nobody starts.
  A request cancelled while it waits (``cancel_requested``) ends with ``cancelled`` when its turn
  comes and never reaches the engine.
* **Stop sequences** (``Request.stop``: up to 4 lists of token ids, the reference's ``--stop`` on
  token ids instead of text, crates/mrun/src/chat/stop.rs:24-85, crates/mrun/src/chat/limits.rs:6):
  the request ends with ``stop`` as soon as its output ends with one of them, the longest if
  several do; the sequence is cut from the output and named in ``Request.stop_sequence``.  Tokens
  that may still begin a stop sequence are held back from ``on_token`` until they cannot, or until
  the request ends for another reason.
* **Constrained decoding** (``Request.allowed_tokens``): before each of the request's tokens is
  sampled the callable gives the tokens allowed next as a ``sampling.TokenMask`` (or None); such
  a request is read back step by step.  A mask that allows nothing, or one over more tokens than
  the model has logits, ends the request with ``invalid`` and the reference's message
  (crates/mrun-engine/src/engine.rs:571-576).
* **Cancelling**: ``on_token`` returning False, or ``Request.cancel_requested`` set by the caller,
  ends the request with ``cancelled`` when its next token is read: the tokens read so far stay,
  a token still in flight for it is dropped, its pages go back, and the other requests of the
  step go on unchanged (the reference's cancel flag, crates/mrun-engine/src/engine.rs:463-479).
"""
from __future__ import annotations

import ctypes
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache import native
from ..cache.manager import CacheManager, RequestCache
from ..sampling.params import GREEDY, SamplingParams, fresh_seed

LOOP_WINDOW, LOOP_MAX_PERIOD = 512, 256
END_REASONS = (None, "stop", "length", "repetition")
MAX_STOPS, MAX_STOP_TOKENS = 4, 64


def checked_stops(stop) -> List[List[int]]:
    """Stop sequences as lists of token ids: at most 4, each of 1 to 64 ids (the reference's
    messages, crates/mrun/src/chat/stop.rs:7-10, with tokens for bytes)."""
    stops = [list(map(int, sequence)) for sequence in (stop or [])]
    if len(stops) > MAX_STOPS:
        raise ValueError(f"at most {MAX_STOPS} stop sequences are allowed, got {len(stops)}")
    for sequence in stops:
        if not 1 <= len(sequence) <= MAX_STOP_TOKENS:
            raise ValueError(f"stop sequences must be 1..={MAX_STOP_TOKENS} tokens, got {len(sequence)}")
    return stops


def chunk_len(depth: int, budget: int = 2048) -> int:
    """Longest prompt portion at ``depth`` tokens already in the cache."""
    return int(native.library().mrun_sched_chunk_len(int(depth), int(budget)))


def looping(output: Sequence[int]) -> bool:
    """Whether the last 512 tokens repeat with a period of at most 256."""
    if len(output) < LOOP_WINDOW:
        return False
    window = native.int_array(output[-LOOP_WINDOW:])
    return bool(native.library().mrun_sched_looping(window, LOOP_WINDOW))


@dataclass
class Request:
    request_id: object
    prompt: List[int]
    max_tokens: int = 2048
    sampling: SamplingParams = GREEDY
    ignore_eos: bool = False
    logprobs: int = 0                  # how many of the most likely tokens to report beside each output token
    on_token: Optional[object] = None  # called with (request, token) as each output token is read back
    stop: List[List[int]] = field(default_factory=list)      # stop sequences of token ids (see checked_stops)
    # constrained decoding: called with the request before each of its tokens is sampled, returns
    # a sampling.TokenMask (the tokens allowed next) or None (no constraint for this token)
    allowed_tokens: Optional[object] = None
    auxiliary: bool = False            # a side request: admitted before the normal ones (handle.rs:563-587)
    turn: Optional[str] = None         # who waits for it: waiting requests are served in turns between members
    # ---- run state
    state: str = "new"                 # new | waiting | running | finished
    output: List[int] = field(default_factory=list)
    fed: int = 0                       # tokens of prompt + output that are in the cache
    limit: int = 0                     # clamped output limit
    seed: int = 0
    cache: Optional[RequestCache] = None
    finish_reason: Optional[str] = None
    message: str = ""
    order: int = -1                    # admission order
    reserved_pages: int = 0
    preemptions: int = 0
    submitted_at: float = 0.0
    first_token_at: float = 0.0
    finished_at: float = 0.0
    token_times: List[float] = field(default_factory=list)   # when each output token was read back
    top_logprobs: List[list] = field(default_factory=list)   # per output token: [(id, log-probability), ...]
    stop_sequence: Optional[List[int]] = None    # the stop sequence that ended the request, if one did
    streamed: int = 0                  # output tokens that on_token has seen
    cancel_requested: bool = False     # set from outside (or by on_token returning False): end at the next token read
    inflight: int = 0                  # tokens sampled on the device that the host has not read yet
    retiring: bool = False             # finished, but a step in flight still holds a row of it

    @property
    def sequence_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens still to feed, counting a sampled token that has not been read back yet."""
        return self.sequence_len + self.inflight - self.fed

    def next_tokens(self, n: int) -> List[int]:
        start = self.fed
        p = len(self.prompt)
        if start + n <= p:
            return self.prompt[start:start + n]
        if start >= p:
            return self.output[start - p:start - p + n]
        return self.prompt[start:] + self.output[:start + n - p]

    def recent(self, n: int) -> List[int]:
        if len(self.output) >= n:
            return self.output[-n:]
        return (self.prompt + self.output)[-n:]


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    wants_logits: bool
    from_device: bool = False          # its one token is still on the device (sampled by the step before)


@dataclass
class StepPlan:
    entries: List[PlannedEntry]

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)

    @property
    def sampled(self) -> List[Request]:
        return [e.request for e in self.entries if e.wants_logits]


class Scheduler:
    def __init__(self, cache: CacheManager, eos_token_ids: Sequence[int] = (), max_batch_tokens: int = 2048,
                 max_running: Optional[int] = None, max_queue: Optional[int] = None, reserve: bool = True,
                 max_positions: Optional[int] = None):
        if max_batch_tokens < 1:
            raise ValueError(f"max_batch_tokens must be at least 1, got {max_batch_tokens}")
        self.cache = cache
        self.eos = frozenset(eos_token_ids)
        self.max_batch_tokens = max_batch_tokens
        self.max_running = min(max_running or cache.max_requests, cache.max_requests)
        self.max_queue = max_queue
        self.reserve = reserve
        self.capacity_tokens = cache.num_pages * cache.page_size
        if max_positions is not None:
            self.capacity_tokens = min(self.capacity_tokens, max_positions)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._admitted = 0
        self._reserved = 0
        self.preemptions = 0
        self._turn_ids: Dict[str, int] = {}          # members' names as numbers for the native rule
        self._last_turn: Optional[tuple] = None      # (turn of the request started last,), None before the first
        self.cancelled_waiting: List[Request] = []   # requests that were cancelled before they were admitted
        self._core = native.library()
        self._loop_check_every = int(self._core.mrun_sched_loop_check_every())

    # ------------------------------------------------------------------ submission
    def submit(self, request: Request) -> Optional[str]:
        """Queues the request, or finishes it at once with a refusal (returned)."""
        request.submitted_at = time.perf_counter()
        reason = None
        if len(request.prompt) == 0:
            reason, request.message = "invalid", "the prompt is empty"
        elif request.max_tokens < 1:
            reason, request.message = "invalid", "max tokens must be at least 1"
        else:
            try:
                request.sampling.validate()
                request.stop = checked_stops(request.stop)
            except (ValueError, TypeError) as error:
                reason, request.message = "invalid", str(error)
        if reason is None:
            limit = ctypes.c_int64(0)
            code = self._core.mrun_sched_submit_check(len(request.prompt), int(request.max_tokens), self.capacity_tokens,
                                                      len(self.waiting), -1 if self.max_queue is None else self.max_queue,
                                                      ctypes.byref(limit))
            request.limit = int(limit.value)
            if code == 1:
                reason = "too_long"
                request.message = (f"prompt is too long: {len(request.prompt)} tokens, the cache holds "
                                   f"{self.capacity_tokens}")
            elif code == 2:
                reason, request.message = "queue_full", f"{len(self.waiting)} requests are waiting already"
        if reason is not None:
            self._finish(request, reason)
            return reason
        request.seed = request.sampling.seed if request.sampling.seed is not None else fresh_seed()
        request.state = "waiting"
        self.waiting.append(request)
        return None

    def has_work(self) -> bool:
        """Whether a further step can be planned now (requests that only wait for tokens in flight
        do not count)."""
        if self.waiting:
            return True
        return any(not r.retiring and len(r.output) + r.inflight < r.limit for r in self.running)

    def unsettled(self) -> bool:
        """Whether any request is still admitted (running, or waiting for tokens in flight)."""
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ admission
    def _need_pages(self, request: Request) -> int:
        return self.cache.blocks_for(len(request.prompt) + request.limit)

    def _can_admit(self, request: Request) -> bool:
        # with reservations: pages for prompt + clamped output beside what is reserved; on demand:
        # room for its whole sequence and one more page, beside what the running requests still
        # have to bring in
        running = self.running
        return bool(self._core.mrun_sched_can_admit(
            len(running), self.max_running, self.cache.free_slots, 1 if self.reserve else 0, self._reserved,
            self.cache.num_pages, self.cache.page_size, self.cache.free_pages(), len(request.prompt) + request.limit,
            request.sequence_len, len(running), native.long_array(r.sequence_len for r in running),
            native.long_array(r.fed for r in running)))

    def _next_turn(self) -> int:
        """Index of the waiting request to start next (side requests first, then the oldest of
        another member than the one served last, else the oldest; a preempted request before all)."""
        waiting = list(self.waiting)
        names = self._turn_ids
        turns = [(-1 if r.turn is None else names.setdefault(r.turn, len(names))) for r in waiting]
        last = self._last_turn
        return self._core.mrun_sched_next_turn(
            len(waiting), native.int_array(1 if r.auxiliary else 0 for r in waiting), native.int_array(turns),
            native.int_array(1 if r.order >= 0 else 0 for r in waiting), 0 if last is None else 1,
            -1 if last is None or last[0] is None else names.setdefault(last[0], len(names)))

    def _admit(self) -> None:
        while self.waiting:
            at = self._next_turn()
            request = self.waiting[at]
            if not request.cancel_requested and not self._can_admit(request):
                return
            del self.waiting[at]
            self._last_turn = (request.turn,)
            if request.cancel_requested:
                # cancelled while waiting: it never reaches the engine (handle.rs:533-549)
                self._finish(request, "cancelled")
                self.cancelled_waiting.append(request)
                continue
            request.cache = self.cache.admit(request.request_id)
            request.state = "running"
            request.fed = 0
            if request.order < 0:
                request.order = self._admitted
                self._admitted += 1
            if self.reserve:
                request.reserved_pages = self._need_pages(request)
                self._reserved += request.reserved_pages
            self.running.append(request)

    # ------------------------------------------------------------------ one step
    def schedule(self) -> Optional[StepPlan]:
        self._admit()
        if not self.running:
            return None
        running = self.running
        n = len(running)
        which, tokens = native.int_array([0] * n), native.int_array([0] * n)
        wants, from_device = native.int_array([0] * n), native.int_array([0] * n)
        made = self._core.mrun_sched_plan(
            n, native.long_array(r.sequence_len for r in running), native.long_array(r.fed for r in running),
            native.int_array(r.inflight for r in running), native.long_array(len(r.output) for r in running),
            native.long_array(r.limit for r in running), native.int_array(1 if r.retiring else 0 for r in running),
            native.long_array(r.order for r in running), self.max_batch_tokens, which, tokens, wants, from_device)
        entries: List[PlannedEntry] = []
        for e in range(made):
            request = running[which[e]]
            if from_device[e]:
                entries.append(PlannedEntry(request, [0], True, from_device=True))
            else:
                entries.append(PlannedEntry(request, request.next_tokens(tokens[e]), bool(wants[e])))
        return StepPlan(entries) if entries else None

    def launched(self, plan: StepPlan) -> None:
        """Records that the plan's step was handed to the device: its tokens count as fed, and
        every entry that wanted logits has one sampled token on the way."""
        for entry in plan.entries:
            entry.request.fed += len(entry.tokens)
            if entry.wants_logits:
                entry.request.inflight += 1

    def complete(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Records the tokens of a launched step: ``sampled`` holds one per entry that wanted
        logits, in order.  Returns the requests that finished.  The token of a request that
        finished meanwhile (a later step was launched before its end token was read) is dropped."""
        now = time.perf_counter()
        done: List[Request] = []
        sampled = list(sampled)
        if len(sampled) != len(plan.sampled):
            raise ValueError(f"{len(plan.sampled)} tokens were wanted, {len(sampled)} came")
        at = 0
        for entry in plan.entries:
            request = entry.request
            if not entry.wants_logits:
                continue
            token = sampled[at]
            at += 1
            request.inflight -= 1
            if request.retiring:
                if request.inflight == 0:
                    self._retire(request)
                continue
            if token is None:                        # no token could be sampled (request.message says why)
                self._stream(request, len(request.output))
                self._retire(request)
                self._finish(request, "invalid")
                done.append(request)
                continue
            token = int(token)
            # The end token itself is not part of the output: it is neither counted, streamed nor
            # returned (crates/mrun/src/runtime/generate.rs:868-874 returns Stop before pushing).
            count = len(request.output) + 1
            recent, recent_len = None, 0             # the loop guard looks every few tokens only
            if count % self._loop_check_every == 0 and count >= LOOP_WINDOW and not request.ignore_eos:
                recent = native.int_array(request.output[-(LOOP_WINDOW - 1):] + [token])
                recent_len = LOOP_WINDOW
            reason = END_REASONS[self._core.mrun_sched_end_reason(
                1 if token in self.eos else 0, 1 if request.ignore_eos else 0, count, request.limit, recent, recent_len)]
            if request.first_token_at == 0.0:
                request.first_token_at = now
            cancelled = False
            if reason != "stop":
                request.output.append(token)
                request.token_times.append(now)
                held = 0
                if request.stop:
                    matched, held = self._stop_state(request)
                    if matched is not None:              # the output ends before the stop sequence
                        del request.output[-len(matched):]
                        del request.token_times[len(request.output):]
                        request.stop_sequence, reason = matched, "stop"
                if reason is None:
                    cancelled = self._stream(request, len(request.output) - held)
            if reason == "stop":
                del request.top_logprobs[len(request.output):]       # the rows of what is left out go with it
            if reason is None and (cancelled or request.cancel_requested):
                reason = "cancelled"
            if reason is not None and not cancelled:
                self._stream(request, len(request.output))           # what was held back is shown at the end
            if reason is not None:
                if request.inflight:
                    request.retiring = True          # its row in the step in flight is dropped later
                else:
                    self._retire(request)
                self._finish(request, reason)
                done.append(request)
        return done

    def _stop_state(self, request: Request):
        """(the stop sequence the output ends with or None, how many of its last tokens may still
        begin one)."""
        longest = max(len(sequence) for sequence in request.stop)
        tail = request.output[-longest:]
        flat = native.int_array([t for sequence in request.stop for t in sequence])
        lens = native.int_array([len(sequence) for sequence in request.stop])
        tail_array = native.int_array(tail)
        hit = self._core.mrun_sched_stop_match(tail_array, len(tail), flat, lens, len(request.stop))
        if hit >= 0:
            return request.stop[hit], 0
        return None, self._core.mrun_sched_stop_held(tail_array, len(tail), flat, lens, len(request.stop))

    @staticmethod
    def _stream(request: Request, upto: int) -> bool:
        """Shows ``on_token`` the output tokens it has not seen, up to ``upto``; True when it asked
        to cancel."""
        cancelled = False
        while request.streamed < upto:
            token = request.output[request.streamed]
            request.streamed += 1
            if request.on_token is not None and request.on_token(request, token) is False:
                cancelled = True
        return cancelled

    # ------------------------------------------------------------------ out of pages
    def preempt_newest(self) -> Optional[Request]:
        """Gives back everything the running request admitted last holds and puts it at the head
        of the queue.  None when at most one request runs (it is never preempted)."""
        running = self.running
        at = self._core.mrun_sched_preemption_victim(len(running), native.int_array(1 if r.retiring else 0 for r in running),
                                                     native.long_array(r.order for r in running))
        if at < 0:
            return None
        if any(r.inflight for r in running):
            raise RuntimeError("a request cannot be preempted while a step is in flight")
        victim = running[at]
        self._retire(victim)
        victim.state = "waiting"
        victim.fed = 0
        victim.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(victim)
        return victim

    def abort(self, request: Request, message: str = "") -> None:
        if request.state == "running":
            self._retire(request)
        elif request.state == "waiting":
            self.waiting.remove(request)
        request.message = message
        self._finish(request, "aborted")

    # ------------------------------------------------------------------ internals
    def _retire(self, request: Request) -> None:
        self.running.remove(request)
        request.retiring = False
        if request.cache is not None:
            self.cache.release(request.cache)
            request.cache = None
        self._reserved -= request.reserved_pages
        request.reserved_pages = 0

    def _finish(self, request: Request, reason: str) -> None:
        request.state = "finished"
        request.finish_reason = reason
        request.finished_at = time.perf_counter()
        self.finished.append(request)
