"""The step function: runs exactly the tokens it is given, as one batch, from the cache that
earlier steps left, and returns the logits at the wanted places.

A step is plan → do → commit: the pages for the new tokens are taken first (all or nothing), the
model runs, then the requests' lengths advance.  If anything fails before the commit, the pages
go back and every request is as it was (the reference's rule, crates/mrun-engine/src/ledger.rs:5-9).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..config.spec import ModelSpec
from ..parts import Precision, Runtime
from .batch import HostStaging, StepContext, StepEntry, build_context
from .model import Model


class StepError(ValueError):
    """A step that cannot run as given (bad token id, bad place, too long)."""


class LaunchCounter:
    """Counts this library's kernel launches (calls through the C ABI) between begin and end."""

    def __init__(self):
        self.total = 0
        self._mark = 0

    def begin(self) -> None:
        from ..kernels import lib
        self._mark = lib.call_count()

    def end(self) -> int:
        from ..kernels import lib
        n = lib.call_count() - self._mark
        self.total += n
        return n


class Executor:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], dtype: str = "bfloat16",
                 page_size: int = 16, num_pages: int = 256, max_requests: int = 8,
                 device: str = "cuda:0", sizing=None):
        """``sizing(model) -> (num_pages, memory)`` replaces ``num_pages`` once the weights are
        on the device: the memory budget needs their size and the parts' needs to say how many
        pages fit; ``memory`` is kept for :meth:`Engine.info`."""
        if not torch.cuda.is_available():
            raise RuntimeError("mrun_b200 runs on a CUDA device only: no GPU is visible and there "
                               "is no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.precision = Precision.of(dtype)
        self.runtime = Runtime(self.device, self.precision, page_size)
        self.spec = spec
        self.model = Model(spec, tensors, self.runtime)
        self.memory = None
        if sizing is not None:
            num_pages, self.memory = sizing(self.model)
        self.cache = CacheManager(self.model.cache_needs(), self.model.cache_shares(), page_size,
                                  num_pages, max_requests, device=self.device, dtype=self.precision.act,
                                  max_blocks_per_request=-(-spec.max_positions // page_size))
        self.staging = HostStaging(self.device)
        self.steps_run = 0
        self.launches = LaunchCounter()
        self.use_graphs = self.model.graph_safe
        # captured decode steps: rows (a power of two) -> reach -> graph.  The reach is an upper
        # bound of the contexts a graph was captured for (parts see it as ``ctx.max_kv_len`` and
        # may choose kernels by it); the host takes the smallest reach that covers the step.
        self._graphs: Dict[int, Dict[int, "DecodeGraph"]] = {}
        self._graph_tokens: Dict[int, torch.Tensor] = {}
        self._last_graph: Dict[int, "DecodeGraph"] = {}

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: object) -> RequestCache:
        return self.cache.admit(request_id)

    def release(self, request: RequestCache) -> None:
        self.cache.release(request)

    def trim(self, request: RequestCache, length: int) -> None:
        """Cuts a request back to its first ``length`` tokens; its next step goes on from there
        (the reference's ``trim``, crates/mrun-engine/src/engine.rs:746)."""
        self.cache.trim(request, length)

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        vocab, limit = self.spec.vocab_size, self.spec.max_positions
        for entry in entries:
            n = len(entry.tokens)
            if n < 1:
                raise StepError(f"request {entry.request.request_id!r}: a step brings at least one token")
            tokens = np.asarray(entry.tokens)
            if tokens.dtype.kind not in "iu":
                raise StepError(f"request {entry.request.request_id!r}: token ids must be integers")
            if tokens.min() < 0 or tokens.max() >= vocab:
                raise StepError(f"request {entry.request.request_id!r}: token id outside [0, {vocab})")
            if entry.request.length + n > limit:
                raise StepError(f"request {entry.request.request_id!r}: {entry.request.length + n} tokens "
                                f"exceed max_position_embeddings={limit}")
            for w in entry.want:
                if not 0 <= w < n:
                    raise StepError(f"request {entry.request.request_id!r}: wanted place {w} is outside "
                                    f"its {n} tokens")

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Returns float32 ``[wanted, vocab]`` in the order of the entries and of their ``want``
        lists, or None when nothing is wanted.  Raises :class:`OutOfPages` with nothing changed
        when the pages do not suffice."""
        self._validate(entries)
        plan = self.cache.plan_append([(e.request, len(e.tokens)) for e in entries])
        try:
            ctx = build_context(entries, self.cache, self.staging)
            rows: List[int] = []
            for seg, entry in zip(ctx.segments, entries):
                rows.extend(seg.q_start + w for w in entry.want)
            row_index = None
            if rows:
                row_index = torch.tensor(rows, dtype=torch.int32).to(self.device, non_blocking=True)
            logits = self.model.forward(ctx, self.cache.entries, row_index)
        except BaseException:
            self.cache.rollback(plan)
            raise
        self.cache.commit(plan)
        self.steps_run += 1
        return logits

    def check(self) -> None:
        """Raises if a kernel with bounded waits gave up on one since the last check (reads a
        word from the device, so it waits for the work queued so far)."""
        from ..kernels import ops
        ops.tc5_check(self.device)

    # ------------------------------------------------------------------ captured decode step
    def decode_bucket(self, rows: int) -> Optional[int]:
        """The captured step size that takes ``rows`` decoding requests, or None."""
        if not self.use_graphs or rows < 1:
            return None
        bucket = 1
        while bucket < rows:
            bucket *= 2
        return bucket if bucket <= max(1, self.cache.max_requests) * 2 else None

    REACHES = (4096, 16384)

    def decode_reach(self, longest: int) -> int:
        """The context bound of the captured step that takes a step whose longest request will
        hold ``longest`` tokens: 4,096, 16,384 or the model's positions."""
        for reach in self.REACHES:
            if longest <= reach < self.spec.max_positions:
                return reach
        return self.spec.max_positions

    def decode_step(self, entries: Sequence[StepEntry], sampling=None,
                    sources: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One token for each entry (each brings exactly one token) through a captured graph,
        sampling included.  ``sampling(host, where)`` writes the rows' sampling settings into the
        step's buffer (left at greedy when None).  ``sources[i] >= 0`` says that entry i's token
        is row ``sources[i]`` of the previous captured step of the same size, still on the device
        (the entry's own token value is then ignored).  Returns int32 device tokens, one per
        entry; they stay valid until the next captured step of this size runs."""
        vocab, limit = self.spec.vocab_size, self.spec.max_positions
        for e in entries:
            if len(e.tokens) != 1:
                raise StepError("decode_step takes one token per request")
            if not 0 <= e.tokens[0] < vocab:
                raise StepError(f"request {e.request.request_id!r}: token id outside [0, {vocab})")
            if e.request.length + 1 > limit:
                raise StepError(f"request {e.request.request_id!r}: {e.request.length + 1} tokens exceed "
                                f"max_position_embeddings={limit}")
        bucket = self.decode_bucket(len(entries))
        if bucket is None:
            raise StepError(f"no captured decode step takes {len(entries)} requests")
        reach = self.decode_reach(max(e.request.length for e in entries) + 1)
        graph = self._graphs.get(bucket, {}).get(reach)
        if graph is None:
            tokens = self._graph_tokens.get(bucket)
            if tokens is None:       # one output a size: a step may take its tokens from a step of another reach
                tokens = self._graph_tokens[bucket] = torch.zeros(bucket, dtype=torch.int32, device=self.device)
            graph = DecodeGraph(self, bucket, reach, tokens)
            self._graphs.setdefault(bucket, {})[reach] = graph
        self._last_graph[bucket] = graph
        plan = self.cache.plan_append([(e.request, 1) for e in entries])
        try:
            base = sampling if sampling is not None else _greedy_rows

            def fill(host, where):
                base(host, where)
                if sources is not None:
                    host[where["token_src"]][:len(sources)] = sources
            build_context(entries, self.cache, self.staging, pad_tokens=bucket, out=graph.buffer,
                          sampling=fill)
            graph.replay()
            self.launches.total += graph.kernels_per_replay
        except BaseException:
            self.cache.rollback(plan)
            raise
        self.cache.commit(plan)
        self.steps_run += 1
        return graph.tokens[:len(entries)]

    def decode_logits(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The logits of the last :meth:`decode_step` for its entries."""
        bucket = self.decode_bucket(len(entries))
        return self._last_graph[bucket].logits[:len(entries)]


def _greedy_rows(host, where) -> None:
    host[where["top_p"]] = np.float32(1.0).view(np.int32)
    host[where["penalty"]] = np.float32(1.0).view(np.int32)
    host[where["recent"]] = -1


class DecodeGraph:
    """A captured decode step of a fixed number of rows: every request brings one token, the
    model runs, one token per row is chosen.  Its inputs live in one static int32 buffer that each
    replay refills; rows beyond the live requests are padding (position -1, no cache slot)."""

    def __init__(self, executor: "Executor", rows: int, reach: int, tokens: torch.Tensor):
        from ..kernels import ops
        from .batch import RECENT, GroupView, StepContext, layout
        self.rows, self.reach = rows, reach
        cache, model, device = executor.cache, executor.model, executor.device
        keys = list(cache.groups)
        self.where = where = layout(rows, rows, len(keys), rows)
        self.buffer = torch.zeros(where["_size"].stop, dtype=torch.int32, device=device)
        buf = self.buffer
        buf[where["positions"]] = -1
        for g in range(len(keys)):
            buf[where[f"slot_mapping{g}"]] = -1
        buf[where["recent"]] = -1
        buf[where["token_src"]] = -1
        f32 = lambda name: buf[where[name]].view(torch.float32)
        buf[where["top_p"]] = torch.ones(rows, dtype=torch.float32, device=device).view(torch.int32)
        buf[where["penalty"]] = torch.ones(rows, dtype=torch.float32, device=device).view(torch.int32)
        self.row_index = torch.arange(rows, dtype=torch.int32, device=device)
        groups = {key: GroupView(cache.groups[key].table_device, buf[where[f"slot_mapping{g}"]],
                                 cache.groups[key].max_blocks) for g, key in enumerate(keys)}
        self.ctx = StepContext(
            num_tokens=rows, num_segments=rows, segments=[], token_ids=buf[where["token_ids"]],
            positions=buf[where["positions"]], token_slot=buf[where["token_slot"]],
            seg_q_start=buf[where["seg_q_start"]], seg_kv_len=buf[where["seg_kv_len"]],
            seg_slot=buf[where["seg_slot"]], groups=groups, max_q_len=1,
            max_kv_len=reach, page_size=cache.page_size, real_tokens=rows)
        # The warm-up run writes tokens of its own: the shared output may hold the tokens that
        # the step after this one takes from the device (a graph made in mid-decoding).
        self.tokens = torch.zeros(rows, dtype=torch.int32, device=device)

        def run():
            self.ctx.shared.clear()
            # rows whose token is still on the device take it from the previous replay's output
            ops.select_tokens(buf[where["token_ids"]], self.tokens, buf[where["token_src"]])
            logits = model.forward(self.ctx, cache.entries, self.row_index)
            ops.repetition_penalty(logits, buf[where["recent"]].view(rows, RECENT), f32("penalty"))
            ops.sample(logits, self.tokens, temperature=f32("temperature"), top_p=f32("top_p"),
                       top_k=buf[where["top_k"]], min_p=f32("min_p"),
                       keys=buf[where["keys"]].view(torch.int64))
            return logits

        executor.launches.begin()
        run()                               # all rows are padding: nothing is written to the cache
        self.kernels_per_replay = executor.launches.end()
        torch.cuda.synchronize(device)
        self.tokens = tokens                # the captured step reads and writes the shared output
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = run()
        torch.cuda.synchronize(device)

    def replay(self) -> None:
        self.graph.replay()
