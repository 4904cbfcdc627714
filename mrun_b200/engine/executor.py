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


class Executor:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], dtype: str = "bfloat16",
                 page_size: int = 16, num_pages: int = 256, max_requests: int = 8,
                 device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("mrun_b200 runs on a CUDA device only: no GPU is visible and there "
                               "is no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.precision = Precision.of(dtype)
        self.runtime = Runtime(self.device, self.precision, page_size)
        self.spec = spec
        self.model = Model(spec, tensors, self.runtime)
        self.cache = CacheManager(self.model.cache_needs(), self.model.cache_shares(), page_size,
                                  num_pages, max_requests, device=self.device, dtype=self.precision.act)
        self.staging = HostStaging(self.device)
        self.steps_run = 0

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: object) -> RequestCache:
        return self.cache.admit(request_id)

    def release(self, request: RequestCache) -> None:
        self.cache.release(request)

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
