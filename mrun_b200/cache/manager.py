"""The cache manager: pages of keys and values with a block table per request, grouped by what
the layers need, and slots for per-request state of fixed size.

* A **group** is the set of schedule entries whose need has the same ``group_key`` (all keys, or
  a window of W keys).  A group has one page pool and, per request, one list of pages indexed by
  logical block (position // page_size).  Every owning entry of the group has key and value
  tensors ``[pages, kv_heads, page_size, head_dim]`` of its own, indexed by the same page ids.
* Appending is plan → do → commit, as the reference's ledger works
  (crates/mrun-engine/src/ledger.rs:5-9): :meth:`plan_append` takes every page the step needs
  or raises :class:`OutOfPages` with nothing changed; :meth:`commit` advances the lengths and,
  in a window group, gives back the pages the window has passed; :meth:`rollback` returns what the
  plan took.
* :meth:`release` gives back a request's pages and its state slot.  Pages are not cleared.
* A request also holds a **state slot**: a row index into each ``FixedState`` entry's tensor
  ``[max_requests, *shape]``, zeroed at admission (the reference parks the recurrent state of
  hybrid models per lane, crates/mrun-engine/src/state.rs:63-73,
  crates/mrun-engine/src/nuvec_engine.rs:143-151).  Slots exist even when no entry keeps state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool

FREED = -1  # block-table entry of a logical block whose page was given back (or never taken)


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: object
    slot: int
    length: int = 0                       # tokens committed
    pending: int = 0                      # tokens of a planned, uncommitted step
    blocks: Dict[tuple, List[int]] = field(default_factory=dict)   # group key -> page per logical block
    released: bool = False

    def pages_held(self, key: tuple) -> List[int]:
        return [p for p in self.blocks.get(key, ()) if p != FREED]


@dataclass
class AppendPlan:
    items: List[Tuple[RequestCache, int]]
    taken: List[Tuple[RequestCache, tuple, int, List[int]]]   # (request, group, first block, pages)
    done: bool = False


class PagedGroup:
    """One pool of pages and the block table of every state slot: ``table[slot, block]`` is the
    page of logical block ``block`` of the request in ``slot`` (FREED where it holds none).  The
    host copy is authoritative; changes are queued and reach the device copy in one scatter at
    the start of the next step (:meth:`CacheManager.drain_table_updates`)."""

    def __init__(self, key: tuple, window: Optional[int], num_pages: int, max_requests: int,
                 max_blocks: int):
        self.key = key
        self.window = window
        self.pool = PagePool(num_pages, what=f"pages of group {key}")
        self.entries: List[int] = []
        self.max_blocks = max_blocks
        self.table = np.full((max_requests, max_blocks), FREED, dtype=np.int32)
        self.table_device = None
        self.updates: List[Tuple[int, int]] = []        # (flat index, page)

    def set(self, slot: int, block: int, page: int) -> None:
        self.table[slot, block] = page
        self.updates.append((slot * self.max_blocks + block, page))


class EntryCache:
    """The cache of one schedule entry, as its mixer sees it."""

    def __init__(self, need, group_key, writable: bool, k=None, v=None, state=None):
        self.need = need
        self.group_key = group_key
        self.writable = writable
        self.k, self.v, self.state = k, v, state


def token_bytes(needs: Sequence[object], shares: Sequence[Optional[int]], element_size: int) -> Tuple[int, int]:
    """(bytes one token holds in the pages of every owning schedule entry, bytes of fixed-size
    state one request slot holds), from the needs alone: what a memory budget needs before any
    tensor exists.  A windowed group is counted like a full one (an upper bound)."""
    per_token = per_slot = 0
    for need, share in zip(needs, shares):
        if share is not None or need is None:
            continue
        if isinstance(need, PagedKV):
            per_token += 2 * need.kv_heads * need.head_dim * element_size
        elif isinstance(need, FixedState):
            count = 1
            for extent in need.shape:
                count *= extent
            per_slot += count * _STATE_BYTES.get(need.dtype, 4)
    return per_token, per_slot


_STATE_BYTES = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "float64": 8}


class CacheManager:
    def __init__(self, needs: Sequence[object], shares: Sequence[Optional[int]], page_size: int,
                 num_pages: int, max_requests: int, device=None, dtype=None,
                 max_blocks_per_request: Optional[int] = None):
        """``needs[i]`` is the need of schedule entry i (None: keeps nothing); ``shares[i]`` is the
        entry whose cache entry i reads instead of owning one.  ``device`` None builds the
        bookkeeping only (no tensors), which is what the host-side tests use."""
        if page_size < 1:
            raise ValueError(f"page_size must be at least 1, got {page_size}")
        if max_requests < 1:
            raise ValueError(f"max_requests must be at least 1, got {max_requests}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.device, self.dtype = device, dtype
        # a request never holds more logical blocks than its longest sequence needs
        self.max_blocks = max(1, min(max_blocks_per_request or num_pages, max(num_pages, 1)))
        self.groups: Dict[tuple, PagedGroup] = {}
        self.entries: List[Optional[EntryCache]] = []
        self._slots = PagePool(max_requests, what="state slots")
        self._live: Dict[object, RequestCache] = {}
        self._state_tensors = []

        for i, (need, share) in enumerate(zip(needs, shares)):
            if share is not None:
                owner = self.entries[share]
                if owner is None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {share}, which keeps none")
                self.entries.append(EntryCache(owner.need, owner.group_key, False, owner.k, owner.v, owner.state))
                continue
            if need is None:
                self.entries.append(None)
            elif isinstance(need, PagedKV):
                if need.window is not None and need.window < 1:
                    raise ValueError(f"schedule entry {i}: window must be at least 1, got {need.window}")
                key = need.group_key()
                group = self.groups.get(key)
                if group is None:
                    group = self.groups[key] = PagedGroup(key, need.window, num_pages, max_requests,
                                                          self.max_blocks)
                    if device is not None:
                        import torch
                        group.table_device = torch.full((max_requests, self.max_blocks), FREED,
                                                        dtype=torch.int32, device=device)
                group.entries.append(i)
                k = v = None
                if device is not None:
                    import torch
                    shape = (num_pages, need.kv_heads, page_size, need.head_dim)
                    k = torch.zeros(shape, dtype=dtype, device=device)
                    v = torch.zeros(shape, dtype=dtype, device=device)
                self.entries.append(EntryCache(need, key, True, k=k, v=v))
            elif isinstance(need, FixedState):
                state = None
                if device is not None:
                    import torch
                    state = torch.zeros((max_requests, *need.shape), dtype=getattr(torch, need.dtype),
                                        device=device)
                    self._state_tensors.append(state)
                self.entries.append(EntryCache(need, need.group_key(), True, state=state))
            else:
                raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")

    # ------------------------------------------------------------------ sizes
    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def free_pages(self, key: Optional[tuple] = None) -> int:
        if key is not None:
            return self.groups[key].pool.free_count
        return min((g.pool.free_count for g in self.groups.values()), default=self.num_pages)

    @property
    def free_slots(self) -> int:
        return self._slots.free_count

    @property
    def live(self) -> List[RequestCache]:
        return list(self._live.values())

    def bytes_per_page(self) -> int:
        total = 0
        for entry in self.entries:
            if entry is not None and entry.writable and isinstance(entry.need, PagedKV) and entry.k is not None:
                total += 2 * entry.k[0].numel() * entry.k.element_size()
        return total

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: object) -> RequestCache:
        if request_id in self._live:
            raise ValueError(f"request {request_id!r} is already live")
        (slot,) = self._slots.alloc(1)
        request = RequestCache(request_id, slot, blocks={key: [] for key in self.groups})
        self._live[request_id] = request
        for state in self._state_tensors:
            state[slot].zero_()
        return request

    def get(self, request_id: object) -> RequestCache:
        return self._live[request_id]

    def release(self, request: RequestCache) -> None:
        if request.released:
            raise ValueError(f"request {request.request_id!r} is released twice")
        if request.pending:
            raise ValueError(f"request {request.request_id!r} has an uncommitted step")
        for key, group in self.groups.items():
            group.pool.free(request.pages_held(key))
            for block, page in enumerate(request.blocks[key]):
                if page != FREED:
                    group.set(request.slot, block, FREED)
            request.blocks[key] = []
        self._slots.free([request.slot])
        request.released = True
        del self._live[request.request_id]

    # ------------------------------------------------------------------ appending
    def pages_needed(self, request: RequestCache, tokens: int) -> Dict[tuple, int]:
        """Pages each group must add so that ``request`` can take ``tokens`` more."""
        target = self.blocks_for(request.length + request.pending + tokens)
        return {key: max(0, target - len(request.blocks[key])) for key in self.groups}

    def plan_append(self, items: Sequence[Tuple[RequestCache, int]]) -> AppendPlan:
        wanted: Dict[tuple, int] = {key: 0 for key in self.groups}
        seen = set()
        for request, tokens in items:
            if request.released:
                raise ValueError(f"request {request.request_id!r} was released")
            if id(request) in seen:
                raise ValueError(f"request {request.request_id!r} is in the step twice")
            seen.add(id(request))
            if tokens < 1:
                raise ValueError(f"request {request.request_id!r}: a step brings at least one token")
            if request.pending:
                raise ValueError(f"request {request.request_id!r} has an uncommitted step")
            if self.groups and self.blocks_for(request.length + tokens) > self.max_blocks:
                raise OutOfPages(f"blocks of request {request.request_id!r}",
                                 self.blocks_for(request.length + tokens), self.max_blocks)
            for key, n in self.pages_needed(request, tokens).items():
                wanted[key] += n
        for key, n in wanted.items():
            free = self.groups[key].pool.free_count
            if n > free:
                raise OutOfPages(self.groups[key].pool.what, n, free)
        taken = []
        for request, tokens in items:
            for key, n in self.pages_needed(request, tokens).items():
                if n:
                    group = self.groups[key]
                    pages = group.pool.alloc(n)
                    first = len(request.blocks[key])
                    taken.append((request, key, first, pages))
                    request.blocks[key].extend(pages)
                    for i, page in enumerate(pages):
                        group.set(request.slot, first + i, page)
            request.pending = tokens
        return AppendPlan(list(items), taken)

    def commit(self, plan: AppendPlan) -> None:
        if plan.done:
            raise ValueError("the plan was already committed or rolled back")
        plan.done = True
        for request, tokens in plan.items:
            request.length += tokens
            request.pending = 0
            for key, group in self.groups.items():
                if group.window is None:
                    continue
                # the next token sits at position >= length and sees keys >= length - window + 1
                first_needed = max(0, request.length - group.window + 1) // self.page_size
                blocks = request.blocks[key]
                passed = [b for b in range(min(first_needed, len(blocks))) if blocks[b] != FREED]
                if passed:
                    group.pool.free([blocks[b] for b in passed])
                    for b in passed:
                        blocks[b] = FREED
                        group.set(request.slot, b, FREED)

    def rollback(self, plan: AppendPlan) -> None:
        if plan.done:
            raise ValueError("the plan was already committed or rolled back")
        plan.done = True
        for request, key, first, pages in reversed(plan.taken):
            blocks = request.blocks[key]
            assert blocks[first:first + len(pages)] == pages and len(blocks) == first + len(pages)
            del blocks[first:]
            self.groups[key].pool.free(pages)
            for i in range(len(pages)):
                self.groups[key].set(request.slot, first + i, FREED)
        for request, _ in plan.items:
            request.pending = 0

    # ------------------------------------------------------------------ device tables
    def drain_table_updates(self) -> Dict[tuple, Tuple[np.ndarray, np.ndarray]]:
        """The queued block-table changes per group as (flat indices, pages), oldest first with
        only the last change of an index kept; the queues are emptied."""
        out = {}
        for key, group in self.groups.items():
            if group.updates:
                last = dict(group.updates)          # later entries overwrite earlier ones
                out[key] = (np.fromiter(last.keys(), dtype=np.int32, count=len(last)),
                            np.fromiter(last.values(), dtype=np.int32, count=len(last)))
                group.updates = []
        return out

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, held by two requests, or free while held."""
        self._slots.check()
        slots = [r.slot for r in self._live.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("two live requests share a state slot")
        if self._slots.free_count + len(slots) != self.max_requests:
            raise AssertionError("a state slot is lost")
        for key, group in self.groups.items():
            group.pool.check()
            held: List[int] = []
            for request in self._live.values():
                held.extend(request.pages_held(key))
            if len(set(held)) != len(held):
                raise AssertionError(f"group {key}: a page is held twice")
            for page in held:
                if not group.pool.is_held(page):
                    raise AssertionError(f"group {key}: page {page} is in a block table and free")
            for request in self._live.values():
                row = self.groups[key].table[request.slot]
                blocks = request.blocks[key]
                if list(row[:len(blocks)]) != blocks or (row[len(blocks):] != FREED).any():
                    raise AssertionError(f"group {key}: the block table of slot {request.slot} differs "
                                         f"from request {request.request_id!r}'s pages")
            if len(held) + group.pool.free_count != group.pool.num_pages:
                raise AssertionError(f"group {key}: {group.pool.num_pages - len(held) - group.pool.free_count} pages lost")
