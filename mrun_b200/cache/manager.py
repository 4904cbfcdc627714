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

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import native
from .needs import FixedState, PagedKV
from .pages import OutOfPages

FREED = -1  # block-table entry of a logical block whose page was given back (or never taken)


class RequestCache:
    """What one live request holds: a view of the native books through its state slot."""

    def __init__(self, manager: "CacheManager", request_id: object, slot: int):
        self._manager = manager
        self.request_id = request_id
        self.slot = slot
        self.released = False

    @property
    def length(self) -> int:
        """Tokens committed."""
        return 0 if self.released else self._manager._lib.mrun_cache_length(self._manager._core, self.slot)

    @property
    def pending(self) -> int:
        """Tokens of a planned, uncommitted step."""
        return 0 if self.released else self._manager._lib.mrun_cache_pending(self._manager._core, self.slot)

    @property
    def blocks(self) -> Dict[tuple, List[int]]:
        """Group key -> page per logical block (FREED where a window has passed)."""
        m = self._manager
        out = {}
        for g, (key, group) in enumerate(m.groups.items()):
            n = 0 if self.released else m._lib.mrun_cache_blocks(m._core, self.slot, g)
            out[key] = group.table[self.slot, :n].tolist()
        return out

    def block_row(self, key: tuple) -> np.ndarray:
        """The request's pages of one group as a view of the host block table."""
        m = self._manager
        n = m._lib.mrun_cache_blocks(m._core, self.slot, m._group_index[key])
        return m.groups[key].table[self.slot, :n]

    def pages_held(self, key: tuple) -> List[int]:
        return [p for p in self.blocks.get(key, ()) if p != FREED]


@dataclass
class AppendPlan:
    items: List[Tuple[RequestCache, int]]
    plan_id: int
    done: bool = False


class _PoolView:
    """The page pool of a group as the tests and the scheduler look at it."""

    def __init__(self, manager: "CacheManager", index: int, what: str):
        self._manager, self._index, self.what = manager, index, what
        self.num_pages = manager.num_pages

    @property
    def free_count(self) -> int:
        return self._manager._lib.mrun_cache_free_pages(self._manager._core, self._index)

    def is_held(self, page: int) -> bool:
        return bool(self._manager._lib.mrun_cache_is_held(self._manager._core, self._index, page))


class PagedGroup:
    """One pool of pages and the block table of every state slot: ``table[slot, block]`` is the
    page of logical block ``block`` of the request in ``slot`` (FREED where it holds none).  The
    host copy (a view of the native library's memory) is authoritative; changes are queued and
    reach the device copy in one scatter at the start of the next step
    (:meth:`CacheManager.drain_table_updates`)."""

    def __init__(self, key: tuple, window: Optional[int], max_blocks: int):
        self.key = key
        self.window = window
        self.entries: List[int] = []
        self.max_blocks = max_blocks
        self.table: np.ndarray = np.empty((0, 0), dtype=np.int32)      # set once the books exist
        self.table_device = None
        self.pool: Optional[_PoolView] = None


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
                    group = self.groups[key] = PagedGroup(key, need.window, self.max_blocks)
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

        # the books: pools, block tables, lengths, plans (csrc/host/cache_core.cpp)
        self._lib = native.library()
        windows = [-1 if g.window is None else g.window for g in self.groups.values()]
        self._core = self._lib.mrun_cache_create(len(windows), native.int_array(windows), page_size, num_pages,
                                                 max_requests, self.max_blocks)
        if not self._core:
            raise ValueError(f"bad cache sizes: page_size={page_size} num_pages={num_pages} "
                             f"max_requests={max_requests}")
        self._group_index = {key: g for g, key in enumerate(self.groups)}
        for g, (key, group) in enumerate(self.groups.items()):
            pointer = self._lib.mrun_cache_table(self._core, g)
            group.table = np.ctypeslib.as_array(pointer, shape=(max_requests, self.max_blocks))
            group.pool = _PoolView(self, g, f"pages of group {key}")
        self._by_slot: Dict[int, RequestCache] = {}

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            for group in self.groups.values():          # the views must not outlive the memory
                group.table = np.empty((0, 0), dtype=np.int32)
            self._lib.mrun_cache_destroy(core)

    def _message(self) -> str:
        return self._lib.mrun_cache_error(self._core).decode()

    # ------------------------------------------------------------------ sizes
    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def free_pages(self, key: Optional[tuple] = None) -> int:
        if key is not None:
            return self.groups[key].pool.free_count
        return min((g.pool.free_count for g in self.groups.values()), default=self.num_pages)

    @property
    def free_slots(self) -> int:
        return self._lib.mrun_cache_free_slots(self._core)

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
        slot = self._lib.mrun_cache_admit(self._core)
        if slot < 0:
            raise OutOfPages("state slots", 1, 0)
        request = RequestCache(self, request_id, slot)
        self._live[request_id] = request
        self._by_slot[slot] = request
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
        if self._lib.mrun_cache_release(self._core, request.slot):
            raise ValueError(f"request {request.request_id!r}: {self._message()}")
        request.released = True
        del self._live[request.request_id]
        del self._by_slot[request.slot]

    def trim(self, request: RequestCache, length: int) -> None:
        """Cuts the request back to its first ``length`` tokens: the pages beyond them go back
        and the next step writes from position ``length`` on (the reference's ``trim``,
        crates/mrun-engine/src/engine.rs:746, crates/mrun-engine/src/ledger.rs:400-441).  Refused
        while a step is uncommitted, and for a group whose window has already given back keys
        that the shorter request would need.  Per-request state of fixed size is not rewound:
        a mixer that keeps such state cannot be cut back."""
        if request.released:
            raise ValueError(f"request {request.request_id!r} is released")
        if length != request.length and any(e is not None and isinstance(e.need, FixedState) for e in self.entries):
            raise ValueError("a request with per-request state of fixed size cannot be cut back")
        if self._lib.mrun_cache_trim(self._core, request.slot, int(length)):
            raise ValueError(f"request {request.request_id!r}: {self._message()}")

    # ------------------------------------------------------------------ appending
    def pages_needed(self, request: RequestCache, tokens: int) -> Dict[tuple, int]:
        """Pages each group must add so that ``request`` can take ``tokens`` more."""
        target = self.blocks_for(request.length + request.pending + tokens)
        return {key: max(0, target - self._lib.mrun_cache_blocks(self._core, request.slot, g))
                for key, g in self._group_index.items()}

    def plan_append(self, items: Sequence[Tuple[RequestCache, int]]) -> AppendPlan:
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
        n = len(items)
        plan_id = self._lib.mrun_cache_plan(self._core, n, native.int_array(r.slot for r, _ in items),
                                            native.int_array(t for _, t in items))
        if plan_id < 0:
            raise ValueError(self._message())
        if plan_id == 0:
            group, wanted, free, slot = (ctypes.c_int() for _ in range(4))
            self._lib.mrun_cache_shortage(self._core, ctypes.byref(group), ctypes.byref(wanted), ctypes.byref(free),
                                          ctypes.byref(slot))
            if group.value == -2:
                raise OutOfPages(f"blocks of request {self._by_slot[slot.value].request_id!r}", wanted.value, free.value)
            key = list(self.groups)[group.value]
            raise OutOfPages(self.groups[key].pool.what, wanted.value, free.value)
        return AppendPlan(list(items), plan_id)

    def commit(self, plan: AppendPlan) -> None:
        if plan.done:
            raise ValueError("the plan was already committed or rolled back")
        plan.done = True
        if self._lib.mrun_cache_commit(self._core, plan.plan_id):
            raise ValueError(self._message())

    def rollback(self, plan: AppendPlan) -> None:
        if plan.done:
            raise ValueError("the plan was already committed or rolled back")
        plan.done = True
        if self._lib.mrun_cache_rollback(self._core, plan.plan_id):
            raise ValueError(self._message())

    def layout_step(self, slots: Sequence[int], counts: Sequence[int], positions: np.ndarray,
                    token_slot: np.ndarray, seg_q_start: np.ndarray, seg_kv_len: np.ndarray,
                    seg_slot: np.ndarray, maps: Sequence[np.ndarray]) -> int:
        """Fills the per-token arrays of a step (int32 views of the step's host buffer): entry s
        brings ``counts[s]`` tokens of the request in ``slots[s]``.  ``maps[g]`` gets each token's
        place in the pages of group g.  Returns the number of tokens."""
        as_ints = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
        pointers = (ctypes.POINTER(ctypes.c_int) * max(1, len(maps)))(*[as_ints(m) for m in maps])
        n = self._lib.mrun_cache_layout_step(self._core, len(slots), native.int_array(slots), native.int_array(counts),
                                             as_ints(positions), as_ints(token_slot), as_ints(seg_q_start),
                                             as_ints(seg_kv_len), as_ints(seg_slot), pointers)
        if n < 0:
            raise ValueError(self._message())
        return n

    # ------------------------------------------------------------------ device tables
    def drain_table_updates(self) -> Dict[tuple, Tuple[np.ndarray, np.ndarray]]:
        """The queued block-table changes per group as (flat indices, pages), oldest first with
        only the last change of an index kept; the queues are emptied."""
        out = {}
        for key, g in self._group_index.items():
            queued = self._lib.mrun_cache_pending_updates(self._core, g)
            if not queued:
                continue
            index = np.empty(queued, dtype=np.int32)
            value = np.empty(queued, dtype=np.int32)
            as_ints = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
            n = self._lib.mrun_cache_drain(self._core, g, as_ints(index), as_ints(value), queued)
            out[key] = (index[:n].copy(), value[:n].copy())
        return out

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, held by two requests, or free while held; the block tables agree with
        what the live requests hold."""
        problem = self._lib.mrun_cache_check(self._core).decode()
        if problem:
            raise AssertionError(problem)
        slots = [r.slot for r in self._live.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("two live requests share a state slot")
        if self.free_slots + len(slots) != self.max_requests:
            raise AssertionError("a state slot is lost")
