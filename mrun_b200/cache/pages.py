"""A pool of equally sized pages with a free list (the books are kept by the host runtime library,
``csrc/host/cache_core.cpp``).

Freed pages go on top of the list and are handed out first, so a page that one request gave back
is soon written by another without being cleared; the tests rely on that to show that nothing
reads stale contents.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List

from . import native


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots); nothing was taken."""

    def __init__(self, what: str, wanted: int, free: int):
        self.what, self.wanted, self.free = what, wanted, free
        super().__init__(f"out of {what}: {wanted} wanted, {free} free")


class PagePool:
    def __init__(self, num_pages: int, what: str = "pages"):
        if num_pages < 0:
            raise ValueError(f"num_pages must not be negative, got {num_pages}")
        self.num_pages = num_pages
        self.what = what
        self._lib = native.library()
        self._handle = self._lib.mrun_pool_create(num_pages)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.mrun_pool_destroy(handle)

    @property
    def free_count(self) -> int:
        return self._lib.mrun_pool_free_count(self._handle)

    def alloc(self, n: int) -> List[int]:
        """All ``n`` pages or :class:`OutOfPages` with nothing taken."""
        out = (ctypes.c_int * max(1, n))()
        if self._lib.mrun_pool_alloc(self._handle, n, out):
            raise OutOfPages(self.what, n, self.free_count)
        return list(out[:n])

    def free(self, pages: Iterable[int]) -> None:
        pages = [int(p) for p in pages]
        bad = ctypes.c_int(0)
        status = self._lib.mrun_pool_free(self._handle, native.int_array(pages), len(pages), ctypes.byref(bad))
        if status == 1:
            raise ValueError(f"{self.what}: page {bad.value} is outside the pool")
        if status == 2:
            raise ValueError(f"{self.what}: page {bad.value} is freed twice")

    def is_held(self, page: int) -> bool:
        return bool(self._lib.mrun_pool_is_held(self._handle, page))

    def check(self) -> None:
        """Raises if a page is lost, listed twice, or both free and held."""
        problem = self._lib.mrun_pool_check(self._handle).decode()
        if problem:
            raise AssertionError(f"{self.what}: {problem}")
