"""A pool of equally sized pages with a free list.

Freed pages go on top of the list and are handed out first, so a page that one request gave back
is soon written by another without being cleared; the tests rely on that to show that nothing
reads stale contents.
"""
from __future__ import annotations

from typing import Iterable, List


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
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        """All ``n`` pages or :class:`OutOfPages` with nothing taken."""
        if n > len(self._free):
            raise OutOfPages(self.what, n, len(self._free))
        taken = [self._free.pop() for _ in range(n)]
        for page in taken:
            self._held[page] = True
        return taken

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise ValueError(f"{self.what}: page {page} is outside the pool")
            if not self._held[page]:
                raise ValueError(f"{self.what}: page {page} is freed twice")
            self._held[page] = False
        self._free.extend(pages)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> None:
        """Raises if a page is lost, listed twice, or both free and held."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError(f"{self.what}: a page is on the free list twice")
        for page in self._free:
            if self._held[page]:
                raise AssertionError(f"{self.what}: page {page} is free and held")
        if len(self._free) + sum(self._held) != self.num_pages:
            raise AssertionError(f"{self.what}: {self.num_pages - len(self._free) - sum(self._held)} pages lost")
