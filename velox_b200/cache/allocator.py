"""Page allocator of one pool: reference-counted pages handed out from a free stack.

Semantics follow the reference's allocator (src/block_allocator.py:6-102) because traces that
run with few pages depend on them being deterministic: page 0 is reserved and never handed out
(padded rows of a batch point at it, so they always touch valid memory); the free stack starts
as N-1 .. 1 and pops from the end, so the first pages given are 1, 2, 3, ...; a page returned
is pushed on the end and is the next one given (last in, first out).
"""
from __future__ import annotations

from typing import Iterable, List

NULL_PAGE = 0


class OutOfPagesError(RuntimeError):
    """The pool has fewer free pages than were asked for."""


class PageAllocator:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 2:
            raise ValueError("a pool needs at least 2 pages (page 0 is reserved)")
        self.num_pages = num_pages
        self._refs: List[int] = [0] * num_pages
        self._refs[NULL_PAGE] = 1
        self._stack: List[int] = [page for page in range(num_pages - 1, NULL_PAGE, -1)]

    # ------------------------------------------------------------------ counts
    @property
    def num_free(self) -> int:
        return len(self._stack)

    @property
    def num_used(self) -> int:
        return self.num_pages - 1 - len(self._stack)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    # ------------------------------------------------------------------ take / give back
    def take(self, count: int = 1) -> List[int]:
        """Hand out ``count`` pages, or none at all if that many are not free."""
        if count < 0:
            raise ValueError("count must be non-negative")
        if count > len(self._stack):
            raise OutOfPagesError(f"asked for {count} pages, {len(self._stack)} are free")
        pages = []
        for _ in range(count):
            page = self._stack.pop()
            self._refs[page] = 1
            pages.append(page)
        return pages

    def share(self, page: int) -> int:
        """Add a holder to a page that is in use."""
        self._check(page)
        if self._refs[page] <= 0:
            raise RuntimeError(f"page {page} is free and cannot be shared")
        self._refs[page] += 1
        return self._refs[page]

    def give_back(self, page: int) -> int:
        """Drop one holder; the page becomes free when the last holder is gone."""
        self._check(page)
        if page == NULL_PAGE:
            return self._refs[page]
        if self._refs[page] <= 0:
            raise RuntimeError(f"page {page} was given back twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._stack.append(page)
        return self._refs[page]

    def give_back_all(self, pages: Iterable[int]) -> None:
        for page in pages:
            self.give_back(page)

    def holders(self, page: int) -> int:
        self._check(page)
        return self._refs[page]

    def _check(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise IndexError(f"page {page} is outside [0, {self.num_pages})")

    # ------------------------------------------------------------------ invariants
    def assert_consistent(self) -> None:
        """No page is both free and held, free twice, or held a negative number of times."""
        free = set(self._stack)
        if len(free) != len(self._stack):
            raise AssertionError("a page is on the free stack twice")
        if NULL_PAGE in free:
            raise AssertionError("the reserved page is on the free stack")
        for page, refs in enumerate(self._refs):
            if refs < 0:
                raise AssertionError(f"page {page} has {refs} holders")
            if (refs == 0) != (page in free):
                raise AssertionError(f"page {page}: holders={refs}, on free stack={page in free}")

    def __repr__(self) -> str:
        return f"PageAllocator(pages={self.num_pages}, free={self.num_free}, used={self.num_used})"
