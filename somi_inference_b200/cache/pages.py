"""Page pool: a stack of free page ids with loud failure on misuse.

The reference's allocator is a LIFO free list with reference counts that only
its tests use (somi_inference/core/paged_attention.py:24-59); running out of
blocks there is a bare IndexError from `list.pop()` (paged_attention.py:37).
This pool keeps the LIFO order (a page given back is the next one handed out,
which is what makes reuse show up quickly in tests), has no reference counts,
raises `OutOfPages` when empty, and refuses to free a page that is not held.
"""

from __future__ import annotations


class OutOfPages(RuntimeError):
    """A request needs more pages than the pool has free."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # page 0 is handed out first
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> list[int]:
        """Hand out `n` pages, or none at all (raises OutOfPages)."""
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._held[p] = 1
        return pages

    def give_back(self, pages: list[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} does not belong to this pool")
            if not self._held[p]:
                raise RuntimeError(f"page {p} is given back but is not held")
            self._held[p] = 0
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return bool(self._held[page])
