"""A pool of fixed-size pages with reference counts.

The reference keeps a free list of page ids per layer and hands them out in ascending order
(crates/ferrisinfer-runtime/src/paged_kv.rs:469-527, 794-796), and counts references to shared
blocks in a separate, metadata-only table (crates/ferrisinfer-runtime/src/block_manager.rs:58-171).
Here one pool serves every request of a page group; a page carries its own count, goes back to
the free list when the count reaches zero, and is the next one handed out (last freed, first
reused), so that stale contents of reused pages are met early rather than late.
"""

from __future__ import annotations

from ..errors import CacheError, OutOfPages


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, not {num_pages}")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))  # pop() hands out 0, 1, 2, ...
        self._refs = [0] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def alloc(self, n: int) -> list:
        """``n`` pages, each with one reference; all or nothing."""
        if n < 0:
            raise CacheError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._refs[p] = 1
        return pages

    def retain(self, page: int) -> None:
        """One more holder of a page that is in use (prefix sharing)."""
        if not (0 <= page < self.num_pages) or self._refs[page] <= 0:
            raise CacheError(f"page {page} is not in use and cannot be shared")
        self._refs[page] += 1

    def release(self, page: int) -> bool:
        """Drop one reference; True if the page went back to the free list."""
        if not (0 <= page < self.num_pages) or self._refs[page] <= 0:
            raise CacheError(f"page {page} is freed twice (or was never handed out)")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False

    def check(self, holders: dict) -> None:
        """``holders``: page -> number of block-table entries that name it.  Raises CacheError if a
        page is lost (neither free nor held), held without a count, or on the free list twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            held = holders.get(p, 0)
            if held != self._refs[p]:
                raise CacheError(f"page {p}: {held} holders but a count of {self._refs[p]}")
            if (p in free) == (held > 0):
                raise CacheError(f"page {p} is {'both free and held' if held else 'lost: neither free nor held'}")
