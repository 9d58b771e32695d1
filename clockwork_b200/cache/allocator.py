"""Page pool bookkeeping: reference counts, a LIFO free list, copy-on-write.

Behaviour follows the reference's ``clockwork/kvcache/block.py:5-85``: a fresh pool hands out
0, 1, 2, … (``:15-17``), a freed page is the next one handed out (``:52-57``), ``allocate_many``
takes all or nothing (``:39-45``), copy-on-write allocates before it lets go of the shared page
so that running out leaves the shared page untouched (``:74-81``), and ids that are out of range
or not allocated raise ``ValueError`` (``:23-30``).
"""

from __future__ import annotations


class OutOfPages(RuntimeError):
    """The pool cannot satisfy an allocation."""


class PageAllocator:
    def __init__(self, num_pages: int, page_size: int) -> None:
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive, got {num_pages}")
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.num_pages = num_pages
        self.page_size = page_size
        self._refcounts = [0] * num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() yields 0 first

    @property
    def num_free(self) -> int:
        return len(self._free)

    def _check_id(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page id {page} out of range [0, {self.num_pages})")

    def _check_allocated(self, page: int) -> None:
        self._check_id(page)
        if self._refcounts[page] == 0:
            raise ValueError(f"page {page} is not allocated")

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free pages")
        page = self._free.pop()
        self._refcounts[page] = 1
        return page

    def allocate_many(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise OutOfPages(f"requested {n} pages, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def incref(self, page: int) -> int:
        self._check_allocated(page)
        self._refcounts[page] += 1
        return self._refcounts[page]

    def decref(self, page: int) -> int:
        self._check_allocated(page)
        self._refcounts[page] -= 1
        if self._refcounts[page] == 0:
            self._free.append(page)
        return self._refcounts[page]

    def free(self, page: int) -> None:
        self.decref(page)

    def free_many(self, pages: list[int]) -> None:
        for page in pages:
            self.decref(page)

    def refcount(self, page: int) -> int:
        self._check_id(page)
        return self._refcounts[page]

    def is_shared(self, page: int) -> bool:
        self._check_id(page)
        return self._refcounts[page] > 1

    def copy_on_write(self, page: int) -> tuple[int, int] | None:
        """None when the page has one owner; else (src, dst) with dst freshly allocated and the
        caller's reference moved from src to dst."""
        self._check_allocated(page)
        if self._refcounts[page] == 1:
            return None
        dst = self.allocate()
        self.decref(page)
        return (page, dst)

    def reset(self) -> None:
        self._refcounts = [0] * self.num_pages
        self._free = list(range(self.num_pages - 1, -1, -1))

    def check_invariants(self) -> None:
        """Every page is either free exactly once or referenced; raises AssertionError otherwise."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        for page, count in enumerate(self._refcounts):
            assert count >= 0, f"page {page} has a negative reference count"
            assert (count == 0) == (page in free), f"page {page}: refcount {count}, on free list: {page in free}"
