"""Which pages of a pool are free, and how many holders each page in use has.

What it must do is what the reference's pool does (``clockwork/kvcache/block.py:5-85``): a fresh
pool hands out pages 0, 1, 2, …; the page given back last is handed out next; asking for several
pages either gives all of them or changes nothing; a page with several holders is copied for the
holder that wants to write, the copy being taken before the shared page is let go, so that a pool
with no free page leaves everything as it was; and a page id that the pool does not know, or a page
that nobody holds, is an error and not a silent no-op.

How it is kept: two int arrays and a head.  ``_holders[p]`` counts the holders of page ``p``.  The
free pages form a stack threaded through ``_below``: ``_top`` is the page handed out next, and
``_below[p]`` the free page under ``p`` (``END`` under the last).  Taking and giving back are a few
array reads and writes whatever the pool's size; nothing is searched or sorted.
"""

from __future__ import annotations

from array import array

END = -1  # under the lowest page of the free stack


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for."""


class PageAllocator:
    def __init__(self, num_pages: int, page_size: int) -> None:
        if num_pages < 1 or page_size < 1:
            raise ValueError(f"a pool needs at least one page of at least one token (got {num_pages} pages of {page_size})")
        self.num_pages = num_pages
        self.page_size = page_size
        self.reset()

    def reset(self) -> None:
        """Every page free again, in the order of a fresh pool."""
        n = self.num_pages
        self._holders = array("i", bytes(4 * n))
        self._below = array("i", range(1, n + 1))
        self._below[n - 1] = END
        self._top = 0
        self.num_free = n

    # ---- taking --------------------------------------------------------------------------------
    def _pop(self) -> int:
        page = self._top
        self._top = self._below[page]
        self._holders[page] = 1
        self.num_free -= 1
        return page

    def allocate(self) -> int:
        if self.num_free == 0:
            raise OutOfPages("the pool has no free page")
        return self._pop()

    def allocate_many(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError(f"a count of pages cannot be negative ({n})")
        if n > self.num_free:
            raise OutOfPages(f"{n} pages wanted, {self.num_free} free")
        return [self._pop() for _ in range(n)]

    # ---- holders -------------------------------------------------------------------------------
    def _known(self, page: int) -> int:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is out of range: the pool has pages 0 to {self.num_pages - 1}")
        return self._holders[page]

    def _held(self, page: int) -> int:
        holders = self._known(page)
        if holders == 0:
            raise ValueError(f"page {page} is not allocated: nobody holds it")
        return holders

    def refcount(self, page: int) -> int:
        return self._known(page)

    def is_shared(self, page: int) -> bool:
        return self._known(page) > 1

    def incref(self, page: int) -> int:
        """One more holder of a page that is in use.  Returns the new count."""
        holders = self._held(page) + 1
        self._holders[page] = holders
        return holders

    def decref(self, page: int) -> int:
        """One holder fewer; the last one puts the page on top of the free stack."""
        holders = self._held(page) - 1
        self._holders[page] = holders
        if holders == 0:
            self._below[page] = self._top
            self._top = page
            self.num_free += 1
        return holders

    def free(self, page: int) -> None:
        self.decref(page)

    def free_many(self, pages: list[int]) -> None:
        for page in pages:
            self.decref(page)

    def copy_on_write(self, page: int) -> tuple[int, int] | None:
        """For a holder about to write into ``page``: None if it is the only holder; otherwise
        ``(page, copy)``, where ``copy`` is a page taken for it and its hold on ``page`` is given up.
        The caller copies the contents.  With no free page nothing changes and ``OutOfPages`` is raised."""
        if self._held(page) == 1:
            return None
        copy = self.allocate()
        self._holders[page] -= 1
        return page, copy

    # ---- checking ------------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """Every page is on the free stack exactly once or has holders; AssertionError otherwise."""
        seen = set()
        page = self._top
        while page != END:
            assert 0 <= page < self.num_pages, f"the free stack leads to {page}, which is no page"
            assert page not in seen, f"page {page} is on the free stack twice"
            assert self._holders[page] == 0, f"page {page} is free and has {self._holders[page]} holders"
            seen.add(page)
            page = self._below[page]
        assert len(seen) == self.num_free, f"{len(seen)} pages on the free stack, {self.num_free} counted"
        for page, holders in enumerate(self._holders):
            assert holders >= 0, f"page {page} has {holders} holders"
            assert (holders == 0) == (page in seen), f"page {page} has {holders} holders and is {'free' if page in seen else 'not free'}"
