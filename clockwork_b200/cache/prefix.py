"""Prefix cache: a tree over whole pages of token ids that lets a new request reuse the pages an
earlier request filled with the same leading tokens.

Behaviour follows the reference's ``clockwork/radix/tree.py`` and ``clockwork/radix/cache.py``:

* only whole pages are shared; a match never covers the whole sequence, so at least one token is
  always left to compute (``cache.py:43-47``);
* ``match`` takes one reference per matched page for the request and locks the deepest matched
  node so the path cannot be evicted while the request runs (``cache.py:51-54``);
* ``insert`` adopts (and takes a reference on) only pages the tree did not already hold for
  those tokens; duplicates stay owned by the request alone (``cache.py:58-70``);
* ``release`` undoes ``match`` (``cache.py:72-77``); ``evict`` drops least-recently-used unlocked
  leaves (``tree.py:166-187``); ``reset`` drops everything (``cache.py:85-89``).

Difference in structure: every tree node here is exactly one page (the edge label is that
page's tokens), where the reference compresses runs of pages into one node and splits nodes on
divergence (``tree.py:110-132``).  With one page per node there is nothing to split, locks sit on
nodes directly, and eviction frees exactly the number of pages asked for instead of whole runs.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .allocator import PageAllocator


class _Node:
    __slots__ = ("parent", "key", "page", "children", "last_access", "locks")

    def __init__(self, parent, key, page) -> None:
        self.parent: _Node | None = parent
        self.key: tuple[int, ...] = key
        self.page: int = page
        self.children: dict[tuple[int, ...], _Node] = {}
        self.last_access = 0
        self.locks = 0


class PrefixTree:
    def __init__(self, page_size: int) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.root = _Node(None, (), -1)
        self._clock = 0
        self._by_page: dict[int, _Node] = {}

    def num_pages(self) -> int:
        return len(self._by_page)

    def pages(self) -> list[int]:
        return list(self._by_page)

    def holds(self, page: int) -> bool:
        return page in self._by_page

    def match(self, token_ids: list[int]) -> list[int]:
        """Pages holding the longest cached prefix made of whole pages of ``token_ids``."""
        self._clock += 1
        ps = self.page_size
        node, pages = self.root, []
        for i in range(len(token_ids) // ps):
            child = node.children.get(tuple(token_ids[i * ps : (i + 1) * ps]))
            if child is None:
                break
            child.last_access = self._clock
            pages.append(child.page)
            node = child
        return pages

    def insert(self, token_ids: list[int], pages: list[int]) -> list[int]:
        """Store ``pages`` for the whole pages of ``token_ids``; returns the pages newly adopted
        (those whose tokens the tree did not hold yet)."""
        self._clock += 1
        ps = self.page_size
        n = min(len(token_ids) // ps, len(pages))
        node, adopted = self.root, []
        for i in range(n):
            key = tuple(token_ids[i * ps : (i + 1) * ps])
            child = node.children.get(key)
            if child is None:
                if pages[i] in self._by_page:
                    break  # one page cannot stand for two prefixes; keep what was adopted so far
                child = _Node(node, key, pages[i])
                node.children[key] = child
                self._by_page[pages[i]] = child
                adopted.append(pages[i])
            child.last_access = self._clock
            node = child
        return adopted

    def lock(self, page: int) -> None:
        self._by_page[page].locks += 1

    def unlock(self, page: int) -> None:
        node = self._by_page.get(page)
        if node is not None and node.locks > 0:
            node.locks -= 1

    def evictable_pages(self) -> int:
        """Pages not on the path to any locked node."""
        def walk(node: _Node) -> tuple[bool, int]:
            locked, count = node.locks > 0, 0
            for child in node.children.values():
                child_locked, child_count = walk(child)
                locked = locked or child_locked
                count += child_count
            if not locked and node is not self.root:
                count += 1
            return locked, count

        return walk(self.root)[1]

    def evict(self, num_pages: int) -> list[int]:
        """Remove up to ``num_pages`` pages, least recently used unlocked leaves first."""
        evicted: list[int] = []
        while len(evicted) < num_pages:
            leaves = [n for n in self._by_page.values() if not n.children and n.locks == 0]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.last_access)
            for victim in leaves:
                if len(evicted) >= num_pages:
                    break
                if victim.children:  # cannot happen within one pass, kept for safety
                    continue
                del victim.parent.children[victim.key]
                del self._by_page[victim.page]
                evicted.append(victim.page)
        return evicted


@dataclass
class PrefixCacheStats:
    queries: int = 0
    hit_tokens: int = 0
    prompt_tokens: int = 0

    @property
    def hit_rate(self) -> float:
        return self.hit_tokens / self.prompt_tokens if self.prompt_tokens else 0.0


@dataclass
class PrefixMatch:
    num_tokens: int
    pages: list[int] = field(default_factory=list)


class PrefixCache:
    """The tree plus page ownership: one allocator reference per page the tree holds."""

    def __init__(self, allocator: PageAllocator, page_size: int, enabled: bool = True) -> None:
        self.allocator = allocator
        self.page_size = page_size
        self.enabled = enabled
        self.stats = PrefixCacheStats()
        self.tree = PrefixTree(page_size)

    def match(self, token_ids: list[int]) -> PrefixMatch:
        self.stats.queries += 1
        self.stats.prompt_tokens += len(token_ids)
        if not token_ids or not self.enabled:
            return PrefixMatch(0)
        cap = (len(token_ids) - 1) // self.page_size * self.page_size
        if cap == 0:
            return PrefixMatch(0)
        pages = self.tree.match(token_ids[:cap])
        for page in pages:
            self.allocator.incref(page)
        if pages:
            self.tree.lock(pages[-1])
        self.stats.hit_tokens += len(pages) * self.page_size
        return PrefixMatch(len(pages) * self.page_size, pages)

    def insert(self, token_ids: list[int], pages: list[int]) -> None:
        if not self.enabled:
            return
        full = min(len(token_ids) // self.page_size, len(pages))
        if full == 0:
            return
        # spans the tree already holds keep the tree's pages; the request stays sole owner of
        # its duplicates and frees them itself
        for page in self.tree.insert(token_ids[: full * self.page_size], pages[:full]):
            self.allocator.incref(page)

    def release(self, pages: list[int]) -> None:
        if not pages:
            return
        self.tree.unlock(pages[-1])
        for page in pages:
            self.allocator.decref(page)

    def evict(self, num_pages: int) -> int:
        removed = self.tree.evict(num_pages)
        for page in removed:
            self.allocator.decref(page)
        return len(removed)

    def reset(self) -> None:
        for page in self.tree.pages():
            self.allocator.decref(page)
        self.tree = PrefixTree(self.page_size)
        self.stats = PrefixCacheStats()

    def references(self) -> dict[int, int]:
        return {page: 1 for page in self.tree.pages()}
