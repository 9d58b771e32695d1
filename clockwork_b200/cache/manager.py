"""The cache manager: pages of keys and values with a block table per request, one page pool per
group of layers with the same needs, and slots for per-request state of fixed size.

What the reference has (``clockwork/kvcache/block_manager.py:6-101``, ``kv_cache.py:4-56``): one
pool for all layers, per layer K and V tensors ``[num_blocks, block_size, kv_heads, head_dim]``, a
block table per sequence, ``slot = page * page_size + position % page_size``, admission with a
watermark (``:31-36``), growth by one slot with copy-on-write of a shared tail page (``:48-75``),
``fork`` (``:77-83``), ``free`` with a double-free guard (``:85-90``).

What is added: layers are sorted into *groups* by what their mixer keeps (``PagedKVNeed``: KV
head count, head size, window).  Each group has its own pool, allocator and per-request block
table, so layers that keep every key and layers that keep a window of them never share pages;
a windowed group gives pages back as soon as the window has passed them.  Mixers that keep a
state of fixed size (``SlotStateNeed``) get a row per request in a slot tensor instead of pages.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import PagedKVNeed, PagedView, SlotStateNeed, StateView
from .allocator import OutOfPages, PageAllocator

NO_PAGE = -1


class PageGroup:
    """Layers with identical needs: one allocator, one device tensor
    ``[layers, 2 (K, V), pages, page_size, kv_heads, head_dim]``."""

    def __init__(self, need: PagedKVNeed, cache_layers: list[int], num_pages: int, page_size: int,
                 dtype: torch.dtype | None, device) -> None:
        self.need = need
        self.cache_layers = list(cache_layers)
        self.page_size = page_size
        self.allocator = PageAllocator(num_pages, page_size)
        self.kv: torch.Tensor | None = None
        if device is not None and dtype is not None:
            self.kv = torch.zeros(
                (len(cache_layers), 2, num_pages, page_size, need.num_kv_heads, need.head_dim),
                dtype=dtype, device=device,
            )
        self._index = {layer: i for i, layer in enumerate(self.cache_layers)}

    def layer_kv(self, cache_layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        plane = self.kv[self._index[cache_layer]]
        return plane[0], plane[1]

    def bytes_per_token(self) -> int:
        elem = self.kv.element_size() if self.kv is not None else 2
        return len(self.cache_layers) * 2 * self.need.num_kv_heads * self.need.head_dim * elem


@dataclass
class RequestCache:
    """What one request holds."""

    request_id: str
    tables: list[list[int]]  # per group: logical block -> page (NO_PAGE once given back)
    num_tokens: int = 0  # positions [0, num_tokens) have a slot reserved
    num_computed: int = 0  # positions [0, num_computed) have their keys/values (or state) stored
    shared_prefix_pages: int = 0  # leading pages of group 0 owned through the prefix cache
    state_slot: int | None = None
    live_from: list[int] = field(default_factory=list)  # per group: first logical block still held
    table_epoch: int = 0  # counts changes of existing table entries (a copied page): holders of a copy of the table compare it
    writable_len: int = 0  # positions below this need neither a new page nor a copy: the request owns their pages alone


REQUEST_STATE_FIELDS = ("position", "last_token", "draws", "seed_lo", "seed_hi", "temperature", "top_k", "top_p")


class StateSlots:
    """Per-request state of fixed size.  Every request that holds cache also holds one slot, which
    names its column in

    * ``request``: an int32 table ``[fields, slots]`` on the device with the request's progress and
      sampling state, ``{position, last_token, draws, seed (two words), temperature, top_k, top_p}``
      (floats as their bits).  Single-token steps read their inputs from it and the sampling kernels
      write the new token back (``csrc/request_state.cu``), so that such a step does not wait for the
      host.  The reference keeps the same on the host (``clockwork/engine/model_runner.py:46``,
      ``139-145``: Sequence fields and a CPU generator per request).
    * one tensor ``[slots, *shape]`` per cache layer whose mixer asked for state of its own
      (``SlotStateNeed``), zeroed when a request takes the slot, plus one scratch row for the padding
      rows of captured steps.  This architecture has none."""

    def __init__(self, needs: dict[int, SlotStateNeed], num_slots: int, device) -> None:
        self.num_slots = num_slots
        self.needs = dict(needs)
        self._free = list(range(num_slots - 1, -1, -1))
        self._owner: dict[int, str] = {}
        self.tensors: dict[int, torch.Tensor] = {}
        self.request: torch.Tensor | None = None
        self.scratch_slot = num_slots  # a row beyond the requests' rows: where padding rows of a fixed-shape step read and write
        if device is not None:
            for layer, need in needs.items():
                self.tensors[layer] = torch.zeros((num_slots + 1, *need.shape), dtype=need.dtype, device=device)
            self.request = torch.zeros((len(REQUEST_STATE_FIELDS), num_slots), dtype=torch.int32, device=device)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, request_id: str) -> int:
        if not self._free:
            raise OutOfPages("no free state slots")
        slot = self._free.pop()
        self._owner[slot] = request_id
        for t in self.tensors.values():
            t[slot].zero_()
        return slot

    def give_back(self, slot: int) -> None:
        if slot not in self._owner:
            raise ValueError(f"state slot {slot} is not in use (double free?)")
        del self._owner[slot]
        self._free.append(slot)

    def copy(self, src: int, dst: int) -> None:
        for t in self.tensors.values():
            t[dst].copy_(t[src])

    def check_invariants(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free), "a state slot is on the free list twice"
        assert not (free & set(self._owner)), "a state slot is both free and owned"
        assert len(free) + len(self._owner) == self.num_slots, "a state slot was lost"


class CacheManager:
    def __init__(self, needs: dict[int, PagedKVNeed | SlotStateNeed], num_pages: int, page_size: int,
                 dtype: torch.dtype | None = None, device=None, num_state_slots: int = 64,
                 watermark: float = 0.0) -> None:
        if watermark < 0:
            raise ValueError(f"watermark must be non-negative, got {watermark}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.device = torch.device(device) if device is not None else None
        by_need: dict[PagedKVNeed, list[int]] = {}
        state_needs: dict[int, SlotStateNeed] = {}
        for layer in sorted(needs):
            need = needs[layer]
            if isinstance(need, PagedKVNeed):
                by_need.setdefault(need, []).append(layer)
            elif isinstance(need, SlotStateNeed):
                state_needs[layer] = need
            else:
                raise TypeError(f"cache layer {layer}: unknown need {need!r}")
        self.groups = [PageGroup(need, layers, num_pages, page_size, dtype, device) for need, layers in by_need.items()]
        self.group_of_layer = {layer: g for g, group in enumerate(self.groups) for layer in group.cache_layers}
        self.state = StateSlots(state_needs, num_state_slots, device)
        self.watermark_pages = int(watermark * num_pages)  # clockwork/kvcache/block_manager.py:20
        self.requests: dict[str, RequestCache] = {}
        self.status: torch.Tensor | None = None
        if self.device is not None and self.device.type == "cuda":
            from .. import ops

            self.status = ops.device_status(self.device)

    # ---- requests ---------------------------------------------------------------------------
    def open(self, request_id: str, shared_prefix: list[int] | None = None) -> RequestCache:
        """Start holding memory for a request.  ``shared_prefix``: pages of group 0 that already
        hold its first tokens (a prefix-cache hit; the caller took the references)."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} already holds cache")
        req = RequestCache(request_id, [[] for _ in self.groups], live_from=[0] * len(self.groups))
        if shared_prefix:
            if len(self.groups) != 1 or self.groups[0].need.window is not None or self.state.needs:
                raise ValueError("shared prefixes need a single group of full-attention layers")
            req.tables[0] = list(shared_prefix)
            req.shared_prefix_pages = len(shared_prefix)
            req.num_tokens = len(shared_prefix) * self.page_size
            req.num_computed = req.num_tokens
        req.state_slot = self.state.take(request_id)
        self.requests[request_id] = req
        return req

    def get(self, request_id: str) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise ValueError(f"request {request_id!r} holds no cache (double free?)") from None

    def _blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def pages_needed(self, req: RequestCache, new_len: int) -> list[int]:
        """Per group: pages to allocate so that positions [0, new_len) have slots, counting a
        page for copy-on-write when the page that the next token lands in is shared."""
        need = []
        for g, group in enumerate(self.groups):
            table = req.tables[g]
            n = max(0, self._blocks_for(new_len) - len(table))
            if new_len > req.num_tokens:
                blk = req.num_tokens // self.page_size
                if blk < len(table) and table[blk] != NO_PAGE and group.allocator.is_shared(table[blk]):
                    n += 1
            need.append(n)
        return need

    def can_reserve(self, req: RequestCache, new_len: int, keep_watermark: bool = False) -> bool:
        """clockwork/kvcache/block_manager.py:31-36 (admission leaves the watermark free) and
        :48-54 (growth needs the pages only)."""
        if new_len <= req.writable_len:
            return True  # the common decode step: the next token lands in a page the request owns alone
        floor = self.watermark_pages if keep_watermark else 0
        return all(
            group.allocator.num_free - n >= floor
            for group, n in zip(self.groups, self.pages_needed(req, new_len))
        )

    def can_open(self, num_tokens: int, shared_pages: int = 0) -> bool:
        """Whether a new request of ``num_tokens`` could be given its pages and a state slot with
        the watermark left free."""
        if self.state.num_free == 0:
            return False
        need = max(0, self._blocks_for(num_tokens) - shared_pages)
        return all(g.allocator.num_free - need >= self.watermark_pages for g in self.groups)

    def reserve(self, req: RequestCache, new_len: int) -> None:
        """Make sure positions [0, new_len) have slots in every group: allocate pages, and give
        the request its own copy of a shared page that it is about to write into
        (clockwork/kvcache/block_manager.py:56-75).  All or nothing."""
        if new_len <= req.num_tokens:
            return
        if new_len <= req.writable_len:
            req.num_tokens = new_len
            return
        if not self.can_reserve(req, new_len):
            raise OutOfPages(f"request {req.request_id!r}: not enough free pages to reach {new_len} tokens")
        for g, group in enumerate(self.groups):
            table = req.tables[g]
            blk = req.num_tokens // self.page_size
            if blk < len(table) and table[blk] != NO_PAGE:
                cow = group.allocator.copy_on_write(table[blk])
                if cow is not None:
                    src, dst = cow
                    self._copy_page(group, src, dst)
                    table[blk] = dst
                    req.table_epoch += 1
                    if g == 0 and blk < req.shared_prefix_pages:
                        req.shared_prefix_pages = blk  # no longer the prefix cache's page
            missing = self._blocks_for(new_len) - len(table)
            if missing > 0:
                table.extend(group.allocator.allocate_many(missing))
        req.num_tokens = new_len
        # From the page that new_len - 1 falls into onwards, every page was allocated or copied for this
        # request just now or earlier, so nobody else holds it (until a fork, which resets this).
        req.writable_len = min(len(t) for t in req.tables) * self.page_size if req.tables else new_len

    def _copy_page(self, group: PageGroup, src: int, dst: int) -> None:
        if group.kv is None:
            return
        from .. import ops

        planes = group.kv.view(group.kv.shape[0] * 2, *group.kv.shape[2:])
        pairs = torch.tensor([[src, dst]], dtype=torch.int32, device=group.kv.device)
        ops.copy_pages(planes, pairs, self.status)

    def release_behind_window(self, req: RequestCache, computed: int) -> int:
        """Give back pages of windowed groups that no later token can read: a query at position
        p >= computed reads keys in [p + 1 - window, p] only.  Returns the number given back."""
        given = 0
        for g, group in enumerate(self.groups):
            window = group.need.window
            if window is None:
                continue
            first_needed = max(0, computed + 1 - window)
            keep_from = first_needed // self.page_size
            table = req.tables[g]
            for blk in range(req.live_from[g], min(keep_from, len(table))):
                if table[blk] != NO_PAGE:
                    group.allocator.decref(table[blk])
                    table[blk] = NO_PAGE
                    given += 1
            req.live_from[g] = max(req.live_from[g], min(keep_from, len(table)))
        return given

    def fork(self, parent: RequestCache, child_id: str) -> RequestCache:
        """A child that shares every page of the parent (clockwork/kvcache/block_manager.py:77-83);
        the first write into a shared page copies it.  Fixed-size state is copied."""
        if child_id in self.requests:
            raise ValueError(f"request {child_id!r} already holds cache")
        child = RequestCache(child_id, [list(t) for t in parent.tables], num_tokens=parent.num_computed,
                             num_computed=parent.num_computed, shared_prefix_pages=0,
                             live_from=list(parent.live_from))
        for g, group in enumerate(self.groups):
            for page in child.tables[g]:
                if page != NO_PAGE:
                    group.allocator.incref(page)
        parent.writable_len = 0  # its pages are shared now: the next write must look (and copy)
        child.state_slot = self.state.take(child_id)
        self.state.copy(parent.state_slot, child.state_slot)
        self.requests[child_id] = child
        return child

    def truncate(self, req: RequestCache, num_tokens: int) -> None:
        """Forget reservations beyond ``num_tokens`` (pages stay; used when a planned step is dropped)."""
        req.num_tokens = min(req.num_tokens, num_tokens)

    def close(self, request_id: str) -> list[int]:
        """Give back everything the request holds.  Returns the leading pages of group 0 that
        belong to the prefix cache (the caller releases those references there)."""
        req = self.get(request_id)
        del self.requests[request_id]
        shared: list[int] = []
        for g, group in enumerate(self.groups):
            table = req.tables[g]
            start = 0
            if g == 0 and req.shared_prefix_pages:
                shared = table[: req.shared_prefix_pages]
                start = req.shared_prefix_pages
            for page in table[start:]:
                if page != NO_PAGE:
                    group.allocator.decref(page)
            table.clear()
        if req.state_slot is not None:
            self.state.give_back(req.state_slot)
            req.state_slot = None
        return shared

    # ---- what a step needs --------------------------------------------------------------------
    def slots(self, req: RequestCache, group: int, start: int, end: int) -> list[int]:
        """clockwork/kvcache/block_manager.py:92-98."""
        table, size = req.tables[group], self.page_size
        if not 0 <= start <= end <= len(table) * size:
            raise ValueError(f"token range [{start}, {end}) outside the covered range [0, {len(table) * size})")
        out = []
        for pos in range(start, end):
            page = table[pos // size]
            if page == NO_PAGE:
                raise ValueError(f"position {pos} lies in a page that was already given back")
            out.append(page * size + pos % size)
        return out

    def views(self, block_tables: list[torch.Tensor], slots: list[torch.Tensor], state_slots: torch.Tensor | None,
              state_slots_host: list[int]) -> dict[int, PagedView | StateView]:
        """Per cache layer, what its mixer sees this step."""
        out: dict[int, PagedView | StateView] = {}
        for g, group in enumerate(self.groups):
            for layer in group.cache_layers:
                k, v = group.layer_kv(layer)
                out[layer] = PagedView(k, v, block_tables[g], slots[g], True)
        for layer, tensor in self.state.tensors.items():
            out[layer] = StateView(tensor, state_slots, list(state_slots_host))
        return out

    # ---- accounting -----------------------------------------------------------------------------
    def num_free_pages(self) -> list[int]:
        return [g.allocator.num_free for g in self.groups]

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def check_invariants(self, extra_refs: dict[int, int] | None = None) -> None:
        """No page lost, held twice without a reference for each holder, or freed twice.
        ``extra_refs``: references to pages of group 0 held outside (the prefix cache)."""
        for g, group in enumerate(self.groups):
            group.allocator.check_invariants()
            held: dict[int, int] = {}
            for req in self.requests.values():
                for page in req.tables[g]:
                    if page != NO_PAGE:
                        held[page] = held.get(page, 0) + 1
            if g == 0 and extra_refs:
                for page, n in extra_refs.items():
                    held[page] = held.get(page, 0) + n
            for page in range(group.allocator.num_pages):
                assert group.allocator.refcount(page) == held.get(page, 0), (
                    f"group {g} page {page}: refcount {group.allocator.refcount(page)}, holders {held.get(page, 0)}"
                )
        self.state.check_invariants()
