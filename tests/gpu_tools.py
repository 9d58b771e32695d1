"""Helpers of the GPU tests: build a cache and a step context for a part under test."""

from __future__ import annotations

import torch

from clockwork_b200 import ops
from clockwork_b200.cache import CacheManager
from clockwork_b200.engine.step import StepBuilder, StepEntry

DEV = "cuda:0"


class PartHarness:
    """A cache manager plus step builder around one mixer's cache need (cache layer 0)."""

    def __init__(self, needs: dict, dtype: torch.dtype, num_pages: int = 64, page_size: int = 8, slots: int = 8):
        self.cache = CacheManager(needs, num_pages=num_pages, page_size=page_size, dtype=dtype, device=DEV,
                                  num_state_slots=slots)
        self.status = self.cache.status
        self.builder = StepBuilder(self.cache, dtype, DEV, self.status)

    def prepare(self, portions: dict[str, int]):
        """portions: request id -> number of next tokens (token ids do not matter to a part)."""
        entries = []
        for rid, n in portions.items():
            if rid not in self.cache.requests:
                self.cache.open(rid)
            entries.append(StepEntry(rid, [0] * n, []))
        return self.builder.prepare(entries)

    def commit(self, prepared) -> None:
        self.builder.commit(prepared)
        ops.raise_on_status(self.status)
