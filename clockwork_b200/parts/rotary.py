"""Rotate-half (neox) rotary position encoding, fused with the write of K and V into the cache.

Reference: ``clockwork/engine/model.py:171-175`` (``inv_freq[j] = 1 / theta^(2j/rotary_dim)`` in
float32), ``:186-191`` (angle = float(position) * inv_freq), ``:32-35`` and ``:92-95`` (element j
pairs with j + rotary_dim/2).  Parameters: ``theta``, ``rotary_dim``.  No tensors: ``inv_freq``
is derived (the reference keeps it out of checkpoints too, ``model.py:169``) and always float32.

``NoPosition`` stores K and V unrotated: the interface another position encoding must have is
``apply_and_store(ctx, qkv, view, num_heads, num_kv_heads, head_dim)``.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import PagedView, PositionEncoding, StepContext
from .registry import register_position


class RotaryNeox(PositionEncoding):
    graph_safe = True
    graph_safe_portions = True

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be positive and even")
        # the reference's expression, evaluated in float32 on the host, then uploaded
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta**exponents)).to(device)

    def apply_and_store(self, ctx: StepContext, qkv: torch.Tensor, view: PagedView | None,
                        num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} exceeds head_dim {head_dim}")
        write = view is not None and view.write
        ops.rope_store(qkv, ctx.positions, view.slots if write else None, self.inv_freq,
                       view.k_cache if write else None, view.v_cache if write else None,
                       num_heads, num_kv_heads, head_dim, self.rotary_dim, ctx.status, write_cache=write)


    def fused_decode_args(self, head_dim: int):
        """(inv_freq, rotary_dim) for kernels that apply this encoding themselves, or None."""
        return (self.inv_freq, self.rotary_dim) if self.rotary_dim <= head_dim else None


class NoPosition(PositionEncoding):
    graph_safe = True
    graph_safe_portions = True

    def fused_decode_args(self, head_dim: int):
        return (None, 0)

    def apply_and_store(self, ctx, qkv, view, num_heads, num_kv_heads, head_dim) -> None:
        if view is not None and view.write:
            ops.rope_store(qkv, ctx.positions, view.slots, None, view.k_cache, view.v_cache,
                           num_heads, num_kv_heads, head_dim, 0, ctx.status, write_cache=True)


register_position("rope_neox", RotaryNeox, replace=True)
register_position("none", NoPosition, replace=True)
