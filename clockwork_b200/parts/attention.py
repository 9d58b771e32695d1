"""Grouped-query causal attention over the paged cache.

Reference: ``clockwork/engine/model.py:66-128``: q/k/v projections (biased in Qwen2), position
encoding on q and k, K/V written to the cache by slot before attention reads them, causal
attention with the query aligned to the end of its request's context, output projection
(bias-free in Qwen2).  Parameters: ``hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias,
o_bias, scale, window, position`` (a position-encoding spec).  Tensors (Hugging Face names):
``q_proj/k_proj/v_proj.weight`` (+ ``.bias``), ``o_proj.weight`` (+ ``.bias``).

At load q, k and v rows are concatenated so that one product yields [q | k | v] per token.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops import attention as attention_ops
from ..weights.decl import TensorDecl
from .base import Mixer, PagedKVNeed, PagedView, ResidualStream, StepContext
from .linear import Linear
from .registry import build_part, register_mixer


class Attention(Mixer):
    takes_half_normed = True  # x only feeds the q/k/v product

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.o_bias = bool(p.get("o_bias", False))
        self.scale = float(p.get("scale", self.head_dim**-0.5))
        self.window = p.get("window")
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads {self.num_heads} not a multiple of num_kv_heads {self.num_kv_heads}")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim}: the attention kernels take multiples of 16 up to 256")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("window must be positive or None")
        self.position = build_part("position", p["position"], prefix, dtype, device)
        self.graph_safe = bool(self.position.graph_safe)
        self.graph_safe_portions = bool(getattr(self.position, "graph_safe_portions", False))
        self.qkv: Linear | None = None
        self.o: Linear | None = None

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.num_kv_heads, self.head_dim, int(self.window) if self.window else None)

    def step_scalars(self):
        """How finely the decode kernel cuts contexts is decided per step from the live requests."""
        nh, nkv, hd, device = self.num_heads, self.num_kv_heads, self.head_dim, self.device
        if self.dtype != torch.bfloat16:
            return {}
        return {attention_ops.decode_split_name(nh, nkv, hd):
                lambda num_seqs, max_ctx: attention_ops.decode_split(num_seqs, nh, nkv, max_ctx, device, hd)}

    def step_arrays(self, max_tokens: int, max_seqs: int, page_size: int, max_portions: int | None = None,
                    max_ctx: int | None = None) -> dict:
        """The work list of the prefill kernel (which 128 query rows of which request, cut how) depends on
        how a step's tokens are divided among its requests."""
        if self.dtype != torch.bfloat16:
            return {}
        return attention_ops.portion_step_arrays(self.num_heads, self.head_dim, page_size, max_tokens, max_seqs, self.device,
                                                 max_portions, max_ctx)

    def reserve_for_steps(self, max_seqs: int, max_ctx: int) -> None:
        if self.dtype == torch.bfloat16:
            attention_ops.reserve_decode_scratch(self.device, max_seqs, self.num_heads, self.num_kv_heads,
                                                 self.head_dim, max_ctx)

    def tensor_decls(self):
        q_out, kv_out = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        for proj, out in (("q_proj", q_out), ("k_proj", kv_out), ("v_proj", kv_out)):
            yield TensorDecl(self.name(f"{proj}.weight"), (out, self.hidden_size), "matrix", "linear")
            if self.qkv_bias:
                yield TensorDecl(self.name(f"{proj}.bias"), (out,), "vector", "bias")
        yield TensorDecl(self.name("o_proj.weight"), (self.hidden_size, q_out), "matrix", "linear")
        if self.o_bias:
            yield TensorDecl(self.name("o_proj.bias"), (self.hidden_size,), "vector", "bias")
        yield from self.position.tensor_decls()

    def load_weights(self, fetch) -> None:
        w = torch.cat([fetch(self.name(f"{p}.weight")) for p in ("q_proj", "k_proj", "v_proj")], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([fetch(self.name(f"{p}.bias")) for p in ("q_proj", "k_proj", "v_proj")], dim=0)
        self.qkv = Linear(w.contiguous(), b)
        self.o = Linear(fetch(self.name("o_proj.weight")), fetch(self.name("o_proj.bias")) if self.o_bias else None)
        self.position.load_weights(fetch)

    def forward(self, ctx: StepContext, x: torch.Tensor, view: PagedView, stream: ResidualStream):
        qkv = self.qkv(x)  # [N, (nh + 2 nkv) hd]
        # When every request decodes one token, the attention kernel itself rotates q and the new k and
        # stores the new k, v (one kernel less per layer), provided the position part can hand its
        # constants over; otherwise the position part runs its own kernel first.
        fused = None
        if view.write and hasattr(self.position, "fused_decode_args") and attention_ops.decode_kernel_takes(
                ctx, qkv, view, self.num_heads, self.num_kv_heads, self.head_dim, self.window):
            fused = self.position.fused_decode_args(self.head_dim)
        if fused is None:
            self.position.apply_and_store(ctx, qkv, view, self.num_heads, self.num_kv_heads, self.head_dim)
        out = attention_ops.paged_attention(ctx, qkv, view, self.num_heads, self.num_kv_heads,
                                            self.head_dim, self.scale, self.window, fused_position=fused)
        return self.o.add_or_defer(out, stream)


register_mixer("attention", Attention, replace=True)
