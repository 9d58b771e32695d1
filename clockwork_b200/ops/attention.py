"""Chooses the attention kernel for a step.

float32 runs use the general kernel (``cw_attention_ref``) for everything.  bfloat16 runs use
the split-context decode kernel when every request brings one token and the tensor-core
prefill kernel for prompt portions, when those kernels take the sizes; otherwise the general
kernel on bfloat16 data.  All of them read the same cache through the same block tables."""

from __future__ import annotations

import torch

from . import attention_ref

_decode = None  # set by ops.attention_decode when present
_prefill = None  # set by ops.attention_prefill when present


def decode_kernel_takes(ctx, qkv: torch.Tensor, view, num_heads: int, num_kv_heads: int, head_dim: int,
                        window: int | None) -> bool:
    """Whether this step's attention will run in the split-context decode kernel (which can also do
    the position encoding and the cache write of the new token itself)."""
    return (qkv.dtype == torch.bfloat16 and ctx.all_single_token and _decode is not None
            and _decode.accepts(ctx, view, num_heads, num_kv_heads, head_dim, window))


def decode_split_name(num_heads: int, num_kv_heads: int, head_dim: int) -> str:
    """Name of the per-step device scalar (``Part.step_scalars``) that holds the tokens per CTA of the
    decode kernel for layers of these sizes."""
    return f"attention_decode_split/{num_heads}/{num_kv_heads}/{head_dim}"


def decode_split(num_seqs: int, num_heads: int, num_kv_heads: int, max_ctx: int, device, head_dim: int) -> int:
    return _attention_fast_module.decode_split(num_seqs, num_heads, num_kv_heads, max_ctx, device, head_dim)


def portion_step_arrays(num_heads: int, head_dim: int, page_size: int, max_tokens: int, max_seqs: int, device,
                        max_portions: int | None = None, max_ctx: int | None = None) -> dict:
    """What ``Part.step_arrays`` of an attention layer of these sizes returns: the prefill kernel's work
    list, for captured steps that hold prompt portions (empty when the bfloat16 kernels do not take the
    head size: such a model's steps are not captured)."""
    return _attention_fast_module.portion_step_arrays(num_heads, head_dim, page_size, max_tokens, max_seqs, device, max_portions,
                                                      max_ctx)


def reserve_decode_scratch(device, max_seqs: int, num_heads: int, num_kv_heads: int, head_dim: int, max_ctx: int) -> None:
    if head_dim in _attention_fast_module.DECODE_HEAD_DIMS:
        _attention_fast_module.reserve_decode_scratch(device, max_seqs, num_heads, num_kv_heads, head_dim, max_ctx)


def paged_attention(ctx, qkv: torch.Tensor, view, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int | None, fused_position=None) -> torch.Tensor:
    """``fused_position`` = (inv_freq or None, rotary_dim): q and k in ``qkv`` are still raw and the new
    token is not in the cache yet; only valid when ``decode_kernel_takes`` said yes."""
    if qkv.dtype == torch.bfloat16:
        if ctx.all_single_token and _decode is not None and _decode.accepts(ctx, view, num_heads, num_kv_heads, head_dim, window):
            return _decode.run(ctx, qkv, view, num_heads, num_kv_heads, head_dim, scale, window,
                               fused_position=fused_position)
    if fused_position is not None:
        raise RuntimeError("fused position encoding was asked of a kernel that does not do it")
    if qkv.dtype == torch.bfloat16:
        if not ctx.all_single_token and _prefill is not None and _prefill.accepts(ctx, view, num_heads, num_kv_heads, head_dim, window):
            return _prefill.run(ctx, qkv, view, num_heads, num_kv_heads, head_dim, scale, window)
    return attention_ref(qkv, view.k_cache, view.v_cache, view.block_tables, ctx.tok_seq, ctx.positions,
                         num_heads, num_kv_heads, head_dim, scale, window, ctx.status)


from . import attention_fast as _attention_fast_module  # noqa: E402,F401  (registers the bfloat16 kernels)
