"""Matrix products of the product path, chosen by run precision.

float32: ``cw_gemm_ref`` (CUDA cores, fmaf, float32 throughout).
bfloat16: the tcgen05 tensor-core kernel when it takes the sizes (``cw_gemm_tc``), else the
plain kernel on bfloat16 operands."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from . import EPILOGUE_ADD_F32, EPILOGUE_STORE, EPILOGUE_STORE_F32, gemm_ref, gemm_ref_swiglu

_tc = None  # set by ops.gemm_tc (imported at the end of this module)


@dataclass
class RowScaled:
    """An activation whose RMSNorm is half done: ``x = bf16(residual * norm_weight)`` and, per row,
    ``parts`` whose sum is the row's sum of squares.  The product that consumes it multiplies its
    result by ``rsqrt(parts.sum(1) / dim + eps)`` in its epilogue; ``materialize`` runs the norm kernel
    on the residual instead, for a consumer that wants a plain tensor."""

    x: torch.Tensor
    parts: torch.Tensor
    eps: float
    dim: int
    materialize: Callable[[], torch.Tensor]

    @property
    def shape(self):
        return self.x.shape

    def row_scale(self) -> tuple:
        return (self.parts, self.eps, self.dim)


def _use_tc(x: torch.Tensor, w: torch.Tensor) -> bool:
    return _tc is not None and x.dtype == torch.bfloat16 and _tc.accepts(x, w)


def can_split_norm(rows: int, dtype: torch.dtype) -> bool:
    """Whether products of this many rows can begin and finish a norm in their epilogues."""
    return _tc is not None and dtype == torch.bfloat16 and 0 < rows <= _tc.NORM_SPLIT_MAX_TOKENS


def _plain(x):
    """(tensor, row_scale or None): a half-normed activation stays so only if the tensor-core kernel takes it."""
    if isinstance(x, RowScaled):
        return x, x.x
    return None, x


def linear(x, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    lazy, xt = _plain(x)
    if lazy is not None:
        if _use_tc(xt, w) and can_split_norm(xt.shape[0], xt.dtype):
            return _tc.gemm(xt, w, bias, epilogue=EPILOGUE_STORE, row_scale=lazy.row_scale())
        xt = lazy.materialize()
    if _use_tc(xt, w):
        return _tc.gemm(xt, w, bias, epilogue=EPILOGUE_STORE)
    return gemm_ref(xt, w, bias, epilogue=EPILOGUE_STORE)


def linear_add_into(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor,
                    begin_norm: torch.Tensor | None = None):
    """residual += x W^T (+ bias).  ``begin_norm``: the weight [N] of an RMSNorm that follows; when the
    sizes allow, the kernel also begins that norm and ``(xg, parts)`` is returned (see ``RowScaled``),
    else None."""
    if _use_tc(x, w):
        if (begin_norm is not None and can_split_norm(x.shape[0], x.dtype) and begin_norm.dtype == torch.float32
                and begin_norm.shape[0] == w.shape[0]):
            t, n = x.shape[0], w.shape[0]
            xg = torch.empty((t, n), dtype=torch.bfloat16, device=x.device)
            parts = torch.empty((t, _tc.norm_tiles(n)), dtype=torch.float32, device=x.device)
            _tc.gemm(x, w, bias, out=residual, epilogue=EPILOGUE_ADD_F32, emit=(begin_norm, xg, parts))
            return xg, parts
        _tc.gemm(x, w, bias, out=residual, epilogue=EPILOGUE_ADD_F32)
    else:
        gemm_ref(x, w, bias, out=residual, epilogue=EPILOGUE_ADD_F32)
    return None


def linear_partial_sums(x: torch.Tensor, w: torch.Tensor):
    """x W^T as ``ops.PartialSums`` when the product is one whose inner dimension is worth splitting with
    the splits kept apart (a few hundred tokens against a long K: few tiles, and splits that add into
    the residual one after the other would take turns), else None.  The width must suit the kernel
    that adds the slabs up (a multiple of 4, at most 4096)."""
    n = w.shape[0]
    if not _use_tc(x, w) or n % 4 or n > 4096 or x.stride(1) != 1:
        return None
    splits = _tc.partial_sums_splits(x.shape[0], n, x.shape[1], x.device)
    if splits <= 1:
        return None
    return _tc.gemm_partial_sums(x, w, splits)


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    if _use_tc(x, w):
        return _tc.gemm(x, w, bias, epilogue=EPILOGUE_STORE_F32)
    return gemm_ref(x, w, bias, epilogue=EPILOGUE_STORE_F32)


def swiglu(x, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T)."""
    lazy, xt = _plain(x)
    if lazy is not None:
        if _use_tc(xt, w_gate) and can_split_norm(xt.shape[0], xt.dtype):
            return _tc.gemm_swiglu(xt, w_gate, w_up, row_scale=lazy.row_scale())
        xt = lazy.materialize()
    if _use_tc(xt, w_gate):
        return _tc.gemm_swiglu(xt, w_gate, w_up)
    return gemm_ref_swiglu(xt, w_gate, w_up)


from . import gemm_tc as _gemm_tc_module  # noqa: E402,F401  (registers itself as ``_tc``)
