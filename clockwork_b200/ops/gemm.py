"""Matrix products of the product path, chosen by run precision.

float32: ``cw_gemm_ref`` (CUDA cores, fmaf, float32 throughout).
bfloat16: the tcgen05 tensor-core kernel when it takes the sizes (``cw_gemm_tc``), else the
plain kernel on bfloat16 operands."""

from __future__ import annotations

import torch

from . import EPILOGUE_ADD_F32, EPILOGUE_STORE, EPILOGUE_STORE_F32, gemm_ref, gemm_ref_swiglu

_tc = None  # set by ops.gemm_tc (imported at the end of this module)


def _use_tc(x: torch.Tensor, w: torch.Tensor) -> bool:
    return _tc is not None and x.dtype == torch.bfloat16 and _tc.accepts(x, w)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    if _use_tc(x, w):
        return _tc.gemm(x, w, bias, epilogue=EPILOGUE_STORE)
    return gemm_ref(x, w, bias, epilogue=EPILOGUE_STORE)


def linear_add_into(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor) -> None:
    if _use_tc(x, w):
        _tc.gemm(x, w, bias, out=residual, epilogue=EPILOGUE_ADD_F32)
    else:
        gemm_ref(x, w, bias, out=residual, epilogue=EPILOGUE_ADD_F32)


def linear_f32(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    if _use_tc(x, w):
        return _tc.gemm(x, w, bias, epilogue=EPILOGUE_STORE_F32)
    return gemm_ref(x, w, bias, epilogue=EPILOGUE_STORE_F32)


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T)."""
    if _use_tc(x, w_gate):
        return _tc.gemm_swiglu(x, w_gate, w_up)
    return gemm_ref_swiglu(x, w_gate, w_up)


from . import gemm_tc as _gemm_tc_module  # noqa: E402,F401  (registers itself as ``_tc``)
