"""Python face of the tcgen05 matrix-product kernels (``csrc/gemm_tc.cu``, ``csrc/gemm_tc_pair.cuh``).

One entry point picks the kernel by the number of rows: up to 256 tokens one tile per CTA, the inner
dimension split over the CTAs of a thread-block cluster when the grid would idle SMs (the partial
tiles meet in distributed shared memory, so a call needs no scratch memory); more tokens run the
persistent kernels (CTA pairs without SwiGLU, single CTAs with)."""

from __future__ import annotations

from ctypes import POINTER, byref, c_float, c_int, c_longlong, c_void_p

import torch

from . import EPILOGUE_STORE, _need, _ptr, _stream, device_status, gemm as gemm_dispatch
from .library import check, library

_state: dict[int, dict] = {}
_configured = False
SPLIT_FLAG_WORDS = 8192


def _configure() -> None:
    global _configured
    if _configured:
        return
    lib = library()
    P, I, LL = c_void_p, c_int, c_longlong
    lib.cw_gemm_tc.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, P, P]
    lib.cw_gemm_tc.restype = c_int
    lib.cw_gemm_tc_norm.argtypes = [P, P, P, P, P, I, I, I, I, I, I, I, P, I, c_float, I, P, P, P, P, P]
    lib.cw_gemm_tc_norm.restype = c_int
    lib.cw_gemm_tc_plan.argtypes = [I, I, I, I, I, POINTER(c_int), POINTER(c_int), POINTER(c_int)]
    lib.cw_gemm_tc_plan.restype = c_int
    lib.cw_gemm_tc_parts_plan.argtypes = [I, I, I, I, POINTER(c_int)]
    lib.cw_gemm_tc_parts_plan.restype = c_int
    lib.cw_gemm_tc_parts.argtypes = [P, P, P, I, I, I, I, I, I, I, P, P]
    lib.cw_gemm_tc_parts.restype = c_int
    lib.cw_gemm_tc_set_persistent_from.argtypes = [I]
    lib.cw_gemm_tc_set_persistent_from.restype = c_int
    lib.cw_gemm_tc_set_pair_swiglu.argtypes = [I]
    lib.cw_gemm_tc_set_pair_swiglu.restype = c_int
    lib.cw_gemm_tc_set_pair.argtypes = [I]
    lib.cw_gemm_tc_set_pair.restype = c_int
    lib.cw_gemm_tc_set_stream.argtypes = [I]
    lib.cw_gemm_tc_set_stream.restype = c_int
    lib.cw_gemm_tc_set_tile.argtypes = [I]
    lib.cw_gemm_tc_set_tile.restype = c_int
    lib.cw_gemm_tc_set_split_flags.argtypes = [P, I]
    lib.cw_gemm_tc_set_split_flags.restype = c_int
    _configured = True


def set_token_tile(bn: int) -> None:
    """Forces the token-tile width of the prompt-portion kernels (a multiple of 16 in 64..256; 0: automatic)."""
    _configure()
    check(library().cw_gemm_tc_set_tile(int(bn)), "gemm_tc_set_tile")


def set_pair_kernel(on: bool) -> None:
    """Prompt-portion products run on CTA pairs (tcgen05 cta_group::2) by default; ``False`` keeps them
    on the single-CTA persistent kernel (for measurements and for testing that kernel)."""
    _configure()
    library().cw_gemm_tc_set_pair(1 if on else 0)


def set_pair_swiglu(on: bool) -> None:
    """The SwiGLU product of prompt portions runs on the single-CTA persistent kernel by default; ``True``
    puts it on CTA pairs (two weight tiles per stage, two accumulators per tile): measured equal within
    2 %, kept for measurements."""
    _configure()
    library().cw_gemm_tc_set_pair_swiglu(1 if on else 0)


def set_persistent_from(tokens: int) -> None:
    """From how many tokens on a product runs on the persistent kernels (for measurements)."""
    _configure()
    check(library().cw_gemm_tc_set_persistent_from(int(tokens)), "gemm_tc_set_persistent_from")


def set_stream_kernel(on: bool) -> None:
    """Products of few tokens with a very tall weight matrix (the logits) run on the persistent kernel
    with narrow token tiles by default; ``False`` gives each weight tile a CTA of its own (for measurements)."""
    _configure()
    library().cw_gemm_tc_set_stream(1 if on else 0)


def _device_state(device: torch.device) -> dict:
    index = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(index)
    if st is None:
        st = {
            "status": device_status(device),  # the word the engine reads after its steps
            "sms": torch.cuda.get_device_properties(device).multi_processor_count,
            # the words through which the splits of a tile take turns when a prompt-portion product is
            # split over its inner dimension; zero between launches, never freed
            "split_flags": torch.zeros(SPLIT_FLAG_WORDS, dtype=torch.int32, device=device),
        }
        _state[index] = st
        _configure()
        library().cw_gemm_tc_set_split_flags(_ptr(st["split_flags"]), SPLIT_FLAG_WORDS)
    return st


def status(device) -> torch.Tensor:
    return _device_state(torch.device(device))["status"]


def plan(t: int, n: int, k: int, swiglu: bool, device) -> dict:
    """How a call would be tiled: token tile, splits of the inner dimension (cluster size), CTAs."""
    _configure()
    bn, splits, ctas = c_int(0), c_int(0), c_int(0)
    library().cw_gemm_tc_plan(t, n, k, 1 if swiglu else 0, _device_state(torch.device(device))["sms"],
                              byref(bn), byref(splits), byref(ctas))
    return {"token_tile": bn.value, "splits": splits.value, "ctas": ctas.value}


def accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Sizes and alignments the TMA descriptors allow: rows of 16-byte multiples at 16-byte bases."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    k = x.shape[1]
    if k % 8 or x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8) or x.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return w.is_contiguous()


NORM_SPLIT_MAX_TOKENS = 128  # the kernel that can begin or finish a norm takes token tiles up to this


def norm_tiles(n: int) -> int:
    """Partial sums of squares per token that a product with N = ``n`` output features writes when it
    begins a norm: one per tile of 128 features."""
    return (n + 127) // 128


def _run(x, w, w2, bias, out, epilogue, row_scale=None, emit=None) -> None:
    _configure()
    st = _device_state(x.device)
    t, k = x.shape
    n = w.shape[0]
    ldx = x.stride(0) if t > 1 else max(x.stride(0), k)
    if ldx % 8:
        ldx = k
    if row_scale is None and emit is None:
        check(library().cw_gemm_tc(_ptr(x), _ptr(w), _ptr(w2), _ptr(bias), _ptr(out), t, n, k, ldx, out.stride(0), epilogue,
                                   st["sms"], _ptr(st["status"]), _stream()), "gemm_tc")
        return
    parts, eps, dim = row_scale if row_scale is not None else (None, 0.0, 1)
    if parts is not None:
        _need(parts, torch.float32, "row_scale parts", 2)
        if parts.shape[0] != t or not parts.is_contiguous():
            raise ValueError("row_scale parts must be a contiguous [T, P] tensor")
    g, ex, ep = emit if emit is not None else (None, None, None)
    if emit is not None:
        _need(g, torch.float32, "emit weight", 1)
        _need(ex, torch.bfloat16, "emit x", 2)
        _need(ep, torch.float32, "emit parts", 2)
        if g.shape[0] != n or tuple(ex.shape) != (t, n) or tuple(ep.shape) != (t, norm_tiles(n)) or not (
                ex.is_contiguous() and ep.is_contiguous()):
            raise ValueError("emit buffers must be weight [N], x [T, N], parts [T, ceil(N / 128)], contiguous")
    check(library().cw_gemm_tc_norm(
        _ptr(x), _ptr(w), _ptr(w2), _ptr(bias), _ptr(out), t, n, k, ldx, out.stride(0), epilogue, st["sms"],
        _ptr(parts), 0 if parts is None else parts.shape[1], float(eps), int(dim), _ptr(g), _ptr(ex), _ptr(ep),
        _ptr(st["status"]), _stream()), "gemm_tc_norm")


def partial_sums_splits(t: int, n: int, k: int, device) -> int:
    """Into how many slabs ``gemm_partial_sums`` would split a product of these sizes over K: 1 when
    splitting does not pay (many tiles already, a short inner dimension, or too few tokens for the
    CTA-pair kernel), and then the product is better added into its output directly."""
    _configure()
    splits = c_int(1)
    check(library().cw_gemm_tc_parts_plan(t, n, k, _device_state(torch.device(device))["sms"], byref(splits)), "gemm_tc_parts_plan")
    return splits.value


def gemm_partial_sums(x: torch.Tensor, w: torch.Tensor, splits: int):
    """``x [T,K] @ w[N,K]^T`` as ``splits`` float32 slabs whose sum, in slab order, is the product
    (``ops.PartialSums``): every split of K stores its part at once, nothing takes turns, and the
    kernel that reads the result next adds the slabs up."""
    from . import PartialSums

    _configure()
    st = _device_state(x.device)
    t, k = x.shape
    n = w.shape[0]
    slab_rows = -(-t // 16) * 16
    slabs = torch.empty((splits, slab_rows, n), dtype=torch.float32, device=x.device)
    check(library().cw_gemm_tc_parts(_ptr(x), _ptr(w), _ptr(slabs), t, n, k, x.stride(0), slab_rows, splits, st["sms"],
                                     _ptr(st["status"]), _stream()), "gemm_tc_parts")
    return PartialSums(slabs, t)


def gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out: torch.Tensor | None = None,
         epilogue: int = EPILOGUE_STORE, row_scale: tuple | None = None, emit: tuple | None = None) -> torch.Tensor:
    """``x [T,K] @ w[N,K]^T (+ bias)`` in bfloat16 on the tensor cores, float32 accumulation.
    Epilogues as for ``gemm_ref``: store bfloat16, add into float32 ``out``, store float32.

    An RMSNorm between two products can be split over them (at most ``NORM_SPLIT_MAX_TOKENS`` rows).
    ``emit=(g, xg, parts)`` with the add epilogue: beside ``out += ...`` the kernel writes
    ``xg = bf16(out * g)`` and per-token partial sums of ``out**2`` into ``parts [T, norm_tiles(N)]``.
    ``row_scale=(parts, eps, dim)``: ``x`` is such an ``xg`` and the product is multiplied, row by row,
    by ``rsqrt(parts.sum(1) / dim + eps)`` before the bias is added."""
    _need(w, torch.bfloat16, "w", 2)
    t, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"inner sizes differ: x has K={k}, w has K={w.shape[1]}")
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
    want = torch.bfloat16 if epilogue == EPILOGUE_STORE else torch.float32
    if out is None:
        if epilogue == 1:
            raise ValueError("the add epilogue needs an output to add into")
        out = torch.empty((t, n), dtype=want, device=x.device)
    _need(out, want, "out", 2)
    if tuple(out.shape) != (t, n):
        raise ValueError(f"out has shape {tuple(out.shape)}, expected {(t, n)}")
    _run(x, w, None, bias, out, epilogue, row_scale, emit)
    return out


def gemm_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, row_scale: tuple | None = None) -> torch.Tensor:
    _need(w_gate, torch.bfloat16, "w_gate", 2)
    _need(w_up, torch.bfloat16, "w_up", 2)
    if w_gate.shape != w_up.shape or w_gate.shape[1] != x.shape[1]:
        raise ValueError("gate and up weights must both be [N, K] with x's K")
    out = torch.empty((x.shape[0], w_gate.shape[0]), dtype=torch.bfloat16, device=x.device)
    _run(x, w_gate, w_up, None, out, 0, row_scale)
    return out


def enable() -> None:
    """Route the product path's bfloat16 products to this kernel."""
    import sys

    gemm_dispatch._tc = sys.modules[__name__]


enable()
