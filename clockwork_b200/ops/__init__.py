"""Python faces of the CUDA kernels.  Each checks shapes, dtypes and contiguity, then calls the
``extern "C"`` entry point on the current CUDA stream.  Tensors must live on a CUDA device;
nothing here has a CPU path."""

from __future__ import annotations

import ctypes

import torch

from .library import KernelLibraryError, check, library, serial_launch, set_pdl

__all__ = [
    "KernelLibraryError", "library", "dtype_code", "new_status", "device_status", "raise_on_status",
    "embed", "add_rmsnorm", "rmsnorm_rows", "silu_mul", "add_to_residual", "gemm_ref",
    "gemm_ref_swiglu", "rope_store", "copy_pages", "attention_ref", "argmax", "sample", "step_from_state",
    "REQUEST_STATE_FIELDS",
]

STATUS_MESSAGES = {
    1: "token id outside the vocabulary (row {a}, id {b})",
    2: "cache slot outside the pool (token {a}, slot {b})",
    3: "page id outside the pool ({a}, {b})",
    4: "a device-side wait ran out (kernel {a}, stage {b})",
    5: "row index outside the batch (row {a}, index {b})",
    6: "shared memory of block {a} is not 1024-byte aligned (offset {b})",
    7: "work item {a} names a cut of its keys that the kernel does not take (word {b})",
    8: "the context split of a decode step is longer than the bound its page list was sized for (request {a}, split {b})",
}


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise ValueError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked of torch's C layer directly: the Python-level
    ``torch.cuda.current_stream()`` costs more than the launch it is asked for."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype | None, name: str, ndim: int | None = None) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


_device_status: dict[int, torch.Tensor] = {}


def device_status(device) -> torch.Tensor:
    """The one status word set of a device that the engine's kernels report into: the cache manager,
    the step function and the tensor-core products all hand this to their kernels, so that one read
    (``raise_on_status``) sees whatever any of them recorded.  Never freed (captured graphs hold its
    address)."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    status = _device_status.get(index)
    if status is None:
        status = _device_status[index] = new_status(torch.device("cuda", index))
    return status


def raise_on_status(status: torch.Tensor) -> None:
    """Reads the status words (one small device-to-host copy) and raises if a kernel
    recorded an out-of-range index."""
    code, a, b, _ = status.tolist()
    if code != 0:
        status.zero_()
        raise RuntimeError("kernel status: " + STATUS_MESSAGES.get(code, f"code {code}").format(a=a, b=b))


def embed(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor, serial: bool = False) -> torch.Tensor:
    """float32 [N, H] rows of ``table`` (float32 or bfloat16 [V, H]) for int32 ``ids`` [N].  ``serial``: the
    kernel starts only when everything before it on the stream has finished (for a step whose inputs a
    kernel has just written: the step's later kernels read them before they wait for anything)."""
    _need(table, None, "table", 2)
    _need(ids, torch.int32, "ids", 1)
    n, (v, h) = ids.shape[0], table.shape
    out = torch.empty((n, h), dtype=torch.float32, device=table.device)

    def launch():
        check(library().cw_embed(_ptr(out), _ptr(table), _ptr(ids), n, h, v, dtype_code(table.dtype), _ptr(status), _stream()), "embed")

    if serial:
        with serial_launch():
            launch()
    else:
        launch()
    return out


class PartialSums:
    """A product that was split over its inner dimension with the splits kept apart: ``slabs`` float32
    [splits, slab_rows, N], of which rows [0, rows) of every slab count; the product is their sum, taken
    in slab order by whoever adds it to the residual (``add_rmsnorm``, ``add_to_residual``)."""

    __slots__ = ("slabs", "rows")

    def __init__(self, slabs: torch.Tensor, rows: int) -> None:
        self.slabs, self.rows = slabs, rows


def _add_partial_sums(resid: torch.Tensor, parts: PartialSums, weight: torch.Tensor | None, eps: float,
                      out: torch.Tensor | None) -> None:
    _need(parts.slabs, torch.float32, "partial sums", 3)
    n, h = resid.shape
    splits, slab_rows, width = parts.slabs.shape
    if width != h or parts.rows != n or slab_rows < n:
        raise ValueError(f"partial sums {tuple(parts.slabs.shape)} of {parts.rows} rows do not match residual {tuple(resid.shape)}")
    check(library().cw_add_parts_rmsnorm(_ptr(resid), _ptr(parts.slabs), splits, slab_rows, _ptr(weight), _ptr(out), n, h,
                                         float(eps), 0 if out is None else dtype_code(out.dtype), _stream()), "add_parts_rmsnorm")


def add_rmsnorm(resid: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, status: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``resid += delta`` (if given: a tensor, or the ``PartialSums`` of a product), then returns
    ``weight * rmsnorm(resid)`` as ``out_dtype``."""
    _need(resid, torch.float32, "resid", 2)
    _need(weight, torch.float32, "weight", 1)
    n, h = resid.shape
    if weight.shape[0] != h:
        raise ValueError(f"norm weight has {weight.shape[0]} elements, rows have {h}")
    if isinstance(delta, PartialSums):
        if out is None:
            out = torch.empty((n, h), dtype=out_dtype, device=resid.device)
        _add_partial_sums(resid, delta, weight, eps, out)
        return out
    if delta is not None:
        _need(delta, out_dtype, "delta", 2)
        if delta.shape != resid.shape:
            raise ValueError(f"delta {tuple(delta.shape)} does not match residual {tuple(resid.shape)}")
    if out is None:
        out = torch.empty((n, h), dtype=out_dtype, device=resid.device)
    check(library().cw_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), None, n, n, h, float(eps),
                                   dtype_code(out_dtype), _ptr(status), _stream()), "add_rmsnorm")
    return out


def rmsnorm_rows(resid: torch.Tensor, rows: torch.Tensor, weight: torch.Tensor, eps: float,
                 out_dtype: torch.dtype, status: torch.Tensor) -> torch.Tensor:
    """``weight * rmsnorm(resid[rows])`` as ``out_dtype`` [R, H]."""
    _need(resid, torch.float32, "resid", 2)
    _need(rows, torch.int32, "rows", 1)
    _need(weight, torch.float32, "weight", 1)
    n, h = resid.shape
    r = rows.shape[0]
    out = torch.empty((r, h), dtype=out_dtype, device=resid.device)
    check(library().cw_add_rmsnorm(_ptr(resid), None, _ptr(weight), _ptr(out), _ptr(rows), r, n, h, float(eps),
                                   dtype_code(out_dtype), _ptr(status), _stream()), "rmsnorm_rows")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    _need(gate_up, None, "gate_up", 2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise ValueError("gate_up must have an even number of columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(library().cw_silu_mul(_ptr(gate_up), _ptr(out), n, two_i // 2, dtype_code(gate_up.dtype), _stream()), "silu_mul")
    return out


def add_to_residual(resid: torch.Tensor, delta) -> None:
    _need(resid, torch.float32, "resid", 2)
    if isinstance(delta, PartialSums):
        _add_partial_sums(resid, delta, None, 0.0, None)
        return
    _need(delta, None, "delta", 2)
    if delta.shape != resid.shape:
        raise ValueError("delta and residual shapes differ")
    n, h = resid.shape
    check(library().cw_add_to_residual(_ptr(resid), _ptr(delta), n, h, dtype_code(delta.dtype), _stream()), "add_to_residual")


EPILOGUE_STORE, EPILOGUE_ADD_F32, EPILOGUE_STORE_F32 = 0, 1, 2


def gemm_ref(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *,
             out: torch.Tensor | None = None, epilogue: int = EPILOGUE_STORE) -> torch.Tensor:
    """``a [M,K] @ w[N,K]^T (+ bias)`` on the CUDA cores with float32 accumulation.
    ``a`` may be a column slice of a wider matrix (row stride > K).  Epilogues: store in
    ``a``'s dtype; add into the float32 ``out``; store float32."""
    if not a.is_cuda or a.dim() != 2 or a.stride(1) != 1:
        raise ValueError("a must be a 2-d CUDA tensor with unit column stride")
    _need(w, a.dtype, "w", 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError(f"inner sizes differ: a has K={k}, w has K={w.shape[1]}")
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
        if bias.shape[0] != n:
            raise ValueError("bias length does not match w's rows")
    want = a.dtype if epilogue == EPILOGUE_STORE else torch.float32
    if out is None:
        if epilogue == EPILOGUE_ADD_F32:
            raise ValueError("the add epilogue needs an output to add into")
        out = torch.empty((m, n), dtype=want, device=a.device)
    _need(out, want, "out", 2)
    if tuple(out.shape) != (m, n):
        raise ValueError(f"out has shape {tuple(out.shape)}, expected {(m, n)}")
    lda = a.stride(0) if m > 1 else max(a.stride(0), k)
    check(library().cw_gemm_ref(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, lda, n, epilogue,
                                dtype_code(a.dtype), _stream()), "gemm_ref")
    return out


def gemm_ref_swiglu(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    _need(a, None, "a", 2)
    _need(w_gate, a.dtype, "w_gate", 2)
    _need(w_up, a.dtype, "w_up", 2)
    m, k = a.shape
    n = w_gate.shape[0]
    if w_gate.shape != w_up.shape or w_gate.shape[1] != k:
        raise ValueError("gate and up weights must both be [N, K] with a's K")
    out = torch.empty((m, n), dtype=a.dtype, device=a.device)
    check(library().cw_gemm_ref_swiglu(_ptr(a), _ptr(w_gate), _ptr(w_up), _ptr(out), m, n, k,
                                       dtype_code(a.dtype), _stream()), "gemm_ref_swiglu")
    return out


def rope_store(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor | None,
               inv_freq: torch.Tensor | None, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
               num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
               status: torch.Tensor, write_cache: bool = True) -> None:
    """Rotates q and k inside ``qkv`` [N, (nh+2nkv)*hd] in place and stores k, v at ``slots``
    of the caches ([pages, page_size, nkv, hd] each)."""
    _need(qkv, None, "qkv", 2)
    _need(positions, torch.int32, "positions", 1)
    n = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not match the head counts")
    num_slots = 0
    if write_cache:
        if k_cache is None or v_cache is None or slots is None:
            raise ValueError("writing the cache needs k_cache, v_cache and slots")
        _need(slots, torch.int32, "slots", 1)
        _need(k_cache, qkv.dtype, "k_cache", 4)
        _need(v_cache, qkv.dtype, "v_cache", 4)
        if tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) or k_cache.shape != v_cache.shape:
            raise ValueError("cache shape does not match the KV head count and head size")
        num_slots = k_cache.shape[0] * k_cache.shape[1]
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise ValueError("inv_freq must hold rotary_dim/2 frequencies")
    check(library().cw_rope_store(_ptr(qkv), _ptr(positions), _ptr(slots), _ptr(inv_freq), _ptr(k_cache), _ptr(v_cache),
                                  n, num_heads, num_kv_heads, head_dim, rotary_dim, num_slots,
                                  1 if write_cache else 0, dtype_code(qkv.dtype), _ptr(status), _stream()), "rope_store")


def copy_pages(cache: torch.Tensor, pairs: torch.Tensor, status: torch.Tensor) -> None:
    """``cache`` [planes, pages, ...]: copies page ``pairs[i,0]`` to ``pairs[i,1]`` in every plane."""
    _need(cache, None, "cache")
    _need(pairs, torch.int32, "pairs", 2)
    planes, pages = cache.shape[0], cache.shape[1]
    page_bytes = cache[0, 0].numel() * cache.element_size()
    check(library().cw_copy_pages(_ptr(cache), _ptr(pairs), pairs.shape[0], planes, pages, page_bytes,
                                  _ptr(status), _stream()), "copy_pages")


def attention_ref(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                  tok_seq: torch.Tensor, positions: torch.Tensor, num_heads: int, num_kv_heads: int,
                  head_dim: int, scale: float, window: int | None, status: torch.Tensor) -> torch.Tensor:
    """General paged causal attention.  ``q`` is [N, >= nh*hd] with unit column stride (the
    first nh*hd columns of each row are the query heads); returns [N, nh*hd]."""
    if not q.is_cuda or q.dim() != 2 or q.stride(1) != 1:
        raise ValueError("q must be a 2-d CUDA tensor with unit column stride")
    _need(k_cache, q.dtype, "k_cache", 4)
    _need(v_cache, q.dtype, "v_cache", 4)
    _need(block_tables, torch.int32, "block_tables", 2)
    _need(tok_seq, torch.int32, "tok_seq", 1)
    _need(positions, torch.int32, "positions", 1)
    n = q.shape[0]
    pages, page_size = k_cache.shape[0], k_cache.shape[1]
    if tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim):
        raise ValueError("cache shape does not match the KV head count and head size")
    if head_dim > 256:
        raise ValueError(f"head_dim {head_dim} is larger than the attention kernels take (256)")
    out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    check(library().cw_attention_ref(_ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
                                     _ptr(tok_seq), _ptr(positions), n, num_heads, num_kv_heads, head_dim, page_size,
                                     block_tables.shape[1], pages, float(scale), int(window or 0),
                                     dtype_code(q.dtype), _ptr(status), _stream()), "attention_ref")
    return out


REQUEST_STATE_FIELDS = ("position", "last_token", "draws", "seed_lo", "seed_hi", "temperature", "top_k", "top_p")


def _state_args(into_state) -> tuple:
    """``into_state`` = (row_slot int32 [R], state int32 [fields, slots]) or None."""
    if into_state is None:
        return None, None, 0
    row_slot, state = into_state
    _need(row_slot, torch.int32, "row_slot", 1)
    _need(state, torch.int32, "state", 2)
    if state.shape[0] != len(REQUEST_STATE_FIELDS):
        raise ValueError(f"the request-state table has {len(REQUEST_STATE_FIELDS)} fields, got {state.shape[0]} rows")
    return _ptr(row_slot), _ptr(state), state.shape[1]


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None, into_state=None) -> torch.Tensor:
    """First maximal index per row.  ``into_state`` = (row_slot, state table): the token also becomes the
    request's last token in the table and its position and draw counter advance (``step_from_state``)."""
    _need(logits, torch.float32, "logits", 2)
    r, v = logits.shape
    if out is None:
        out = torch.empty((r,), dtype=torch.int32, device=logits.device)
    slot_ptr, state_ptr, slots = _state_args(into_state)
    if into_state is not None and into_state[0].shape[0] < r:
        raise ValueError("row_slot must have an entry per logits row")
    check(library().cw_argmax_state(_ptr(logits), _ptr(out), r, v, v, slot_ptr, state_ptr, slots, _stream()), "argmax")
    return out


def step_from_state(row_slot: torch.Tensor, fresh: torch.Tensor, fresh_values: torch.Tensor, state: torch.Tensor,
                    tables: list[torch.Tensor], kv_slots: list[torch.Tensor], page_size: int, num_pages: int,
                    tokens: torch.Tensor, positions: torch.Tensor, ctx_lens: torch.Tensor, tok_seq: torch.Tensor,
                    temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor, uniform: torch.Tensor,
                    status: torch.Tensor) -> None:
    """The inputs of a single-token step from the per-request state table: row r of the step belongs to
    the request in slot ``row_slot[r]`` (< 0: padding).  Rows flagged in ``fresh`` first take their column
    from ``fresh_values`` [fields, B] (the flag is cleared).  Written: the token to feed, position,
    context length, the row's request index, the cache slot per page group (from ``tables`` [B, max_blocks]
    each), and the sampling parameters with the draw's uniform number."""
    import ctypes

    b = row_slot.shape[0]
    for name, t in (("row_slot", row_slot), ("fresh", fresh), ("tokens", tokens), ("positions", positions),
                    ("ctx_lens", ctx_lens), ("tok_seq", tok_seq), ("top_k", top_k)):
        _need(t, torch.int32, name, 1)
    for name, t in (("temperature", temperature), ("top_p", top_p), ("uniform", uniform)):
        _need(t, torch.float32, name, 1)
    _need(fresh_values, torch.int32, "fresh_values", 2)
    _need(state, torch.int32, "state", 2)
    if state.shape[0] != len(REQUEST_STATE_FIELDS) or tuple(fresh_values.shape) != (len(REQUEST_STATE_FIELDS), b):
        raise ValueError("state must be [fields, slots] and fresh_values [fields, B]")
    if len(tables) != len(kv_slots):
        raise ValueError("one block table and one slot array per page group")
    max_blocks = 1
    for t, k in zip(tables, kv_slots):
        _need(t, torch.int32, "tables", 2)
        _need(k, torch.int32, "kv_slots", 1)
        max_blocks = t.shape[1]
    g = len(tables)
    table_ptrs = (ctypes.c_void_p * max(g, 1))(*[t.data_ptr() for t in tables])
    slot_ptrs = (ctypes.c_void_p * max(g, 1))(*[k.data_ptr() for k in kv_slots])
    check(library().cw_step_from_state(
        _ptr(row_slot), _ptr(fresh), _ptr(fresh_values), _ptr(state), state.shape[1], b, int(page_size), int(max_blocks),
        int(num_pages), g, ctypes.cast(table_ptrs, ctypes.c_void_p), ctypes.cast(slot_ptrs, ctypes.c_void_p), _ptr(tokens),
        _ptr(positions), _ptr(ctx_lens), _ptr(tok_seq), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
        _ptr(status), _stream()), "step_from_state")


_sample_work: dict[int, torch.Tensor] = {}
_sample_work_retired: list[torch.Tensor] = []  # outgrown workspaces: captured graphs may still point at them


def _sample_workspace(device: torch.device, rows: int) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    fn = library().cw_sample_workspace_words
    fn.restype = ctypes.c_longlong
    words = int(fn(rows))
    work = _sample_work.get(index)
    if work is None or work.numel() < words:
        if work is not None:
            _sample_work_retired.append(work)
        work = _sample_work[index] = torch.zeros(max(words, int(fn(8))), dtype=torch.int64, device=device)
    return work


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor | None = None, into_state=None, one_block: bool = False) -> torch.Tensor:
    """One token per row; rows with temperature 0 are greedy.  ``into_state``: as for ``argmax``.
    ``one_block``: the kernel that walks a row with a single thread block (the same rule, much slower for a
    large vocabulary; kept for comparison) instead of the chain of kernels over many blocks per row."""
    _need(logits, torch.float32, "logits", 2)
    r, v = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("uniform", uniform, torch.float32)):
        _need(t, dt, name, 1)
        if t.shape[0] != r:
            raise ValueError(f"{name} must have one entry per row")
    if out is None:
        out = torch.empty((r,), dtype=torch.int32, device=logits.device)
    slot_ptr, state_ptr, slots = _state_args(into_state)
    if one_block:
        check(library().cw_sample_state(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform), _ptr(out),
                                        r, v, v, slot_ptr, state_ptr, slots, _stream()), "sample")
        return out
    work = _sample_workspace(logits.device, r)
    check(library().cw_sample_rows(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform), _ptr(out),
                                   r, v, v, slot_ptr, state_ptr, slots, _ptr(work), _stream()), "sample_rows")
    return out
