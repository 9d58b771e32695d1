"""Loads the kernel library (building it at first use) and declares its C entry points."""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

P, I, F, LL = c_void_p, c_int, c_float, c_longlong

# name -> argument types (the stream is the last c_void_p of each)
_SIGNATURES: dict[str, list] = {
    "cw_embed": [P, P, P, I, I, I, I, P, P],
    "cw_add_rmsnorm": [P, P, P, P, P, I, I, I, F, I, P, P],
    "cw_silu_mul": [P, P, I, I, I, P],
    "cw_add_to_residual": [P, P, I, I, I, P],
    "cw_add_parts_rmsnorm": [P, P, I, I, P, P, I, I, F, I, P],
    "cw_gemm_ref": [P, P, P, P, I, I, I, I, I, I, I, P],
    "cw_gemm_ref_swiglu": [P, P, P, P, I, I, I, I, P],
    "cw_rope_store": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P],
    "cw_copy_pages": [P, P, I, I, I, LL, P, P],
    "cw_attention_ref": [P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P],
    "cw_argmax": [P, P, I, I, LL, P],
    "cw_sample": [P, P, P, P, P, P, I, I, LL, P],
    "cw_argmax_state": [P, P, I, I, LL, P, P, I, P],
    "cw_sample_state": [P, P, P, P, P, P, I, I, LL, P, P, I, P],
    "cw_sample_rows": [P, P, P, P, P, P, I, I, LL, P, P, I, P, P],
    "cw_sample_workspace_words": [I],
    "cw_step_from_state": [P, P, P, P, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P, P, P, P],
}
_OPTIONAL: dict[str, list] = {}


class KernelLibraryError(RuntimeError):
    pass


def register_optional(name: str, argtypes: list) -> None:
    _OPTIONAL[name] = argtypes


def library() -> ctypes.CDLL:
    """The loaded library.  Raises ``KernelLibraryError`` when it cannot be built or loaded:
    there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc.build import ensure_built

        try:
            path = ensure_built()
            lib = ctypes.CDLL(str(path))
        except Exception as exc:  # noqa: BLE001
            raise KernelLibraryError(
                f"the clockwork_b200 CUDA kernels are unavailable ({exc}); "
                "they are required: there is no CPU or library fallback"
            ) from exc
        for name, argtypes in {**_SIGNATURES, **_OPTIONAL}.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                if name in _OPTIONAL:
                    continue
                raise KernelLibraryError(f"{path} does not export {name}") from None
            fn.argtypes = argtypes
            fn.restype = c_int
        _lib = lib
        return lib


ERROR_NAMES = {-1: "refused size", -2: "unknown dtype code", -3: "unsupported combination", -4: "set-up failed",
               -5: "needs more scratch than the built-in maximum"}


_launches = 0
_pdl_on = True


def set_pdl(on: bool) -> None:
    """Whether kernels are launched so that each may begin while its predecessor drains (programmatic
    dependent launch; the default) or strictly one after the other."""
    global _pdl_on
    library().cw_set_pdl(1 if on else 0)
    _pdl_on = bool(on)


class serial_launch:
    """Launches inside this block start only after everything before them on the stream has finished."""

    def __enter__(self):
        self.was = _pdl_on
        if self.was:
            set_pdl(False)

    def __exit__(self, *exc):
        if self.was:
            set_pdl(True)



def launch_count() -> int:
    """Kernel launches made through this library so far (each entry point launches one kernel)."""
    return _launches


def check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code == 0:
        return
    if code < 0:
        raise ValueError(f"{what}: kernel refused the call ({ERROR_NAMES.get(code, code)})")
    raise RuntimeError(f"{what}: CUDA error {code} at launch")
