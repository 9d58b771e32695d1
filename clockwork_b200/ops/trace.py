"""Step timeline: device-side records of when each CTA of a kernel started, when its waits on the
preceding kernel returned (the first and the last: in the matrix-product kernel the last is the
epilogue's, taken when the accumulator is ready), and when it finished.  Kernels that end with
``cw_trace_end()`` take part: the decode-size matrix product and decode attention.

    from clockwork_b200.ops import trace
    trace.enable()
    ... run a step ...
    launches = trace.collect()     # one dict per kernel launch, in time order
    trace.disable()

Times are nanoseconds of the GPU's global timer, relative to the earliest record.  Kernels record only
while a buffer is set; otherwise the cost is one constant load per CTA."""

from __future__ import annotations

import torch

from .library import check, library

_TUS = ("attention_decode", "attention_decode_large", "attention_decode_mid", "attention_prefill", "attention_prefill_tc", "attention_ref", "embed_norm", "gemm_ref",
        "gemm_tc", "rope_cache", "sampling")
_WORDS = 8
_buf: torch.Tensor | None = None


def _set(ptr) -> None:
    from ctypes import c_int, c_void_p

    lib = library()
    for tu in _TUS:
        fn = getattr(lib, f"cw_trace_set_{tu}")
        fn.argtypes, fn.restype = [c_void_p], c_int
        check(fn(ptr), f"trace_set_{tu}")


def enable(capacity: int = 1 << 16, device="cuda:0") -> None:
    global _buf
    torch.cuda.synchronize()
    _buf = torch.zeros(_WORDS * (1 + capacity), dtype=torch.int64, device=device)
    _buf[1] = capacity
    _set(_buf.data_ptr())


def disable() -> None:
    global _buf
    torch.cuda.synchronize()
    _set(None)
    _buf = None


def reset() -> None:
    torch.cuda.synchronize()
    _buf[0] = 0


def records() -> torch.Tensor:
    """[n, 8] int64: start, first release, last release, end (ns), gridDim packed (20 bits each), blockIdx packed,
    the SM the CTA ran on."""
    torch.cuda.synchronize()
    n = min(int(_buf[0]), int(_buf[1]))
    return _buf[_WORDS : _WORDS * (1 + n)].view(n, _WORDS).cpu()


def collect() -> list[dict]:
    """Records grouped into launches (one grid shape, no CTA index twice), ordered by first release."""
    rec = records()
    if rec.numel() == 0:
        return []
    t0 = int(rec[:, 0].min())
    rows = sorted(rec.tolist(), key=lambda r: r[0])
    launches: list[dict] = []
    open_by_grid: dict[int, dict] = {}
    for start, rel0, rel1, end, g, b, *_ in rows:
        cur = open_by_grid.get(g)
        if cur is None or b in cur["_seen"]:
            grid = (g & 0xFFFFF, (g >> 20) & 0xFFFFF, (g >> 40) & 0xFFFFF)
            cur = {"grid": grid, "_seen": set(), "start": [], "released": [], "ready": [], "end": []}
            open_by_grid[g] = cur
            launches.append(cur)
        cur["_seen"].add(b)
        cur["start"].append(start - t0)
        if rel0:
            cur["released"].append(rel0 - t0)
            cur["ready"].append(rel1 - t0)
        cur["end"].append(end - t0)
    out = []
    for l in launches:
        d = {"grid": l["grid"], "ctas": len(l["start"])}
        for key in ("start", "released", "ready", "end"):
            if l[key]:
                d[f"{key}_first"], d[f"{key}_last"] = min(l[key]), max(l[key])
        out.append(d)
    out.sort(key=lambda d: d.get("released_first", d["start_first"]))
    return out
