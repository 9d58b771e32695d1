"""How a product of a few hundred tokens is cut over its inner dimension when its splits are kept apart for
the next norm to add up (``cw_gemm_tc_parts_plan``, host code of the kernel library, no GPU): splits cut the
inner dimension into equal runs of whole 64-element blocks, never shorter than eight blocks, at most eight
of them, and only for token counts that the CTA-pair kernel takes this way."""

import ctypes
import random
import shutil

import pytest

from clockwork_b200.ops.library import library


def plan(t, n, k, sms=148):
    try:
        lib = library()  # (built at first use; the plan is host code and needs no GPU)
    except Exception as err:  # noqa: BLE001
        if shutil.which("nvcc") is None:
            pytest.skip(f"the kernel library is not built and there is no nvcc here: {err}")
        raise
    lib.cw_gemm_tc_parts_plan.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)]
    lib.cw_gemm_tc_parts_plan.restype = ctypes.c_int
    splits = ctypes.c_int(-1)
    assert lib.cw_gemm_tc_parts_plan(t, n, k, sms, ctypes.byref(splits)) == 0
    return splits.value


def test_splits_are_equal_runs_of_whole_blocks():
    rng = random.Random(3)
    seen = set()
    for _ in range(2000):
        t = rng.choice([129, 130, 192, 256, 257, 300, 512, 700, 1000, 1024])
        n = rng.choice([256, 1536, 2048, 3584, 5120, 1000, 130 * 4])
        k = rng.choice([512, 1536, 8960, 18944, 27648, 3584, 5120, 200, 264, 72 * 8])
        splits = plan(t, n, k)
        blocks = -(-k // 64)
        assert 1 <= splits <= 8 and blocks % splits == 0 and (splits == 1 or blocks // splits >= 8), (t, n, k, splits)
        seen.add(splits)
    assert len(seen) > 2  # (the sizes above do get cut in several ways)
    assert plan(256, 1536, 8960) > 1  # the down projection of the 1.5B layer at a few hundred tokens


def test_other_token_counts_are_not_cut():
    for t in (1, 8, 64, 128, 1025, 2048, 4096):
        assert plan(t, 1536, 8960) == 1
    assert plan(256, 1536, 8960, sms=1) == 1
