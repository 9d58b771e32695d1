"""The decode-attention entry point that allocates nothing (``cw_attention_decode_noalloc``, declared
in ``clockwork_b200/csrc/clockwork_b200.h``), called the way a host without an allocator calls it:
through the library's exported C symbol, with raw device pointers.

Some hosts of these kernels cannot call cudaMalloc while they run: a C serving loop with a fixed
device-memory budget, or code at a point where an allocation would synchronise the device.  For them
the library carries a fixed scratch array of its own; this test checks that the variant gives what
the regular entry point (whose caller allocates the scratch) gives, on two calls in a row, the
second with other inputs and sizes so that anything the first call left in the shared scratch would
show, and that a call too large for the built-in scratch is refused.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
    from clockwork_b200.ops.library import library

    handle = library()
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = handle.cw_attention_decode_noalloc
    fn.argtypes = [P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P]
    fn.restype = ctypes.c_int
    handle.cw_error_string.argtypes = [ctypes.c_int]
    handle.cw_error_string.restype = ctypes.c_char_p
    return handle


def case(num_seqs, nh, nkv, hd, page_size, ctx_lens, seed):
    g = torch.Generator().manual_seed(seed)
    blocks = max((c + page_size - 1) // page_size for c in ctx_lens) + 1
    pages = num_seqs * blocks + 3
    order = torch.randperm(pages, generator=g)[: num_seqs * blocks].to(torch.int32)
    tables = order.view(num_seqs, blocks).contiguous()
    k_cache = torch.randn(pages, page_size, nkv, hd, generator=g).bfloat16()
    v_cache = torch.randn(pages, page_size, nkv, hd, generator=g).bfloat16()
    q = (torch.randn(num_seqs, (nh + 2 * nkv) * hd, generator=g) * 2).bfloat16()
    return dict(q=q.to(DEV), k=k_cache.to(DEV), v=v_cache.to(DEV), tables=tables.to(DEV),
                ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh=nh, nkv=nkv, hd=hd,
                scale=hd**-0.5, max_ctx=max(ctx_lens))


def run_both(lib, c, split, window=0, stream=None):
    from clockwork_b200 import ops
    from clockwork_b200.ops import attention_fast

    status = ops.new_status(DEV)
    want = attention_fast.attention_decode(c["q"], c["k"], c["v"], c["tables"], c["ctx"], c["nh"], c["nkv"], c["hd"],
                                           c["scale"], window or None, c["max_ctx"], status, split=split)
    got = torch.full_like(want, float("nan"))
    torch.cuda.synchronize()
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.cw_attention_decode_noalloc(
        c["q"].data_ptr(), c["q"].stride(0), got.data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(),
        c["tables"].data_ptr(), c["ctx"].data_ptr(), c["q"].shape[0], c["nh"], c["nkv"], c["hd"], c["k"].shape[1],
        c["tables"].shape[1], c["k"].shape[0], c["scale"], window, c["max_ctx"], split, status.data_ptr(), handle)
    assert rc == 0, lib.cw_error_string(rc).decode()
    torch.cuda.synchronize()
    # free device memory as the driver counts it: an allocation inside the library would show here
    # (torch's own counters cannot see one); nothing else ran between the two readings
    assert torch.cuda.mem_get_info()[0] >= free_before
    ops.raise_on_status(status)
    return got, want


def plain_attention(c, window=0):
    """What ``tests/plain`` computes for the same inputs: per request, its one query over the keys and
    values gathered from its pages (whole sequences, no cache logic shared with the kernels)."""
    from tests.plain.qwen2_plain import causal_attention

    nh, nkv, hd = c["nh"], c["nkv"], c["hd"]
    k_cache, v_cache, tables = c["k"].float().cpu(), c["v"].float().cpu(), c["tables"].cpu()
    page = k_cache.shape[1]
    rows = []
    for s, n in enumerate(c["ctx"].tolist()):
        pages = tables[s, : (n + page - 1) // page].long()
        k = k_cache[pages].reshape(-1, nkv, hd)[:n]
        v = v_cache[pages].reshape(-1, nkv, hd)[:n]
        q = c["q"][s, : nh * hd].float().cpu().view(1, nh, hd)
        rows.append(causal_attention(q, k, v, c["scale"], window=window or None).reshape(nh * hd))
    return torch.stack(rows)


def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row(lib):
    # contexts long enough to be split over several thread blocks, so the scratch is really used
    first = case(5, 12, 2, 128, 16, [700, 1300, 257, 64, 1025], seed=1)
    second = case(3, 8, 1, 64, 8, [900, 300, 2000], seed=2)
    run_both(lib, first, split=256)  # the first call on a device looks the scratch's address up: not counted below
    for c, window in ((first, 0), (second, 0), (first, 200)):
        got, want = run_both(lib, c, split=256, window=window)
        # the tolerance of the other bfloat16 attention tests; the two run the same kernel
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want)
        torch.testing.assert_close(got.float().cpu(), plain_attention(c, window), rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_on_another_stream_after_a_sync(lib):
    """Calls share the one scratch array, so they are serialised: here by a synchronize between a call
    on the current stream and one on a second stream."""
    c = case(4, 12, 2, 128, 16, [1500, 129, 640, 2], seed=4)
    run_both(lib, c, split=128)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    got, want = run_both(lib, c, split=128, stream=side)
    assert torch.equal(got, want)
    torch.testing.assert_close(got.float().cpu(), plain_attention(c), rtol=2e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit(lib):
    c = case(2, 12, 2, 128, 16, [300, 400], seed=3)
    out = torch.zeros(2, 12 * 128, dtype=torch.bfloat16, device=DEV)
    # 4096 requests of 32 heads with contexts bounded by 65536 tokens would need gigabytes of scratch
    rc = lib.cw_attention_decode_noalloc(
        c["q"].data_ptr(), c["q"].stride(0), out.data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["tables"].data_ptr(),
        c["ctx"].data_ptr(), 4096, 32, 8, 128, 16, c["tables"].shape[1], c["k"].shape[0], c["scale"], 0, 65536, 256, None,
        torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    assert b"more scratch" in lib.cw_error_string(rc)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0  # nothing was launched
    # the query that answers without a call agrees, at the sizes the header names and one page beyond
    fits = lib.cw_attention_decode_noalloc_fits
    fits.argtypes = [ctypes.c_int] * 5
    fits.restype = ctypes.c_int
    assert fits(4096, 32, 8, 128, 65536) == 0
    assert fits(8, 12, 2, 128, 21632) == 1 and fits(8, 12, 2, 128, 21633) == 0
    assert fits(64, 12, 2, 128, 2688) == 1 and fits(64, 12, 2, 128, 2689) == 0
    assert fits(2, 12, 5, 128, 100) == -1  # heads that do not divide
