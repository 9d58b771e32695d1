"""Python faces of the bfloat16 attention kernels: split-context decode (``csrc/attention_decode_kernel.cuh``, entry points in ``csrc/attention_decode.cu``)
and prefill on the tensor cores (``csrc/attention_prefill_tc.cu``: tcgen05, head sizes 64 and 128;
``csrc/attention_prefill.cu``: mma.sync, the other sizes).  ``ops.attention.paged_attention`` picks
them when a step's sizes allow."""

from __future__ import annotations

import sys
from ctypes import POINTER, byref, c_float, c_int, c_longlong, c_void_p

import numpy as np
import torch

from . import _need, _ptr, _stream, attention as dispatch
from .library import check, library

DECODE_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256)
PREFILL_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
PREFILL_TC_HEAD_DIMS = (64, 128)  # the tcgen05 kernel; pages of 8..128 tokens, a power of two
QUERY_TILE = 128


def prefill_tc_takes(head_dim: int, page_size: int) -> bool:
    return head_dim in PREFILL_TC_HEAD_DIMS and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0

_configured = False
_scratch: dict[int, dict] = {}


def _configure() -> None:
    global _configured
    if _configured:
        return
    lib = library()
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    lib.cw_attention_decode.argtypes = [P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P, P, P, P, P]
    lib.cw_attention_decode.restype = c_int
    lib.cw_attention_decode_fused.argtypes = [P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P, P, P, I, P, I, P, I, P, P]
    lib.cw_attention_decode_fused.restype = c_int
    lib.cw_attention_decode_rows.argtypes = [P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P, P, P, I, P, I, P, I, P, P]
    lib.cw_attention_decode_rows.restype = c_int
    lib.cw_attention_decode_workspace.argtypes = [I, I, I, I, I, POINTER(LL), POINTER(LL), POINTER(I)]
    lib.cw_attention_decode_workspace.restype = c_int
    lib.cw_attention_prefill.argtypes = [P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
    lib.cw_attention_prefill.restype = c_int
    lib.cw_attention_prefill_tc.argtypes = [P, I, I, I, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
    lib.cw_attention_prefill_tc.restype = c_int
    _configured = True


_retired_scratch: list[dict] = []  # superseded sets: captured graphs may still point at them


def _decode_scratch(device: torch.device, part_o: int, part_lse: int, counters: int) -> dict:
    """The split-merge scratch of the decode kernel (float32 partial outputs and log-sum-exps, arrival
    counters that are zero between launches), one set per device, replaced by a larger one when a call
    needs more.  A set that was ever handed out is never freed: a captured CUDA graph has its addresses
    baked in, and memory given back to the allocator would be handed to other tensors under it."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    st = _scratch.get(index)
    if st is None or st["part_o"].numel() < part_o or st["part_lse"].numel() < part_lse or st["counters"].numel() < counters:
        if st is not None:
            _retired_scratch.append(st)
        st = {
            "part_o": torch.empty(max(part_o, 1 << 20), dtype=torch.float32, device=device),
            "part_lse": torch.empty(max(part_lse, 1 << 14), dtype=torch.float32, device=device),
            "counters": torch.zeros(max(counters, 1 << 12), dtype=torch.int32, device=device),
        }
        _scratch[index] = st
    return st


def reserve_decode_scratch(device, max_seqs: int, num_heads: int, num_kv_heads: int, head_dim: int, max_ctx: int) -> None:
    """Size the device's scratch once for the largest decode step that will run (called before steps
    are captured), so that captured graphs share one set."""
    _configure()
    device = torch.device(device)
    po, pl, pc = c_longlong(0), c_longlong(0), c_int(0)
    library().cw_attention_decode_workspace(int(max_seqs), num_heads, num_kv_heads, head_dim, int(max_ctx),
                                            byref(po), byref(pl), byref(pc))
    _decode_scratch(device, po.value, pl.value, pc.value)


MIN_SPLIT = 128
SWIZZLED = 0x100  # flag in the `stages` argument of the decode kernel
TMA_TILES = 0x200  # flag in the same argument: K/V tiles by TMA, one copy per page and operand
_SMS: dict[int, int] = {}


def _pairs(num_seqs: int, num_heads: int, num_kv_heads: int) -> int:
    groups = -(-(num_heads // num_kv_heads) // 16)
    return max(1, num_seqs * num_kv_heads * groups)


def _sm_count(device=None) -> int:
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    sms = _SMS.get(index)
    if sms is None:
        sms = _SMS[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return sms


def _resident_ctas(head_dim: int, stages: int = 2, swizzled: bool = True) -> int:
    """CTAs of the decode kernel that one SM holds: shared memory (q tile, `stages` K and V tiles of
    64 tokens, unpadded when the head size is a multiple of 64, and about 4 KB besides), at most
    three by registers."""
    ldk = head_dim if head_dim % 64 == 0 and swizzled else head_dim + 8
    smem = (16 * (head_dim + 8) + 2 * stages * 64 * ldk) * 2 + 4096
    return max(1, min(3, (227 * 1024) // smem))


def _unpadded(head_dim: int, pairs: int) -> bool:
    """Whether a step that cuts contexts into more than two tiles per CTA runs on unpadded K/V tiles
    (swizzled or by TMA: head sizes of 64n), which lets a third CTA share the SM."""
    return head_dim % 64 == 0 and (pairs > 16 or _tma_tiles)


def _splits_wanted(num_seqs: int, num_heads: int, num_kv_heads: int, device=None, head_dim: int = 128) -> int:
    """Context splits per request that fill the SMs once with resident CTAs of the two-tile variant:
    a CTA that has to wait for a slot starts a whole CTA-time late."""
    pairs = _pairs(num_seqs, num_heads, num_kv_heads)
    return max(1, _resident_ctas(head_dim, swizzled=_unpadded(head_dim, pairs)) * _sm_count(device) // pairs)


def decode_split(num_seqs: int, num_heads: int, num_kv_heads: int, max_live_ctx: int, device=None,
                 head_dim: int = 128) -> int:
    """Tokens per CTA for a decode step: cut contexts so that all CTAs are resident at once, never
    finer than 128 tokens.  The result depends on the number of live requests and their longest
    context only."""
    split = -(-max(1, max_live_ctx) // _splits_wanted(num_seqs, num_heads, num_kv_heads, device, head_dim))
    return max(MIN_SPLIT, -(-split // 64) * 64)


def decode_split_bound(max_seqs: int, num_heads: int, num_kv_heads: int, max_ctx: int, device=None, head_dim: int = 128) -> int:
    """The largest ``decode_split`` of any step of up to ``max_seqs`` requests with contexts up to ``max_ctx``."""
    return max(decode_split(n, num_heads, num_kv_heads, max_ctx, device, head_dim) for n in range(1, max_seqs + 1))


def decode_stages(num_seqs: int, num_heads: int, num_kv_heads: int, max_ctx: int | None = None, device=None,
                  head_dim: int = 128) -> int:
    """The decode kernel's variant for a step: tiles of 64 tokens in flight per CTA, with flags for the
    layout of the tiles and the way they are fetched.  Whatever is chosen leaves as many CTAs resident
    per SM as ``decode_split`` counts on, so that all CTAs of a step run at once.

    * Many CTAs (from 16 requests of two KV heads on): two tiles in flight, unpadded tiles (swizzled,
      and fetched by TMA where the sizes allow it), three CTAs per SM at head size 128.
    * Few CTAs and contexts up to ``max_ctx`` that fit as CTAs of 128 tokens: two padded tiles filled by
      ``cp.async`` hold a whole split, with the shortest way from the CTA's start to its first product.
    * Few CTAs and longer contexts: a CTA walks several tiles; by TMA with two in flight and three CTAs
      per SM, or, for head sizes without that variant, four padded tiles in flight where they leave as
      many CTAs per SM as two would."""
    pairs = _pairs(num_seqs, num_heads, num_kv_heads)
    unpadded = 2 | SWIZZLED | (TMA_TILES if _tma_tiles else 0)
    if pairs > 16:
        return unpadded if head_dim % 64 == 0 else 2
    if max_ctx is not None and -(-max_ctx // MIN_SPLIT) * pairs <= _resident_ctas(head_dim, swizzled=False) * _sm_count(device):
        return 2
    if _unpadded(head_dim, pairs):
        return unpadded
    return 4 if _resident_ctas(head_dim, 4, False) >= _resident_ctas(head_dim, 2, False) else 2


_tma_tiles = True


def set_tma_tiles(on: bool) -> None:
    """Whether the decode kernel fetches K/V tiles by TMA (one copy per page and operand, counted by an
    mbarrier) where head and page sizes allow it, or by 16-byte ``cp.async`` as everywhere else."""
    global _tma_tiles
    _tma_tiles = bool(on)


_cluster_merge = False


def set_cluster_merge(on: bool) -> None:
    """Whether the context splits of a group meet through a thread-block cluster (slices pushed into each
    other's shared memory) instead of the global workspace.  Off by default: measured slower inside the
    step (batch 8: 1.66 against 1.29 ms; batch 64: 2.77 against 2.04 ms), because a cluster's CTAs start
    only when all of them find room at once, which ends the overlap of the kernel's long prologue with the
    product before it."""
    global _cluster_merge
    _cluster_merge = bool(on)


def decode_cluster(num_seqs: int, num_heads: int, num_kv_heads: int, max_ctx: int, device=None, head_dim: int = 128) -> int:
    """CTAs per thread-block cluster through which the context splits of a (request, KV head) group
    meet: as many as fill the SMs once with resident CTAs and as contexts up to ``max_ctx`` can use at
    128 tokens each, a power of two, 16 at most; 0: a single split, or a head size whose tiles leave
    no room (the splits then meet through the global workspace)."""
    if head_dim > 128 or not _cluster_merge:
        return 0
    want = min(16, -(-max_ctx // MIN_SPLIT), _splits_wanted(num_seqs, num_heads, num_kv_heads, device, head_dim))
    size = 1
    while size < want:
        size *= 2
    return size if size > 1 else 0


CLUSTER_SHIFT = 16  # the cluster size rides in these bits of the decode kernel's `stages` argument


class _Decode:
    @staticmethod
    def accepts(ctx, view, num_heads, num_kv_heads, head_dim, window) -> bool:
        return head_dim in DECODE_HEAD_DIMS and ctx.num_tokens == ctx.num_seqs

    @staticmethod
    def run(ctx, qkv, view, num_heads, num_kv_heads, head_dim, scale, window, max_ctx: int | None = None,
            fused_position=None) -> torch.Tensor:
        # a device scalar that a captured step refreshes before every replay, when there is one
        split_dev = ctx.extras.get(dispatch.decode_split_name(num_heads, num_kv_heads, head_dim))
        # (with the device scalar: the largest value it can take for up to this many requests and this context bound)
        split = (decode_split_bound if split_dev is not None else decode_split)(
            ctx.num_seqs, num_heads, num_kv_heads, max_ctx or ctx.max_ctx_len, qkv.device, head_dim)
        return attention_decode(qkv, view.k_cache, view.v_cache, view.block_tables, ctx.ctx_lens, num_heads,
                                num_kv_heads, head_dim, scale, window, max_ctx or ctx.max_ctx_len, ctx.status,
                                split=split, split_dev=split_dev,
                                fused=None if fused_position is None else (*fused_position, view.slots),
                                stages=decode_stages(ctx.num_seqs, num_heads, num_kv_heads, max_ctx or ctx.max_ctx_len, qkv.device, head_dim)
                                | decode_cluster(ctx.num_seqs, num_heads, num_kv_heads, max_ctx or ctx.max_ctx_len, qkv.device, head_dim) << CLUSTER_SHIFT)


def attention_decode(q, k_cache, v_cache, block_tables, ctx_lens, num_heads, num_kv_heads, head_dim, scale, window,
                     max_ctx: int, status, split: int | None = None, split_dev: torch.Tensor | None = None,
                     fused: tuple | None = None, stages: int = 0, q_start: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """One query token per request: ``q`` [S, >= nh*hd] (row s belongs to request s), ``ctx_lens`` [S]
    the tokens of each request in the cache (its own included).  ``split``: tokens per CTA (a multiple
    of 64, at least 128; default: chosen by ``decode_split``), or ``split_dev``, the same as an int32
    device scalar (``split`` is then an upper bound on it, or None: the whole context).  ``fused``: (inv_freq or None, rotary_dim, slots): ``q`` is then the raw [q | k | v]
    rows; q and the new k are rotated inside the kernel and the new token's k and v stored at ``slots``
    (so no separate position-encoding / cache-write kernel is needed).  Returns [S, nh*hd].

    ``q_start`` (int32 [S + 1]) with ``out`` ([N, nh*hd]): the requests are those of a flat batch of N rows
    that also holds prompt portions; request s owns rows q_start[s]:q_start[s+1] of ``q`` and ``out``, and
    only the requests with exactly one row are served (rows of the others are left alone)."""
    _configure()
    if q.dtype != torch.bfloat16 or q.dim() != 2 or q.stride(1) != 1:
        raise ValueError("q must be a 2-d bfloat16 tensor with unit column stride")
    _need(k_cache, torch.bfloat16, "k_cache", 4)
    _need(v_cache, torch.bfloat16, "v_cache", 4)
    _need(block_tables, torch.int32, "block_tables", 2)
    _need(ctx_lens, torch.int32, "ctx_lens", 1)
    if head_dim not in DECODE_HEAD_DIMS:
        raise ValueError(f"head_dim {head_dim} is not one of {DECODE_HEAD_DIMS}")
    s = q.shape[0]
    if q_start is not None:
        _need(q_start, torch.int32, "q_start", 1)
        s = q_start.shape[0] - 1
        if out is None or fused is not None:
            raise ValueError("a flat batch needs the output tensor and runs without the fused position encoding")
    if split_dev is None and split is None:
        split = decode_split(s, num_heads, num_kv_heads, max_ctx, q.device, head_dim)
    po, pl, pc = c_longlong(0), c_longlong(0), c_int(0)
    library().cw_attention_decode_workspace(s, num_heads, num_kv_heads, head_dim, max_ctx, byref(po), byref(pl), byref(pc))
    st = _decode_scratch(q.device, po.value, pl.value, pc.value)
    if out is None:
        out = torch.empty((s, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    elif out.dtype != torch.bfloat16 or out.shape[1] != num_heads * head_dim or not out.is_contiguous():
        raise ValueError("out must be a contiguous bfloat16 [rows, nh*hd] tensor")
    inv_freq, rotary_dim, slots = fused if fused is not None else (None, 0, None)
    if fused is not None:
        if q.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise ValueError("the fused form needs the whole [q | k | v] rows")
        _need(slots, torch.int32, "slots", 1)
        if inv_freq is not None:
            _need(inv_freq, torch.float32, "inv_freq", 1)
            if inv_freq.shape[0] * 2 != rotary_dim:
                raise ValueError("inv_freq must hold rotary_dim/2 frequencies")
    check(library().cw_attention_decode_rows(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(ctx_lens), _ptr(q_start), s, num_heads,
        num_kv_heads, head_dim, k_cache.shape[1], block_tables.shape[1], k_cache.shape[0], float(scale), int(window or 0),
        int(max_ctx), int(split or 0), _ptr(split_dev), _ptr(st["part_o"]), _ptr(st["part_lse"]), _ptr(st["counters"]),
        1 if fused is not None else 0, _ptr(inv_freq), int(rotary_dim), _ptr(slots), int(stages), _ptr(status), _stream()), "attention_decode")
    return out


MIN_PART_KEYS = 4 * QUERY_TILE  # no part of a cut row of keys is shorter than this (a cut costs about three tiles' time)
MAX_PARTS = 8                   # (the kernel's limit)


def prefill_work_items(q_lens, ctx_lens, num_heads: int = 0, sm_count: int = 0,
                       skip_single: bool = False, max_items: int | None = None) -> tuple[list[int], list[int], list[int]]:
    """Work items of a step's portions: (request index, first query row, split word) per 128 query rows,
    longest first (CTAs are handed to SMs in this order, so the short ones fill the tail).

    With ``num_heads`` and ``sm_count`` given, a step whose tiles x heads leave SMs idle has the keys
    of its longest tiles cut into parts, each walked by a CTA of its own and merged by the last to
    finish: the tile with the most keys per part gets one more part until the CTAs fill the SMs once
    (a CTA costs several microseconds besides its keys, so a second round of CTAs would cost more
    than it saves).  A step with more tiles x heads than SMs has its rows cut when that evens out the
    rounds of CTAs (``_cut_for_even_rounds``; never more than ``max_items`` items then).  A part's item repeats its tile's (request, row); the split
    word is (index of the tile's first item) << 8 | parts."""
    groups = []  # [keys the tile's last row sees, request, first row, parts]
    for s, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        if skip_single and n == 1:
            continue  # (requests that bring a single token are the decode kernel's)
        for q0 in range(0, n, QUERY_TILE):
            groups.append([c - n + min(q0 + QUERY_TILE, n), s, q0, 1])
    if num_heads > 0 and sm_count > 0 and groups:
        room = sm_count // num_heads - len(groups)  # items that can be added within one round of CTAs
        while room > 0:
            g = max(groups, key=lambda g: g[0] / g[3])
            if g[3] >= MAX_PARTS or g[0] / (g[3] + 1) < MIN_PART_KEYS:
                break
            g[3] += 1
            room -= 1
        if _even_rounds and sm_count < len(groups) * num_heads <= ROUNDS_MAX_UNCUT * sm_count:
            _cut_for_even_rounds(groups, num_heads, sm_count, ROUNDS_MAX_ITEMS if max_items is None else max_items)
    groups.sort(key=lambda g: -(g[0] / g[3]))
    seqs, q0s, words = [], [], []
    for _, s, q0, parts in groups:
        first = len(seqs)
        for _ in range(parts):
            seqs.append(s)
            q0s.append(q0)
            words.append(first << 8 | parts)
    return seqs, q0s, words


ROUNDS_CTA_TILES = 7        # what a CTA costs besides its key tiles, in tiles' time (launch, look-ups, first loads, last store)
ROUNDS_MERGE_TILES = 3      # what a part adds to its CTA: the partial result written, and read again by the merger
ROUNDS_MIN_PART_TILES = 8   # no part shorter than this when rows are cut to even out rounds of CTAs
ROUNDS_MIN_GAIN = 0.05      # rows are cut only for an estimated gain of this much
ROUNDS_MAX_ITEMS = 64       # and into no more items than this (an unused item of a captured step's list is a CTA per head
                            # that starts and leaves; each item holds 128 x head size floats per head of scratch)
ROUNDS_MAX_UNCUT = 2        # only steps of at most this many rounds of whole CTAs are cut (measured: 448 CTAs of 28 heads, three
                            # rounds, gain 4 % behind 30,720 tokens and lose 3 % behind 18,432; 640 CTAs of 40 heads gain nothing)
ROUNDS_MIN_CTX = 8192       # rows no longer than this are not cut for even rounds (measured: no gain below, 3 % at 10,240 keys,
                            # 8 % at 18,432, 12 % at 30,720 for a 2,048-token portion of 12 heads; two to three parts are best)


def rounds_max_parts(max_ctx: int | None) -> int:
    """The most parts that ``_cut_for_even_rounds`` gives a row of up to ``max_ctx`` keys."""
    if not _even_rounds or (max_ctx is not None and max_ctx <= ROUNDS_MIN_CTX):
        return 1
    return MAX_PARTS


def _rounds_estimate(costs: np.ndarray, sm_count: int) -> float:
    """The time, in tiles, that CTAs of these costs (longest first) take when SMs pick them up in order as they
    become free: estimated by dealing them out in rounds, every other round in reverse."""
    rounds = -(-len(costs) // sm_count)
    table = np.zeros(rounds * sm_count, dtype=np.float64)
    table[: len(costs)] = costs
    table = table.reshape(rounds, sm_count)
    table[1::2] = table[1::2, ::-1]
    return float(table.sum(axis=0).max())


def _cut_for_even_rounds(groups: list[list], num_heads: int, sm_count: int, max_items: int) -> None:
    """More CTAs than SMs, up to ``ROUNDS_MAX_UNCUT`` times: when they are few and long (a portion behind a long context: 16 tiles x 12 heads of
    250 key tiles each on 148 SMs take two rounds for the work of 1.3), rows of keys are cut into parts of
    about equal length so that the rounds come out even.  The grain (tiles per part) is the longest row cut
    into 1, 2, ... parts; the one with the smallest estimated time wins, and nothing is cut for less than
    ``ROUNDS_MIN_GAIN`` or into more than ``max_items`` items.  Sets ``g[3]`` of the groups."""
    tiles = np.array([-(-g[0] // QUERY_TILE) for g in groups], dtype=np.int64)
    longest = int(tiles.max())

    def estimate(parts: np.ndarray) -> float:
        per = -(-tiles // parts)                                     # the kernel's division: every part `per` tiles,
        costs = np.repeat(per, parts)                                # the last what is left (it may be nothing)
        costs[np.cumsum(parts) - 1] = np.maximum(tiles - (parts - 1) * per, 0)
        costs = costs + np.repeat(ROUNDS_CTA_TILES + ROUNDS_MERGE_TILES * (parts > 1), parts)
        return _rounds_estimate(np.repeat(np.sort(costs)[::-1], num_heads), sm_count)

    if longest * QUERY_TILE <= ROUNDS_MIN_CTX:
        return  # (parts would cost about what they walk)
    # which grain: first by the rule for CTAs of equal length (rounds x a part's cost), then the winner as above
    tile_list = tiles.tolist()
    best = -(-len(tile_list) * num_heads // sm_count) * (longest + ROUNDS_CTA_TILES) * (1.0 - ROUNDS_MIN_GAIN)
    best_parts = None
    for most in range(2, MAX_PARTS + 1):
        grain = -(-longest // most)
        if grain < ROUNDS_MIN_PART_TILES:
            break
        parts = [min(MAX_PARTS, -(-t // grain)) for t in tile_list]
        total = sum(parts)
        if total > max_items:
            break
        time = -(-total * num_heads // sm_count) * (grain + ROUNDS_CTA_TILES + ROUNDS_MERGE_TILES)
        if time < best:
            best, best_parts = time, parts
    if best_parts is None:
        return
    best_parts = np.array(best_parts, dtype=np.int64)
    if estimate(best_parts) < estimate(np.ones_like(tiles)) * (1.0 - ROUNDS_MIN_GAIN):
        for g, n in zip(groups, best_parts.tolist()):
            g[3] = max(g[3], int(n))


_cut_long_rows = True
_even_rounds = True
_route_single_tokens = True


def set_even_rounds(on: bool) -> None:
    """Steps with more query tiles x heads than SMs cut their rows of keys when that evens out the rounds of
    CTAs, by default; ``False`` leaves them whole (for measurements; set before steps are captured)."""
    global _even_rounds
    _even_rounds = bool(on)


def set_route_single_tokens(on: bool) -> None:
    """In a step that mixes prompt portions with requests that bring one token, those requests are served
    by the decode kernel by default; ``False`` leaves them to the prefill kernel (for measurements)."""
    global _route_single_tokens
    _route_single_tokens = bool(on)



def set_cut_long_rows(on: bool) -> None:
    """Steps with few work items cut long rows of keys into parts by default; ``False`` gives every query
    tile one CTA (for measurements)."""
    global _cut_long_rows
    _cut_long_rows = bool(on)


def _cuts_for(num_heads: int, head_dim: int, page_size: int) -> int:
    """The head count that ``prefill_work_items`` cuts long rows of keys for: 0 when they are not cut."""
    return num_heads if _cut_long_rows and prefill_tc_takes(head_dim, page_size) else 0


def portion_step_arrays(num_heads: int, head_dim: int, page_size: int, max_tokens: int, max_seqs: int, device,
                        max_portions: int | None = None, max_ctx: int | None = None) -> dict:
    """The prefill kernel's work list as an array of a captured step (``Part.step_arrays``): three rows
    (request, first query row, split word) of fixed length, unused entries naming request -1.  The key
    says whether the step's single-token requests are served apart; with them apart only the
    ``max_portions`` requests that bring more than one token have items (every unused item is a CTA per
    head that starts and leaves)."""
    if head_dim not in PREFILL_HEAD_DIMS:
        return {}
    cuts = _cuts_for(num_heads, head_dim, page_size)
    sms = _sm_count(torch.device(device)) if cuts else 0
    # a tile per 128 rows and one more per request with items; cuts add parts until the CTAs fill the SMs once
    portions = max_seqs if max_portions is None else min(max_seqs, max_portions)
    # (or, with more tiles than that, up to ``rounds_max_parts`` parts per tile for contexts up to ``max_ctx``)
    most = rounds_max_parts(max_ctx) if cuts else 1
    caps = {False: max(max_tokens // QUERY_TILE + max_seqs + (sms // num_heads if cuts else 0),
                       min((max_tokens // QUERY_TILE + max_seqs) * most, ROUNDS_MAX_ITEMS)),
            True: max(max_tokens // QUERY_TILE + portions + (sms // num_heads if cuts else 0),
                      min((max_tokens // QUERY_TILE + portions) * most, ROUNDS_MAX_ITEMS))}

    def fill(q_lens, ctx_lens, apart: bool) -> np.ndarray:
        cap = caps[apart]
        seqs, q0s, words = prefill_work_items(q_lens, ctx_lens, cuts, sms, apart, cap)
        if len(seqs) > cap:
            raise RuntimeError(f"{len(seqs)} work items for a step captured with room for {cap}")
        out = np.zeros((3, cap), dtype=np.int32)
        out[0, :] = -1
        out[2, :] = 1  # (a whole tile: part 1 of 1)
        n = len(seqs)
        out[0, :n], out[1, :n], out[2, :n] = seqs, q0s, words
        return out.reshape(-1)

    def present(view: torch.Tensor, cap: int):
        return view[:cap], view[cap : 2 * cap], (view[2 * cap :] if cuts else None), cap

    # the one list that a step captured with these bounds reads: its single-token requests are served apart
    # (by the decode kernel) when it holds any, which is when the caller bounds its portions
    apart = max_portions is not None and _route_single_tokens and head_dim in DECODE_HEAD_DIMS
    return {("prefill_items", cuts, apart): (3 * caps[apart], lambda q, c: fill(q, c, apart), lambda view: present(view, caps[apart]))}


def _work_items(ctx, num_heads: int, skip_single: bool = False) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None, int]:
    """The step's work items on the device; built once per step and head count (``num_heads`` 0: no
    cuts) and shared by the layers."""
    key = ("prefill_items", num_heads, skip_single)
    cached = ctx.extras.get(key)
    if cached is None:
        if ctx.extras.get("captured_portions") is not None:
            raise RuntimeError(f"a captured step without the work list {key}: its graph was captured for another kind of step")
        seqs, q0s, words = prefill_work_items(ctx.q_lens_host, ctx.ctx_lens_host, num_heads,
                                              _sm_count(ctx.device) if num_heads else 0, skip_single)
        cut = any(w & 0xFF != 1 for w in words)
        host = torch.from_numpy(np.array([seqs, q0s, words], dtype=np.int32))
        dev = host.to(ctx.device, non_blocking=False)
        cached = (dev[0].contiguous(), dev[1].contiguous(), dev[2].contiguous() if cut else None, len(seqs))
        ctx.extras[key] = cached
    return cached


_prefill_scratch_by_device: dict[int, dict] = {}


def _prefill_scratch(device: torch.device, items: int, num_heads: int, head_dim: int) -> dict:
    """Partial results of cut work items (float32 O, (m, l) per row) and their arrival counters, kept
    per device and grown when a step needs more; the counters are zero between launches.  A set that is
    outgrown is kept alive: captured steps may point at it."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    slots = items * num_heads
    st = _prefill_scratch_by_device.get(index)
    if st is None or st["part_o"].numel() < slots * QUERY_TILE * head_dim or st["counters"].numel() < slots:
        if st is not None:
            _retired_scratch.append(st)
        st = {
            "part_o": torch.empty(slots * QUERY_TILE * head_dim, dtype=torch.float32, device=device),
            "part_ml": torch.empty(slots * QUERY_TILE * 2, dtype=torch.float32, device=device),
            "counters": torch.zeros(slots, dtype=torch.int32, device=device),
        }
        _prefill_scratch_by_device[index] = st
    return st


class _Prefill:
    @staticmethod
    def accepts(ctx, view, num_heads, num_kv_heads, head_dim, window) -> bool:
        return head_dim in PREFILL_HEAD_DIMS and ctx.q_start is not None

    @staticmethod
    def run(ctx, qkv, view, num_heads, num_kv_heads, head_dim, scale, window) -> torch.Tensor:
        # Requests that bring a single token go to the decode kernel (a context split over CTAs, the query
        # heads of a KV head sharing every tile) instead of taking a 128-row query tile per head here; the
        # two kernels fill one output tensor.
        captured = ctx.extras.get("captured_portions")
        if captured is not None:
            # a captured step: how its tokens are divided is not known here; the work list is an array of
            # the step, and whether single tokens are served apart was fixed when the step was captured
            singles = ctx.num_seqs if captured["singles"] and _route_single_tokens and head_dim in DECODE_HEAD_DIMS else 0
        else:
            singles = sum(1 for n in ctx.q_lens_host if n == 1) if _route_single_tokens and head_dim in DECODE_HEAD_DIMS else 0
        item_seq, item_q0, item_split, items = _work_items(ctx, _cuts_for(num_heads, head_dim, view.k_cache.shape[1]), singles > 0)
        out = attention_prefill(qkv, view.k_cache, view.v_cache, view.block_tables, ctx.q_start, ctx.ctx_lens,
                                item_seq, item_q0, items, num_heads, num_kv_heads, head_dim, scale, window, ctx.status,
                                item_split=item_split)
        if singles and captured is not None:
            # any of the step's requests may be one that brings a single token, with a context up to the
            # step's bound; how finely contexts are cut is a device scalar of the step
            split_dev = ctx.extras[dispatch.decode_split_name(num_heads, num_kv_heads, head_dim)]
            attention_decode(qkv, view.k_cache, view.v_cache, view.block_tables, ctx.ctx_lens, num_heads, num_kv_heads,
                             head_dim, scale, window, ctx.max_ctx_len, ctx.status,
                             split=decode_split_bound(singles, num_heads, num_kv_heads, ctx.max_ctx_len, qkv.device, head_dim),
                             split_dev=split_dev,
                             stages=decode_stages(singles, num_heads, num_kv_heads, ctx.max_ctx_len, qkv.device, head_dim),
                             q_start=ctx.q_start, out=out)
        elif singles:
            longest = max(c for n, c in zip(ctx.q_lens_host, ctx.ctx_lens_host) if n == 1)
            attention_decode(qkv, view.k_cache, view.v_cache, view.block_tables, ctx.ctx_lens, num_heads, num_kv_heads,
                             head_dim, scale, window, longest, ctx.status,
                             split=decode_split(singles, num_heads, num_kv_heads, longest, qkv.device, head_dim),
                             stages=decode_stages(singles, num_heads, num_kv_heads, longest, qkv.device, head_dim)
                             | decode_cluster(singles, num_heads, num_kv_heads, longest, qkv.device, head_dim) << CLUSTER_SHIFT,
                             q_start=ctx.q_start, out=out)
        return out


def attention_prefill(q, k_cache, v_cache, block_tables, q_start, ctx_lens, item_seq, item_q0, items, num_heads,
                      num_kv_heads, head_dim, scale, window, status, use_tc: bool | None = None,
                      item_split: torch.Tensor | None = None) -> torch.Tensor:
    """Any mixture of portions: ``q`` [N, >= nh*hd]; request s owns rows q_start[s]:q_start[s+1] and has
    ctx_lens[s] tokens in the cache, its portion at the end.  Returns [N, nh*hd].  ``use_tc``: the
    tcgen05 kernel (default: whenever it takes the head size and the page size) or the mma.sync one.
    ``item_split`` (tcgen05 kernel only): the split words of ``prefill_work_items`` when items are parts."""
    _configure()
    if q.dtype != torch.bfloat16 or q.dim() != 2 or q.stride(1) != 1:
        raise ValueError("q must be a 2-d bfloat16 tensor with unit column stride")
    _need(k_cache, torch.bfloat16, "k_cache", 4)
    _need(v_cache, torch.bfloat16, "v_cache", 4)
    _need(block_tables, torch.int32, "block_tables", 2)
    for name, t in (("q_start", q_start), ("ctx_lens", ctx_lens), ("item_seq", item_seq), ("item_q0", item_q0)):
        _need(t, torch.int32, name, 1)
    if head_dim not in PREFILL_HEAD_DIMS:
        raise ValueError(f"head_dim {head_dim} is not one of {PREFILL_HEAD_DIMS}")
    out = torch.empty((q.shape[0], num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    if use_tc is None:
        use_tc = prefill_tc_takes(head_dim, k_cache.shape[1])
    if item_split is not None and not use_tc:
        raise ValueError("only the tcgen05 kernel takes work items that are parts")
    if use_tc:
        st = {"part_o": None, "part_ml": None, "counters": None}
        if item_split is not None:
            _need(item_split, torch.int32, "item_split", 1)
            st = _prefill_scratch(q.device, items, num_heads, head_dim)
        check(library().cw_attention_prefill_tc(
            _ptr(q), q.stride(0), q.shape[1], q.shape[0], _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables),
            _ptr(q_start), _ptr(ctx_lens), _ptr(item_seq), _ptr(item_q0), _ptr(item_split), _ptr(st["part_o"]),
            _ptr(st["part_ml"]), _ptr(st["counters"]), items, num_heads, num_kv_heads, head_dim,
            k_cache.shape[1], block_tables.shape[1], k_cache.shape[0], float(scale), int(window or 0), _ptr(status),
            _stream()), "attention_prefill_tc")
        return out
    check(library().cw_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(q_start), _ptr(ctx_lens),
        _ptr(item_seq), _ptr(item_q0), items, num_heads, num_kv_heads, head_dim, k_cache.shape[1], block_tables.shape[1],
        k_cache.shape[0], float(scale), int(window or 0), _ptr(status), _stream()), "attention_prefill")
    return out


def enable() -> None:
    dispatch._decode = _Decode
    dispatch._prefill = _Prefill


enable()
