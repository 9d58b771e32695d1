"""How the decode kernel's context splits and variants are chosen (host side, no GPU): what a captured step
reserves bounds what any of its replays can ask for, every CTA of a step is resident at once, and a split is
never finer than 128 tokens."""

import random

import pytest

from clockwork_b200.ops import attention_fast as fast

SMS = 148


@pytest.fixture(autouse=True)
def sm_count(monkeypatch):
    monkeypatch.setattr(fast, "_sm_count", lambda device=None: SMS)


SIZES = [(12, 2, 128), (28, 4, 128), (40, 8, 128), (4, 2, 64), (8, 8, 96), (3, 1, 256), (32, 2, 128)]


def test_the_split_bound_of_a_captured_step_covers_every_replay():
    rng = random.Random(1)
    for nh, nkv, hd in SIZES:
        for max_seqs in (1, 8, 32, 64):
            for max_ctx in (1024, 2048, 16384, 32768):
                bound = fast.decode_split_bound(max_seqs, nh, nkv, max_ctx, None, hd)
                for _ in range(40):
                    n, ctx = rng.randint(1, max_seqs), rng.randint(1, max_ctx)
                    split = fast.decode_split(n, nh, nkv, ctx, None, hd)
                    assert fast.MIN_SPLIT <= split <= bound and split % 64 == 0, (nh, nkv, hd, max_seqs, max_ctx, n, ctx)


def test_all_ctas_of_a_step_are_resident_at_once():
    """CTAs = (request, KV head, group of 16 query heads) x splits; the split is chosen for the two-tile variant's
    residency, and whatever variant the step takes holds at least as many CTAs per SM."""
    rng = random.Random(2)
    for nh, nkv, hd in SIZES:
        for _ in range(200):
            n, ctx = rng.randint(1, 64), rng.choice([1, 100, 1024, 1100, 4096, 20000, 32768])
            split = fast.decode_split(n, nh, nkv, ctx, None, hd)
            pairs = fast._pairs(n, nh, nkv)
            splits = -(-ctx // split)
            room = fast._resident_ctas(hd, swizzled=fast._unpadded(hd, pairs)) * SMS
            if split > fast.MIN_SPLIT:  # (at the finest split a long context of many requests may need more than one round)
                assert pairs * splits <= max(room, pairs), (nh, nkv, hd, n, ctx, split, splits, room)
            stages = fast.decode_stages(n, nh, nkv, ctx, None, hd)
            tiles = stages & 0xFF
            unpadded = bool(stages & fast.SWIZZLED)
            assert tiles in (2, 4) and (not unpadded or hd % 64 == 0)
            if stages & fast.TMA_TILES:
                assert unpadded and tiles == 2
            if pairs * splits <= room and split > fast.MIN_SPLIT:
                assert fast._resident_ctas(hd, tiles, unpadded) * SMS >= pairs * splits, (nh, nkv, hd, n, ctx, stages)
