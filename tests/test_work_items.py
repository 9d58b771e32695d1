"""Work items of the prefill attention kernel (host side, no GPU): every query tile is there once per
part, the parts of a tile are consecutive and name their first, tiles are cut while the step's
CTAs leave SMs idle, the longest first, or when more CTAs than SMs come out in uneven rounds, and items come
longest part first."""

from clockwork_b200.ops import attention_fast as fast


def check(q_lens, ctx_lens, num_heads=0, sm_count=0, max_items=None):
    seqs, q0s, words = fast.prefill_work_items(q_lens, ctx_lens, num_heads, sm_count, max_items=max_items)
    assert len(seqs) == len(q0s) == len(words)
    seen, i = {}, 0
    while i < len(words):
        first, parts = words[i] >> 8, words[i] & 0xFF
        assert first == i and 1 <= parts <= fast.MAX_PARTS
        for k in range(parts):
            assert (seqs[i + k], q0s[i + k], words[i + k]) == (seqs[i], q0s[i], words[i])
        seen[(seqs[i], q0s[i])] = parts
        i += parts
    tiles = {(s, q0) for s, n in enumerate(q_lens) for q0 in range(0, n, fast.QUERY_TILE)}
    assert set(seen) == tiles
    keys = {(s, q0): ctx_lens[s] - q_lens[s] + min(q0 + fast.QUERY_TILE, q_lens[s]) for s, q0 in tiles}
    cost = [keys[(s, q0)] / (w & 0xFF) for s, q0, w in zip(seqs, q0s, words)]
    assert cost == sorted(cost, reverse=True)
    for tile, parts in seen.items():
        assert parts == 1 or keys[tile] / parts >= fast.MIN_PART_KEYS
    return seen, keys


def test_a_step_that_fills_the_sms_is_not_cut():
    seen, _ = check([2048], [2048], num_heads=12, sm_count=148)  # 16 tiles x 12 heads
    assert set(seen.values()) == {1}
    seen, _ = check([2048, 7], [2048, 900])  # no head count: no cuts
    assert set(seen.values()) == {1}


def test_few_tiles_with_many_keys_are_cut_until_the_sms_are_full():
    seen, keys = check([128], [40000], num_heads=12, sm_count=148)  # one tile: 12 CTAs without cuts
    assert seen == {(0, 0): 8}
    seen, keys = check([1024], [1024], num_heads=12, sm_count=148)  # 8 tiles, room for 4 more items
    assert seen[(0, 896)] == 2 and sum(seen.values()) == 9  # only the longest row is worth a cut
    seen, keys = check([512], [4096], num_heads=12, sm_count=148)  # 4 tiles of about 4,000 keys, room for 8 more
    assert sorted(seen.values()) == [3, 3, 3, 3]
    seen, _ = check([300, 1, 64, 0], [2500, 5000, 64, 10], num_heads=4, sm_count=148)
    assert seen[(1, 0)] == 8 and seen[(2, 0)] == 1
    seen, _ = check([5, 1], [300, 400], num_heads=2, sm_count=148)  # nothing is worth cutting
    assert set(seen.values()) == {1}


def test_more_ctas_than_sms_are_cut_when_that_evens_out_the_rounds():
    """A 2,048-token portion behind 30,720 tokens: 16 tiles x 12 heads of about 250 key tiles each take two
    rounds on 148 SMs for the work of 1.3; in three parts each they take four rounds of a third."""
    seen, _ = check([2048], [32768], num_heads=12, sm_count=148)
    assert set(seen.values()) == {3}
    seen, _ = check([2048], [32768], num_heads=12, sm_count=148, max_items=40)  # room for two parts each only
    assert set(seen.values()) == {2}
    seen, _ = check([2048], [32768], num_heads=12, sm_count=148, max_items=20)  # no room
    assert set(seen.values()) == {1}
    # a first portion (rows of 128 to 2,048 keys: the short ones fill the second round) and a portion behind a short
    # context (a part would cost about what it walks) stay whole; so does a step whose rounds are even already
    for q, c in (([2048], [2048]), ([2048], [4096]), ([2048], [8192]), ([4096], [16384])):
        seen, _ = check(q, c, num_heads=12, sm_count=148)
        assert set(seen.values()) == {1}, (q, c)
    # two portions of different requests at different contexts beside a single token: parts of about equal length
    seen, keys = check([1024, 1024, 1], [20000, 9000, 5000], num_heads=12, sm_count=148)
    assert all(seen[(0, q0)] == 4 for q0 in range(0, 1024, 128)) and all(seen[(1, q0)] == 2 for q0 in range(0, 1024, 128))
    # more than two rounds of whole CTAs (17 tiles x 28 heads): the rounds are even enough as they are
    seen, keys = check([1024, 1024, 1], [20000, 9000, 5000], num_heads=28, sm_count=148)
    assert set(seen.values()) == {1}
    assert fast.rounds_max_parts(8192) == 1 and fast.rounds_max_parts(16384) == fast.rounds_max_parts(None) == fast.MAX_PARTS


def test_a_captured_step_s_list_always_has_room(monkeypatch):
    """Whatever a step of up to the captured bounds holds (random divisions of its tokens among its requests,
    random contexts up to the tier's bound, with and without single tokens served apart), the work list fits
    the fixed length that the captured step reserved, unused entries name no request, and the entries are a
    valid list of parts."""
    import random

    import numpy as np

    monkeypatch.setattr(fast, "_sm_count", lambda device=None: 148)
    rng = random.Random(7)
    for trial in range(300):
        heads = rng.choice([2, 4, 12, 14, 28, 40])
        max_tokens = rng.choice([128, 256, 512, 1024, 2048, 2560, 4096])
        max_seqs = rng.choice([8, 64])
        max_ctx = rng.choice([1024, 2048, 8192, 16384, 32768])
        singles = rng.random() < 0.5
        decl = fast.portion_step_arrays(heads, 128, 16, max_tokens, max_seqs, "cuda:0", 8 if singles else None, max_ctx)
        (key, (words, fill, present)), = decl.items()
        assert key[2] == singles
        # a step within the bounds: portions (at most 8 beside single tokens), then single tokens if it holds any
        q_lens, left = [], max_tokens
        for _ in range(rng.randint(1, 8 if singles else min(max_seqs, 12))):
            if left < 2:
                break
            n = rng.choice([2, 7, 100, 128, 129, 300, 1000, left])
            n = max(2, min(n, left))
            q_lens.append(n)
            left -= n
        if singles:
            q_lens += [1] * min(left, max_seqs - len(q_lens), rng.randint(1, 40))
        ctx_lens = [rng.randint(n, max(n, max_ctx)) for n in q_lens]
        if rng.random() < 0.5:  # all behind long contexts: the case that cuts the most
            ctx_lens = [max(n, max_ctx - rng.randint(0, 64)) for n in q_lens]
        flat = fill(q_lens, ctx_lens)
        assert flat.dtype == np.int32 and flat.shape == (words,)
        cap = words // 3
        seqs, q0s, split = flat[:cap], flat[cap : 2 * cap], flat[2 * cap :]
        used = int((seqs >= 0).sum())
        assert (seqs[:used] >= 0).all() and (seqs[used:] == -1).all()
        i, tiles = 0, set()
        while i < used:
            first, parts = int(split[i]) >> 8, int(split[i]) & 0xFF
            assert first == i and 1 <= parts <= fast.MAX_PARTS and i + parts <= used
            assert all((seqs[i + k], q0s[i + k], split[i + k]) == (seqs[i], q0s[i], split[i]) for k in range(parts))
            tiles.add((int(seqs[i]), int(q0s[i])))
            i += parts
        want = {(s, q0) for s, n in enumerate(q_lens) if not (singles and n == 1) for q0 in range(0, n, fast.QUERY_TILE)}
        assert tiles == want, (trial, q_lens, ctx_lens)
