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
