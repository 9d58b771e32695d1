"""Which captured step a step of prompt portions replays, as far as its token count decides (host side, no GPU):
short steps are padded to the next of a few buckets, long ones to a multiple of 256 tokens when that wastes at
most 4 %, and the rest are launched kernel by kernel."""

from clockwork_b200.engine.step import ModelRunner


class Rules:
    """The runner's constants without a runner (the rule reads nothing else)."""

    PORTION_TOKEN_BUCKETS = ModelRunner.PORTION_TOKEN_BUCKETS
    PORTION_MAX_TOKENS = ModelRunner.PORTION_MAX_TOKENS
    PORTION_LONG_STEP = ModelRunner.PORTION_LONG_STEP
    PORTION_LONG_WASTE = ModelRunner.PORTION_LONG_WASTE


def bucket(tokens):
    return ModelRunner._portion_token_bucket(Rules, tokens)


def test_short_steps_take_the_next_bucket():
    buckets = ModelRunner.PORTION_TOKEN_BUCKETS
    assert list(buckets) == sorted(buckets) and buckets[0] <= 16 and buckets[-1] == 1024
    for tokens in range(2, buckets[-1] + 1):
        b = bucket(tokens)
        assert b in buckets and b >= tokens
        assert all(other < tokens for other in buckets if other < b)  # the smallest bucket that holds the step


def test_long_steps_are_padded_by_four_percent_at_most():
    captured = 0
    for tokens in range(1025, 6000):
        b = bucket(tokens)
        if b is None:
            continue
        captured += 1
        assert tokens <= b <= ModelRunner.PORTION_MAX_TOKENS and b % 256 == 0 and b <= tokens * 1.04
    assert captured > 1000
    assert bucket(2048) == 2048 and bucket(4096) == 4096 and bucket(2000) == 2048
    assert bucket(1100) is None and bucket(4097) is None  # (16 % of padding; beyond the longest captured step)
