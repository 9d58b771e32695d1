"""Trace replay against the plain implementation, in float32 and bfloat16, for both tiny
configurations: each request whole; most of it in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; and up to four live requests mixed in one batch
(portions of some beside single tokens of others, requests sitting out steps) in a pool so small
that pages are used again.  The models are the 'sharp' variants (peaked attention), so a missed,
misplaced or stale key shows."""

import pytest
import torch

from tests.plain import qwen2_plain as plain
from tests.tiny_configs import TINY, tokens_for
from tests.trace_tools import TraceBuilder, cut, round_up, run_trace

pytestmark = pytest.mark.gpu

# float32: the reference's own gate (tests/test_hf_equivalence.py:15-16), elementwise.
# bfloat16: the yardstick is the plain implementation itself with its activations rounded to
# bfloat16 where a bfloat16 run stores them (qwen2_plain.to_bfloat16_and_back).  How far that moves
# the logits of this very request is what bfloat16 storage costs on this model; the engine, whose
# roundings fall differently, may be off by at most 2.5 times that maximum at any logit, and its
# mean error by at most 2 times that mean.
F32_TOL = dict(rtol=1e-5, atol=1e-5)


def check(got: torch.Tensor, want, dtype: str, what: str) -> None:
    exact, rounded = want
    diff = (got - exact).abs()
    if dtype == "float32":
        ok = torch.isclose(got, exact, **F32_TOL)
        bound = "1e-5"
    else:
        yard = (rounded - exact).abs()
        ok = diff <= 2.5 * float(yard.max())
        bound = f"2.5 x {float(yard.max()):.3e}"
        assert float(diff.mean()) <= 2.0 * float(yard.mean()), (
            f"{what}: mean abs diff {float(diff.mean()):.3e} against {float(yard.mean()):.3e} from rounding alone")
    if not bool(ok.all()):
        bad = (~ok).any(dim=1).nonzero().flatten()
        first = int(bad[0])
        raise AssertionError(
            f"{what}: first wrong position {first} of {got.shape[0]} (max diff there {diff[first].max():.3e}, "
            f"bound {bound}; {len(bad)} positions wrong; overall max {diff.max():.3e})"
        )


@pytest.fixture(scope="module")
def references(sharp_dirs):
    cache = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in cache:
            config, weights = plain.read_model_dir(sharp_dirs[name])
            cache[key] = (plain.all_position_logits(config, weights, tokens),
                          plain.all_position_logits(config, weights, tokens, rnd=plain.to_bfloat16_and_back))
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_one_request_at_a_time(name, dtype, sharp_dirs, references, tmp_path):
    """Whole; decoded tail; portions of changing size.  One process, requests one after another in a
    pool that holds exactly one of them, so each reuses the pages of the one before."""
    raw, _seed, page = TINY[name]
    lengths = {"whole": 150, "tail": 141, "cuts": 150, "first": 3, "one": 1}
    toks = {k: tokens_for(name, n, salt=i) for i, (k, n) in enumerate(lengths.items())}
    tb = TraceBuilder()
    tb.step([("whole", toks["whole"], True)], end=["whole"])
    head = len(toks["tail"]) - 32
    tb.step([("tail", toks["tail"][:head], True)])
    for i, t in enumerate(toks["tail"][head:]):
        tb.step([("tail", [t], True)], end=["tail"] if i == 31 else [])
    portions = cut(toks["cuts"], [7, 2, 13, 2, 5, 3, 2, 11, 16, 2, 1, 9])
    for i, portion in enumerate(portions):
        tb.step([("cuts", portion, True)], end=["cuts"] if i == len(portions) - 1 else [])
    tb.step([("first", toks["first"], True)], end=["first"])  # the first tokens of a sequence
    tb.step([("one", toks["one"], True)], end=["one"])
    out = run_trace(sharp_dirs[name], dtype, round_up(150, 64), tb.steps, tmp_path / "out", raw["vocab_size"], page)
    for rid, tokens in toks.items():
        check(tb.gather(out, rid, len(tokens)), references(name, tokens), dtype, f"{name} {dtype} {rid}")


def mixed_trace(name):
    """Six requests, at most four live; every step is one batch of whatever each live request does
    next: a prompt portion of changing size, or (in its last 32 tokens) a single token; now and then
    a request sits a step out.  Requests end and new ones take over their pages."""
    lengths = [70, 101, 133, 64, 47, 90]
    toks = {f"r{i}": tokens_for(name, n, salt=10 + i) for i, n in enumerate(lengths)}
    sizes = {"r0": [9, 2, 17], "r1": [33, 2, 6], "r2": [2, 40, 3, 11], "r3": [13, 5], "r4": [4, 2, 25], "r5": [50, 2, 7]}
    tb = TraceBuilder()
    waiting = list(toks)
    live: list[str] = []
    pos = {rid: 0 for rid in toks}
    turn = {rid: 0 for rid in toks}
    peak = 0
    n = 0
    while waiting or live:
        while waiting and len(live) < 4 and (n % 3 == 0 or not live):
            live.append(waiting.pop(0))
        portions, ended = [], []
        for k, rid in enumerate(list(live)):
            if (n + k) % 5 == 4 and len(live) > 1:
                continue  # sits this step out and goes on later
            left = len(toks[rid]) - pos[rid]
            size = 1 if left <= 32 else min(sizes[rid][turn[rid] % len(sizes[rid])], left - 32)
            turn[rid] += 1
            portions.append((rid, toks[rid][pos[rid] : pos[rid] + size], True))
            pos[rid] += size
            if pos[rid] == len(toks[rid]):
                ended.append(rid)
        peak = max(peak, sum(round_up(pos[r], 64) for r in live))
        tb.step(portions, end=ended)
        for rid in ended:
            live.remove(rid)
        n += 1
    return tb, toks, peak


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_mixed_batches_with_page_reuse(name, dtype, sharp_dirs, references, tmp_path):
    raw, _seed, page = TINY[name]
    tb, toks, peak = mixed_trace(name)
    assert peak < sum(round_up(len(t), 64) for t in toks.values())  # so pages must be used again
    mixed = [s for s in tb.steps if len(s["entries"]) > 1]
    assert any(len(s["entries"]) == 4 for s in tb.steps)
    assert any({len(e["tokens"]) for e in s["entries"]} >= {1} and max(len(e["tokens"]) for e in s["entries"]) > 1 for s in mixed)
    out = run_trace(sharp_dirs[name], dtype, peak, tb.steps, tmp_path / "out", raw["vocab_size"], page)
    for rid, tokens in toks.items():
        check(tb.gather(out, rid, len(tokens)), references(name, tokens), dtype, f"{name} {dtype} mixed {rid}")


def test_default_page_size_and_unwanted_steps(sharp_dirs, references, tmp_path):
    """The default page size (16); steps that want nothing write no file; wanting a subset."""
    name = "B"
    raw = TINY[name][0]
    tokens = tokens_for(name, 100, salt=77)
    tb = TraceBuilder()
    tb.step([("x", tokens[:50], False)])
    tb.steps.append({"step": 1, "entries": [{"id": "x", "tokens": tokens[50:], "want": [0, 49]}], "end": ["x"]})
    out = run_trace(sharp_dirs[name], "float32", 128, tb.steps, tmp_path / "out", raw["vocab_size"])
    ref = references(name, tokens)[0]
    torch.testing.assert_close(torch.from_numpy(out[1]), ref[[50, 99]], rtol=1e-5, atol=1e-5)
