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


def check(got: torch.Tensor, want, dtype: str, what: str, derived_float32: bool = False) -> None:
    """``want`` = (exact, rounded).  float32: 1e-5 against ``exact``.  bfloat16: at most 2.5 times as far
    from ``exact`` as ``rounded`` is (see above).  ``derived_float32``: the same derived rule for a float32
    run, for models whose inner dimensions are so long that float32 arithmetic alone moves the logits by
    more than 1e-5: ``exact`` is then the plain implementation in float64 and ``rounded`` the plain
    implementation in float32."""
    exact, rounded = want
    exact, rounded = exact.to(torch.float32), rounded.to(torch.float32)
    diff = (got - exact).abs()
    if dtype == "float32" and not derived_float32:
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


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "no-graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_one_request_at_a_time(name, dtype, graphs, sharp_dirs, references, tmp_path):
    """Whole; decoded tail; portions of changing size.  One process, requests one after another in a
    pool that holds exactly one of them, so each reuses the pages of the one before.  Single-token
    steps replay the captured graphs that generation uses, or (``--no-graphs``) the plain step function."""
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
    out = run_trace(sharp_dirs[name], dtype, round_up(150, 64), tb.steps, tmp_path / "out", raw["vocab_size"], page,
                    extra_args=() if graphs else ("--no-graphs",))
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


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "no-graphs"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_forked_requests_copy_on_write(name, dtype, graphs, sharp_dirs, references, tmp_path):
    """A request is forked in the middle of a page and parent and child go on with different tokens:
    whoever writes first into the shared page gets a copy of it (all layers, keys and values), the
    other keeps the original, and every position of both equals the plain implementation (after the
    reference's tests/test_block_manager.py:142-191).  Before the fork the parent decodes single tokens
    beside a bystander, and in the fork's own step the child sits out, so that on the graph path the
    parent's block-table row is already held by that captured step's inputs when the copy changes an
    entry of it.  A second fork falls on a page's edge (nothing to copy), a third forks a child; the
    first parent ends and its children live on."""
    raw, _seed, page = TINY[name]
    vocab = raw["vocab_size"]
    stream = {rid: iter(tokens_for(name, 80, salt=40 + i)) for i, rid in enumerate("pxcde")}
    seqs: dict[str, list[int]] = {"p": [], "x": []}
    forked_at: dict[str, int] = {"p": 0, "x": 0}
    tb = TraceBuilder()

    def feed(rid, n=1):
        tokens = [next(stream[rid]) for _ in range(n)]
        seqs[rid] += tokens
        return (rid, tokens, True)

    def fork(parent, child):
        seqs[child] = list(seqs[parent])
        forked_at[child] = len(seqs[parent])
        return (parent, child)

    tb.step([feed("p", 41), feed("x", 10)])      # 41 + 4 = 45: 45 % 4 == 1 and 45 % 8 == 5, inside a page
    for _ in range(4):
        tb.step([feed("p"), feed("x")])
    assert len(seqs["p"]) % page != 0
    forks = [fork("p", "c")]
    tb.step([feed("p"), feed("x")], fork=forks)   # the parent writes first, the child sits out
    for _ in range(10):
        tb.step([feed("c"), feed("p"), feed("x")])
    to_edge = (-len(seqs["p"])) % page or page
    tb.step([feed("p", to_edge), feed("c"), feed("x")], end=["x"])  # a portion takes the parent to a page's edge
    assert len(seqs["p"]) % page == 0
    forks = [fork("p", "d")]
    tb.step([feed("d", 3), feed("p"), feed("c")], fork=forks)
    assert len(seqs["c"]) % page != 0
    forks = [fork("c", "e")]
    tb.step([feed("e"), feed("c"), feed("d")], fork=forks, end=["p"])
    for i in range(6):
        tb.step([feed("c"), feed("d"), feed("e")], end=["c", "d", "e"] if i == 5 else [])
    budget = sum(round_up(len(t), 64) for t in seqs.values())
    out = run_trace(sharp_dirs[name], dtype, budget, tb.steps, tmp_path / "out", vocab, page,
                    extra_args=() if graphs else ("--no-graphs",))
    assert forked_at["c"] == 45 and forked_at["d"] % page == 0 and forked_at["e"] % page != 0
    for rid, tokens in seqs.items():
        exact, rounded = references(name, tokens)
        first = forked_at[rid]
        check(tb.gather(out, rid, len(tokens), first=first), (exact[first:], rounded[first:]), dtype,
              f"{name} {dtype} fork {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_prefix_cache_hits_keep_logits(name, dtype, sharp_dirs, references, tmp_path):
    """Prompts of 1, 9, 23 and 40 tokens, two of which share their first 16 tokens with an earlier
    40-token prompt, in portions of 7: the later ones take the shared whole pages from the prefix cache
    instead of computing them, and the logits of everything they do compute (the rest of the prompt, in
    portions, then 12 tokens one by one) equal the plain implementation.  The pool is so small that
    pages held only by the prefix cache have to be given back for the last request.  (The workload of
    the second tiny configuration as the benchmark description gives it, run on both.)"""
    raw, _seed, page = TINY[name]
    vocab = raw["vocab_size"]
    shared = tokens_for(name, 16, salt=60)
    prompts = {
        "first40": shared + tokens_for(name, 24, salt=61),
        "one": tokens_for(name, 1, salt=62),
        "hit23": shared + tokens_for(name, 7, salt=63),
        "nine": tokens_for(name, 9, salt=64),
        "hit40": shared + tokens_for(name, 24, salt=65),
        "again40": shared + tokens_for(name, 24, salt=61),   # the first prompt once more: all but its last page is there
        "cold": tokens_for(name, 100, salt=66),               # needs the pages that the prefix cache still holds
    }
    seqs = {rid: p + tokens_for(name, 12, salt=70 + i) for i, (rid, p) in enumerate(prompts.items())}
    tb = TraceBuilder()

    def run_request(rid, others=()):
        prompt, full = prompts[rid], seqs[rid]
        # what a scheduler does: look the whole prompt up, then cut what is left into portions of 7;
        # in a trace the first entry therefore carries the matched part and the first portion
        head = min(len(prompt), 16 + 7) if rid.startswith(("hit", "again")) else min(len(prompt), 7)
        if rid == "again40":
            head = 32 + 7
        tb.step([(rid, full[:head], True)])
        pos = head
        for portion in cut(full[head : len(prompt)], [7]):
            tb.step([(rid, portion, True)])
            pos += len(portion)
        for i, t in enumerate(full[len(prompt):]):
            tb.step([(rid, [t], True)], end=[rid] if i == 11 else [])

    for rid in prompts:
        run_request(rid)
    # 192 tokens of pages: the first six requests and what the prefix cache keeps of them fit (at most
    # 152 tokens), the last request (112 tokens) fits only once the prefix cache gives its idle pages back
    out = run_trace(sharp_dirs[name], dtype, 192, tb.steps, tmp_path / "out", vocab, page,
                    extra_args=("--prefix-cache",))
    taken = {rid: n for cached in out.cached.values() for rid, n in cached.items()}
    last_page = (40 - 1) // page * page
    assert taken == {"hit23": 16, "hit40": 16, "again40": last_page}, taken
    for rid, tokens in seqs.items():
        exact, rounded = references(name, tokens)
        first = taken.get(rid, 0)
        check(tb.gather(out, rid, len(tokens), first=first), (exact[first:], rounded[first:]), dtype,
              f"{name} {dtype} prefix {rid}")
