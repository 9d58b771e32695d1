"""Short steps that hold prompt portions replay captured CUDA graphs (``engine/step.py:PortionGraph``):
that they do, that what they compute is what the uncaptured step computes (both against the plain
implementation), whatever the step holds (one prompt, several, portions deep in a context, single tokens
beside portions, logits wanted at every place or at one per request), and that long steps which would need
much padding, steps in float32 and steps through parts that do not declare themselves safe stay uncaptured."""

import pytest
import torch

from clockwork_b200 import EngineConfig
from clockwork_b200.engine import LLMEngine, StepEntry, load_model
from tests.plain import qwen2_plain as plain
from tests.test_replay_gpu import check
from tests.tiny_configs import TINY, tokens_for

pytestmark = pytest.mark.gpu


def runner_for(folder, name, dtype, graphs=True, max_model_len=2048, seqs=16):
    page = TINY[name][2]
    cfg = EngineConfig.defaults(str(folder), dtype=dtype, block_size=page, num_blocks=(seqs * max_model_len) // page // 4 + 64,
                                max_model_len=max_model_len, max_num_seqs=seqs, max_num_batched_tokens=4096,
                                enable_prefix_cache=False, cuda_graphs=graphs)
    eng = LLMEngine(cfg, model=load_model(folder, cfg.model.dtype))
    return eng, eng.runner, eng.cache


class Replayed:
    """Feeds requests through a runner portion by portion and keeps every position's logits."""

    def __init__(self, runner, cache):
        self.runner, self.cache = runner, cache
        self.done: dict[str, int] = {}
        self.logits: dict[str, list] = {}

    def step(self, portions: dict[str, list[int]], want_all=True) -> None:
        entries = []
        for rid, toks in portions.items():
            if rid not in self.done:
                self.cache.open(rid)
                self.done[rid], self.logits[rid] = 0, []
            entries.append(StepEntry(rid, toks, list(range(len(toks))) if want_all else [len(toks) - 1]))
        out = self.runner.step(entries).float().cpu()
        row = 0
        for e in entries:
            for w in e.want:
                self.logits[e.request_id].append((self.done[e.request_id] + w, out[row].clone()))
                row += 1
            self.done[e.request_id] += len(e.tokens)
        self.runner.check_status()

    def of(self, rid):
        rows = sorted(self.logits[rid], key=lambda pair: pair[0])
        return [p for p, _ in rows], torch.stack([r for _, r in rows])


@pytest.mark.parametrize("name", sorted(TINY))
def test_short_steps_with_portions_replay_captured_graphs(name, sharp_dirs):
    folder = sharp_dirs[name]
    config, weights = plain.read_model_dir(folder)
    _eng, runner, cache = runner_for(folder, name, "bfloat16")
    assert runner.portions_captured
    toks = {rid: tokens_for(name, n, salt=40 + i) for i, (rid, n) in enumerate(
        {"a": 150, "b": 90, "c": 61, "d": 300, "e": 1200, "f": 2040, **{f"m{i}": 20 + i for i in range(9)}}.items())}
    run = Replayed(runner, cache)
    run.step({"a": toks["a"]})                                        # one prompt, logits everywhere
    assert runner.portion_graph_steps == 1
    run.step({"b": toks["b"][:37], "c": toks["c"][:60]})              # two prompts' first portions
    run.step({"b": toks["b"][37:88], "c": toks["c"][60:], "d": toks["d"][:130]}, want_all=False)  # one row per request
    run.step({"b": toks["b"][88:89], "d": toks["d"][130:299]})        # a single token beside a portion deep in a context
    run.step({"b": toks["b"][89:], "d": toks["d"][299:]})             # two single tokens: the decode steps' business
    assert runner.portion_graph_steps == 4
    keys = set(runner.portion_graphs)
    assert {k[4] for k in keys} == {False, True}, keys                # captured with and without single tokens beside the portions
    assert {k[2] for k in keys} == {8, 192, 128}, keys                # rows: one per request, or every place of the bucket
    run.step({"e": toks["e"][:1100]}, want_all=False)                 # a long step far from a multiple of 256 tokens: not padded
    run.step({"e": toks["e"][1100:]}, want_all=False)                 # short again, at a context beyond 1,024: the next tier
    assert runner.portion_graph_steps == 5 and any(k[3] == 2048 for k in runner.portion_graphs)
    run.step({f"m{i}": toks[f"m{i}"][:-2] for i in range(9)})         # more requests than the small bucket holds: the next one
    assert runner.portion_graph_steps == 6 and any(k[1] == 64 for k in runner.portion_graphs)
    run.step({"f": toks["f"]}, want_all=False)                        # a long step just below a multiple of 256 tokens
    assert runner.portion_graph_steps == 7 and any(k[0] == 2048 for k in runner.portion_graphs)
    # fewer tokens than the step has room for requests: nine single tokens beside a new prompt of three (bucket of 16
    # tokens, 64 requests), then nine beside its last two tokens
    toks["n"] = tokens_for(name, 5, salt=99)
    run.step({**{f"m{i}": toks[f"m{i}"][-2:-1] for i in range(9)}, "n": toks["n"][:3]})
    run.step({**{f"m{i}": toks[f"m{i}"][-1:] for i in range(9)}, "n": toks["n"][3:]})
    assert runner.portion_graph_steps == 9 and any(k[0] == 16 and k[1] == 64 for k in runner.portion_graphs)
    for rid in ("a", "b", "c", "d", "e", "f", "m0", "m4", "m8", "n"):
        places, got = run.of(rid)
        exact = plain.all_position_logits(config, weights, toks[rid])
        rounded = plain.all_position_logits(config, weights, toks[rid], rnd=plain.to_bfloat16_and_back)
        check(got, (exact[places], rounded[places]), "bfloat16", f"{name} {rid}")


def test_captured_steps_are_kept_up_to_a_number_and_the_least_recently_used_go(sharp_dirs, monkeypatch):
    folder = sharp_dirs["B"]
    config, weights = plain.read_model_dir(folder)
    _eng, runner, cache = runner_for(folder, "B", "bfloat16")
    monkeypatch.setattr(type(runner), "PORTION_MAX_GRAPHS", 2)
    run = Replayed(runner, cache)
    toks = {rid: tokens_for("B", n, salt=70 + i) for i, (rid, n) in enumerate({"a": 100, "b": 180, "c": 250, "d": 120}.items())}
    for rid in ("a", "b", "c", "d"):   # buckets 128, 192, 256, then 128 again: captured anew, 192 has gone by then
        run.step({rid: toks[rid]})
        assert len(runner.portion_graphs) <= 2
    assert [k[0] for k in runner.portion_graphs] == [256, 128] and runner.portion_graph_steps == 4
    for rid in toks:
        places, got = run.of(rid)
        exact = plain.all_position_logits(config, weights, toks[rid])
        rounded = plain.all_position_logits(config, weights, toks[rid], rnd=plain.to_bfloat16_and_back)
        check(got, (exact[places], rounded[places]), "bfloat16", f"B {rid}")


def test_graphs_captured_ahead_are_the_ones_the_steps_then_replay(sharp_dirs):
    folder = sharp_dirs["A"]
    eng, runner, cache = runner_for(folder, "A", "bfloat16")
    made = eng.capture_graphs_ahead(decode_batches=(1, 3), prompt_tokens=(100, 300), max_ctx=1024)
    assert made == 4 and set(runner.graphs) == {(1, True, 1024), (4, True, 1024)}
    assert {k[0] for k in runner.portion_graphs} == {128, 384}
    assert eng.capture_graphs_ahead(decode_batches=(1, 3), prompt_tokens=(100, 300), max_ctx=1024) == 0
    from clockwork_b200.sampling import SamplingParams
    prompts = [tokens_for("A", 100, salt=5), tokens_for("A", 90, salt=6), tokens_for("A", 110, salt=7)]
    outs = eng.generate(prompts[:1], SamplingParams(max_tokens=4, ignore_eos=True))   # one prompt, then single-token steps of one
    assert len(outs[0].token_ids) == 4 and len(runner.portion_graphs) == 2 and len(runner.graphs) == 2
    assert runner.portion_graph_steps == 1


def test_a_long_prompt_under_a_small_token_budget_through_the_engine(sharp_dirs):
    """The scheduler reserves the pages of a whole prompt when it admits it, so the first portions of a long
    prompt run in a captured step whose context bound (and block-table width) is far below the request's
    table; beside it a short request decodes.  Greedy tokens against the plain implementation."""
    from clockwork_b200.sampling import SamplingParams
    from tests.test_engine_gpu import assert_greedy

    folder = sharp_dirs["B"]
    page = TINY["B"][2]
    cfg = EngineConfig.defaults(str(folder), dtype="bfloat16", block_size=page, num_blocks=600, max_model_len=2048, max_num_seqs=4,
                                max_num_batched_tokens=192, enable_prefix_cache=False)
    eng = LLMEngine(cfg, model=load_model(folder, cfg.model.dtype))
    prompts = [tokens_for("B", 1500, salt=91), tokens_for("B", 40, salt=92)]
    outs = eng.generate(prompts, [SamplingParams(max_tokens=6, ignore_eos=True), SamplingParams(max_tokens=30, ignore_eos=True)])
    assert eng.runner.portion_graph_steps >= 8 and {k[3] for k in eng.runner.portion_graphs} >= {1024, 2048}
    plain_model = plain.read_model_dir(folder)
    for prompt, out in zip(prompts, outs):
        assert_greedy(plain_model, prompt, list(out.token_ids), exact=False)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_compositions_of_steps(seed, dtype, sharp_dirs):
    """Seven requests of lengths that sit on and beside page and tile edges, at most four live, every step
    a random choice of who takes part and with how many tokens (one, a few, a hundred), requests joining
    and leaving in between: every position's logits against the plain implementation (float64 for the
    float32 run: at these lengths float32 sums alone move the sharpened model's logits by 1e-5)."""
    import random

    name = "B"
    folder = sharp_dirs[name]
    config, weights = plain.read_model_dir(folder)
    if dtype == "float32":
        weights64 = {k: v.double() for k, v in weights.items()}
    rng = random.Random(seed)
    _eng, runner, cache = runner_for(folder, name, dtype, max_model_len=1024, seqs=8)
    total = {f"q{i}": tokens_for(name, rng.choice([1, 3, 17, 64, 65, 130, 257, 400]), salt=seed * 10 + i) for i in range(7)}
    run = Replayed(runner, cache)
    waiting, live = list(total), {}
    while waiting or live:
        while waiting and len(live) < 4 and rng.random() < 0.6:
            live[waiting.pop()] = 0
        portions = {}
        for rid in list(live):
            if rng.random() < 0.2:
                continue  # sits this step out
            n = min(len(total[rid]) - live[rid], rng.choice([1, 1, 1, 2, 3, 8, 16, 33, 64, 128, 200]))
            portions[rid] = total[rid][live[rid] : live[rid] + n]
        if not portions:
            continue
        run.step(portions)
        for rid, toks in portions.items():
            live[rid] += len(toks)
            if live[rid] == len(total[rid]):
                cache.close(rid)
                del live[rid]
    for rid, toks in total.items():
        _places, got = run.of(rid)
        if dtype == "float32":
            exact = plain.all_position_logits(config, weights64, toks).float()
            check(got, (exact, exact), dtype, f"{name} {dtype} seed {seed} {rid}")
        else:
            exact = plain.all_position_logits(config, weights, toks)
            rounded = plain.all_position_logits(config, weights, toks, rnd=plain.to_bfloat16_and_back)
            check(got, (exact, rounded), dtype, f"{name} {dtype} seed {seed} {rid}")
    if dtype == "bfloat16":
        assert runner.portion_graph_steps > 3


def test_float32_steps_and_uncaptured_engines_take_the_plain_step(sharp_dirs):
    folder = sharp_dirs["A"]
    for dtype, graphs in (("float32", True), ("bfloat16", False)):
        _eng, runner, cache = runner_for(folder, "A", dtype, graphs=graphs)
        assert not runner.portions_captured
        run = Replayed(runner, cache)
        run.step({"a": tokens_for("A", 40, salt=3)})
        assert runner.portion_graph_steps == 0 and not runner.portion_graphs
