"""Generation through the Python entry point and the command line against the plain
implementation: single and concurrent requests, portions under a token budget, prefix-cache hits,
preemption when pages run out, seeded sampling, finish rules, long decoding."""

import json
import subprocess
import sys

import pytest
import torch

from clockwork_b200 import EngineConfig
from clockwork_b200.engine import LLMEngine, load_model
from clockwork_b200.sampling import SamplingParams, uniform_for
from tests.plain import qwen2_plain as plain
from tests.tiny_configs import TINY, tokens_for
from tests.trace_tools import ROOT

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dirs(sharp_dirs):
    """Every test of this file runs the models with peaked attention (q and k projections scaled up):
    a key that is missed, misplaced or stale after a prefix hit, a preemption or a page's reuse then
    changes the tokens, which the nearly uniform softmax of plain random weights would hide."""
    return sharp_dirs


@pytest.fixture(scope="module")
def models(model_dirs):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = load_model(model_dirs[name], dtype)
        return cache[(name, dtype)]

    return get


@pytest.fixture(scope="module")
def plain_models(model_dirs):
    return {name: plain.read_model_dir(folder) for name, folder in model_dirs.items()}


def engine(models, model_dirs, name, dtype="float32", **overrides):
    page = TINY[name][2]
    defaults = dict(dtype=dtype, block_size=page, num_blocks=128, max_model_len=256, max_num_seqs=8,
                    max_num_batched_tokens=64)
    defaults.update(overrides)
    cfg = EngineConfig.defaults(str(model_dirs[name]), **defaults)
    return LLMEngine(cfg, model=models(name, cfg.model.dtype))


def assert_greedy(plain_model, prompt, tokens, exact):
    """float32: the engine's tokens are the plain implementation's.  bfloat16: every token is, given
    the engine's own history, within rounding of the plain implementation's best, where "rounding" is
    measured on this very sequence: the plain implementation run once more with its activations
    rounded to bfloat16 where a bfloat16 run stores them moves the logits by at most ``yard``; the
    engine's logits may be off by 2.5 times that (the bound of the replay tests), so the token it
    picks may lie at most twice that below the best (a near-tie may fall either way)."""
    config, weights = plain_model
    if exact:
        assert tokens == plain.greedy_generate(config, weights, prompt, len(tokens))
        return
    logits = plain.all_position_logits(config, weights, prompt + tokens)
    rounded = plain.all_position_logits(config, weights, prompt + tokens, rnd=plain.to_bfloat16_and_back)
    yard = float((rounded - logits).abs().max())
    for i, token in enumerate(tokens):
        row = logits[len(prompt) + i - 1]
        gap = float(row.max() - row[token])
        assert gap <= 2 * 2.5 * yard, f"token {i}: {token} is {gap:.4f} below the best (rounding moves logits by {yard:.4f})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_greedy_generate(name, dtype, models, model_dirs, plain_models):
    eng = engine(models, model_dirs, name, dtype)
    prompts = [tokens_for(name, n, salt=n) for n in (5, 11, 17, 1)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.prompt_token_ids for o in outs] == prompts
    for prompt, out in zip(prompts, outs):
        assert out.finished and out.finish_reason == "length" and out.num_generated_tokens == 8
        assert_greedy(plain_models[name], prompt, out.token_ids, exact=dtype == "float32")
    assert not eng.has_unfinished_requests() and eng.cache.requests == {}
    eng.cache.check_invariants(eng.prefix_cache.references())


def test_concurrent_requests_staggered_under_a_small_budget(models, model_dirs, plain_models):
    """Eight requests admitted over several steps with a token budget of 32: each equals the prompt
    run alone (after the reference's tests/test_llm_engine.py:94-131)."""
    name = "A"
    eng = engine(models, model_dirs, name, max_num_batched_tokens=32, enable_prefix_cache=False)
    prompts = [tokens_for(name, n, salt=i) for i, n in enumerate((21, 6, 33, 9, 14, 40, 3, 27))]
    params = SamplingParams(max_tokens=10, ignore_eos=True)
    finals = {}
    pending = list(enumerate(prompts))
    steps = 0
    while pending or eng.has_unfinished_requests():
        for _ in range(2):
            if pending:
                i, p = pending.pop(0)
                eng.add_request(f"req-{i}", prompt_token_ids=p, sampling_params=params)
        for out in eng.step():
            if out.finished:
                finals[out.request_id] = out
        steps += 1
        assert steps < 200
    config, weights = plain_models[name]
    for i, p in enumerate(prompts):
        assert finals[f"req-{i}"].token_ids == plain.greedy_generate(config, weights, p, 10)
    assert eng.stats()["num_scheduled_batches"] == steps and eng.stats()["num_free_blocks"] == 128


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_portions_of_seven_tokens(dtype, models, model_dirs, plain_models):
    name = "B"
    eng = engine(models, model_dirs, name, dtype, prefill_chunk_size=7)
    prompts = [tokens_for(name, n, salt=3 * n) for n in (1, 9, 23, 40)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert_greedy(plain_models[name], prompt, out.token_ids, exact=dtype == "float32")
    assert eng.stats()["num_scheduled_batches"] == 6 + 11  # six portions of the longest prompt, then 11 decodes


def test_prefix_cache_hits_and_shared_prefixes(models, model_dirs, plain_models):
    """A second pass over the same prompts is served from the prefix cache with identical tokens and
    exact cached-token accounting; three prompts sharing 16 tokens hit 16 each
    (after tests/test_llm_engine.py:134-200)."""
    name = "B"  # page size 8
    eng = engine(models, model_dirs, name)
    prompts = [tokens_for(name, n, salt=n) for n in (23, 40, 9)]
    params = SamplingParams(max_tokens=6, ignore_eos=True)
    first = eng.generate(prompts, params)
    assert [o.num_cached_tokens for o in first] == [0, 0, 0]
    second = eng.generate(prompts, params)
    assert [o.token_ids for o in second] == [o.token_ids for o in first]
    assert [o.num_cached_tokens for o in second] == [16, 32, 8]  # whole pages, never the whole prompt
    shared = tokens_for(name, 16, salt=99)
    family = [shared + tokens_for(name, n, salt=50 + n) for n in (5, 9, 13, 2)]
    outs = eng.generate(family[:1], params) + eng.generate(family[1:], params)
    assert [o.num_cached_tokens for o in outs] == [0, 16, 16, 16]
    off = engine(models, model_dirs, name, enable_prefix_cache=False)
    assert [o.token_ids for o in off.generate(family, params)] == [o.token_ids for o in outs]
    config, weights = plain_models[name]
    assert outs[2].token_ids == plain.greedy_generate(config, weights, family[2], 6)
    stats = eng.stats()
    assert stats["prefix_cache_hit_tokens"] == 16 + 32 + 8 + 48 and stats["total_cached_tokens"] == 104
    eng.cache.check_invariants(eng.prefix_cache.references())


def test_pages_run_out_preemption_keeps_outputs_exact(models, model_dirs, plain_models):
    """Eight pages of four tokens, three sequences growing to 16 tokens: preemption by recompute
    happens and the outputs stay exact (after tests/test_llm_engine.py:203-219)."""
    name = "A"
    eng = engine(models, model_dirs, name, num_blocks=8, watermark=0.0, enable_prefix_cache=False)
    prompts = [tokens_for(name, 4, salt=i) for i in range(3)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert eng.stats()["num_preempted_total"] >= 1
    config, weights = plain_models[name]
    for prompt, out in zip(prompts, outs):
        assert out.token_ids == plain.greedy_generate(config, weights, prompt, 12)
    assert eng.stats()["num_free_blocks"] == 8


def test_preemption_by_recompute_in_bfloat16(models, model_dirs, plain_models):
    """The same shortage of pages in bfloat16: sequences are preempted, recomputed from their tokens
    and finish; each token is within rounding of the plain implementation's best given the sequence's
    own history, and every page comes back."""
    name = "B"  # pages of 8 tokens
    eng = engine(models, model_dirs, name, "bfloat16", num_blocks=7, watermark=0.0, enable_prefix_cache=False)
    prompts = [tokens_for(name, 8, salt=20 + i) for i in range(3)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))
    assert eng.stats()["num_preempted_total"] >= 1
    for prompt, out in zip(prompts, outs):
        assert out.num_generated_tokens == 20
        assert_greedy(plain_models[name], prompt, out.token_ids, exact=False)
    assert eng.stats()["num_free_blocks"] == 7 and eng.cache.requests == {}


def test_a_request_that_can_never_fit_is_an_error(models, model_dirs):
    eng = engine(models, model_dirs, "A", num_blocks=4, watermark=0.0)
    eng.add_request("big", prompt_token_ids=tokens_for("A", 30))
    with pytest.raises(RuntimeError, match="cannot be admitted"):
        eng.step()


def test_seeded_sampling(models, model_dirs, plain_models):
    """Temperature / top-k / top-p sampling is reproducible across engines, differs between seeds,
    and equals the plain rule given the same uniform numbers (after tests/test_llm_engine.py:222-236)."""
    name = "B"
    prompts = [tokens_for(name, n, salt=n) for n in (9, 23, 2)]

    def run(seed, **kw):
        eng = engine(models, model_dirs, name, **kw)
        params = SamplingParams(max_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=seed, ignore_eos=True)
        return [o.token_ids for o in eng.generate(prompts, params)]

    a, b, c = run(1), run(1, max_num_batched_tokens=8, prefill_chunk_size=5), run(2)
    assert a == b and a != c
    config, weights = plain_models[name]
    for prompt, tokens in zip(prompts, a):
        logits = plain.all_position_logits(config, weights, prompt + tokens)
        for i, token in enumerate(tokens):
            want = plain.sample_with_uniform(logits[len(prompt) + i - 1], 0.8, 40, 0.95, uniform_for(1, i))
            assert token == want
    plain_temp = engine(models, model_dirs, name).generate(prompts[:1], SamplingParams(max_tokens=5, temperature=0.8, seed=7))
    assert len(plain_temp[0].token_ids) == 5


def test_finish_rules(models, model_dirs, plain_models):
    """EOS, stop ids, ignore_eos, max_tokens, max_model_len (after tests/test_llm_engine.py:239-296)."""
    name = "A"
    config, weights = plain_models[name]
    prompt = tokens_for(name, 7, salt=1)
    free_run = plain.greedy_generate(config, weights, prompt, 10)
    stop_at = free_run[4]
    cut = free_run.index(stop_at) + 1
    eng = engine(models, model_dirs, name)
    out = eng.generate([prompt], SamplingParams(max_tokens=10, stop_token_ids=[stop_at]))[0]
    assert out.finish_reason == "stop" and out.token_ids == free_run[:cut]  # the stopping token is kept
    eng._eos = frozenset({stop_at})
    out = eng.generate([prompt], SamplingParams(max_tokens=10))[0]
    assert out.finish_reason == "stop" and out.token_ids == free_run[:cut]
    out = eng.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0]
    assert out.finish_reason == "length" and out.token_ids == free_run
    short = engine(models, model_dirs, name, max_model_len=12)
    out = short.generate([prompt], SamplingParams(max_tokens=50, ignore_eos=True))[0]
    assert out.finish_reason == "length" and len(prompt) + len(out.token_ids) == 12
    with pytest.raises(ValueError, match="leaves no room"):
        short.add_request("x", prompt_token_ids=list(range(12)))
    with pytest.raises(ValueError, match="exactly one"):
        eng.add_request("x")
    with pytest.raises(ValueError, match="at least one token"):
        eng.add_request("x", prompt_token_ids=[])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        eng.add_request("x", prompt_token_ids=[1, 256])
    eng.add_request("dup", prompt_token_ids=[1, 2])
    with pytest.raises(ValueError, match="already active"):
        eng.add_request("dup", prompt_token_ids=[1, 2])
    eng.abort_request("dup")
    assert not eng.has_unfinished_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_many_pages(dtype, models, model_dirs, plain_models):
    name = "B"
    eng = engine(models, model_dirs, name, dtype, max_model_len=512)
    prompt = tokens_for(name, 9, salt=5)
    out = eng.generate([prompt], SamplingParams(max_tokens=200, ignore_eos=True))[0]
    assert out.num_generated_tokens == 200
    assert_greedy(plain_models[name], prompt, out.token_ids, exact=dtype == "float32")


def test_command_line(model_dirs, plain_models, tmp_path):
    name = "A"
    prompt = tokens_for(name, 6, salt=2)
    profile = tmp_path / "profile.yaml"
    profile.write_text(
        f"model:\n  model: {model_dirs[name]}\n  dtype: float32\n  max_model_len: 128\n"
        "cache:\n  block_size: 4\n  num_blocks: 64\nscheduler:\n  max_num_seqs: 4\n  max_num_batched_tokens: 16\n"
    )
    cmd = [sys.executable, "-m", "clockwork_b200", "generate", "--config", str(profile), "--set", "num_blocks=32",
           "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--ignore-eos", "--stats"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    config, weights = plain_models[name]
    assert record["token_ids"] == plain.greedy_generate(config, weights, prompt, 5)
    # 32 pages by --set; the prompt's one whole page stays in the prefix cache
    assert json.loads(proc.stderr.strip().splitlines()[-1])["num_free_blocks"] == 31
    bad = subprocess.run(cmd[:6] + ["--set", "no_such=1"] + cmd[8:], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert bad.returncode != 0 and "unknown config override" in bad.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_graphs_change_nothing(dtype, models, model_dirs):
    """Steps in which every request decodes one token replay a captured CUDA graph (padded to a
    batch-size bucket); the tokens must be those of the uncaptured step function, greedy and sampled,
    while requests join, leave and change rows."""
    name = "B"
    prompts = [tokens_for(name, n, salt=7 * n) for n in (3, 30, 11, 19, 8)]
    params = [SamplingParams(max_tokens=m, temperature=t, top_k=k, seed=s, ignore_eos=True)
              for m, t, k, s in ((9, 0.0, -1, None), (25, 0.9, 20, 3), (14, 0.0, -1, None), (6, 1.2, -1, 4), (30, 0.0, -1, None))]
    runs = []
    for graphs in (True, False):
        eng = engine(models, model_dirs, name, dtype, cuda_graphs=graphs, max_num_seqs=5)
        assert eng.uses_graphs == graphs
        runs.append([o.token_ids for o in eng.generate(prompts, params)])
        if graphs:
            assert eng.runner.graphs and eng.runner.graph_kernel_launches > 0
    assert runs[0] == runs[1]
    greedy_only = engine(models, model_dirs, name, dtype, max_num_seqs=3)
    outs = greedy_only.generate(prompts[:3], SamplingParams(max_tokens=5, ignore_eos=True))
    # greedy requests do not depend on what else is in the batch: the same first tokens as above
    # (in float32 exactly; in bfloat16 the split of a product may differ with the batch, only its rounding)
    if dtype == "float32":
        assert [outs[i].token_ids for i in (0, 2)] == [runs[0][i][:5] for i in (0, 2)]  # (the second was sampled above)
    assert all(len(o.token_ids) == 5 for o in outs)
    assert {key[1] for key in greedy_only.runner.graphs} == {True}  # only the greedy graphs were captured


def test_a_wait_that_gave_up_in_a_product_kernel_stops_generation(models, model_dirs):
    """The tensor-core products report a device-side wait that ran out into the same status word as
    every other kernel of a step, and the engine reads that word: generation stops with an error
    instead of going on with a tile that was never written.  (The word is set by hand here; nothing
    is made to hang.)"""
    from clockwork_b200 import ops
    from clockwork_b200.ops import gemm_tc

    eng = engine(models, model_dirs, "B", "bfloat16")
    assert gemm_tc.status("cuda:0").data_ptr() == eng.runner.status.data_ptr() == ops.device_status("cuda:0").data_ptr()
    eng.add_request("r", prompt_token_ids=tokens_for("B", 9, 1), sampling_params=SamplingParams(max_tokens=40, ignore_eos=True))
    eng.step()
    gemm_tc.status("cuda:0").copy_(torch.tensor([4, 2, 1, 0], dtype=torch.int32))  # CW_ST_WAIT_TIMEOUT as a kernel writes it
    with pytest.raises(RuntimeError, match="device-side wait ran out"):
        for _ in range(3):  # (the words travel to the host with every step's tokens)
            eng.step()
    eng.abort_request("r")


def test_steps_run_ahead_change_nothing(models, model_dirs):
    """A step in which every request decodes is launched before the tokens of the step before it have
    been read (its inputs come from the requests' state on the device); a sequence that ends by a stop
    token has then computed a token too many, which is dropped; a request that arrives and an abort end
    the running ahead.  Same tokens with and without, sampling and stop tokens included."""
    def run(run_ahead, stop_id=None):
        eng = engine(models, model_dirs, "B", max_num_seqs=5, max_num_batched_tokens=32, max_model_len=96)
        eng.run_ahead = run_ahead
        got = {}
        eng.add_request("greedy", prompt_token_ids=tokens_for("B", 9, 1), sampling_params=SamplingParams(max_tokens=30, ignore_eos=True))
        eng.add_request("short", prompt_token_ids=tokens_for("B", 5, 2), sampling_params=SamplingParams(max_tokens=7, ignore_eos=True))
        eng.add_request("sampled", prompt_token_ids=tokens_for("B", 12, 3),
                        sampling_params=SamplingParams(max_tokens=25, temperature=0.9, top_k=20, seed=7, ignore_eos=True))
        eng.add_request("gone", prompt_token_ids=tokens_for("B", 6, 4), sampling_params=SamplingParams(max_tokens=40, ignore_eos=True))
        if stop_id is not None:  # the first request once more, ended by one of its own tokens
            eng.add_request("stopped", prompt_token_ids=tokens_for("B", 9, 1),
                            sampling_params=SamplingParams(max_tokens=30, stop_token_ids=[stop_id], ignore_eos=True))
        steps = 0
        while eng.has_unfinished_requests():
            for out in eng.step():
                got[out.request_id] = (list(out.token_ids), out.finish_reason)
            steps += 1
            if steps == 12:
                eng.abort_request("gone")
            if steps == 15:
                eng.add_request("late", prompt_token_ids=tokens_for("B", 7, 5), sampling_params=SamplingParams(max_tokens=9, ignore_eos=True))
        assert eng.cache.requests == {} and eng.cache.state.num_free == eng.cache.state.num_slots
        eng.cache.check_invariants(eng.prefix_cache.references())
        return got, eng.steps_run_ahead

    plain_run, none_ahead = run(False)
    stop_id = plain_run["greedy"][0][5]
    ahead, count = run(True, stop_id)
    behind, none_ahead_2 = run(False, stop_id)
    assert count > 10 and none_ahead == 0 and none_ahead_2 == 0
    assert ahead == behind
    tokens, reason = ahead["stopped"]
    assert reason == "stop" and tokens[-1] == stop_id and tokens == plain_run["greedy"][0][: len(tokens)] and len(tokens) <= 6
    assert {k: v for k, v in ahead.items() if k != "stopped"} == plain_run


@pytest.mark.parametrize("seed", [1, 2])
def test_a_random_churn_of_requests(seed, models, model_dirs, plain_models):
    """Ninety requests of random lengths (one token to more than a thousand, some behind a shared prefix),
    random limits and every kind of sampling, added a few at a time while others run, in a pool small
    enough that requests are preempted now and then, with the prefix cache and the captured steps on:
    every request finishes with as many tokens as it asked for, no kernel reports anything, every page and
    state slot comes back, and the greedy requests' tokens are within rounding of the plain
    implementation's best."""
    import random

    name = "B"
    rng = random.Random(seed)
    eng = engine(models, model_dirs, name, "bfloat16", num_blocks=330, max_model_len=2048, max_num_seqs=12,
                 max_num_batched_tokens=320, enable_prefix_cache=True)
    vocab = TINY[name][0]["vocab_size"]
    shared = [rng.randrange(vocab) for _ in range(300)]
    pending, asked, prompts = [], {}, {}
    for i in range(90):
        n = rng.choice([1, 2, 7, 30, 100, 129, 200, 513, 700, 1100])
        prompt = shared[: rng.choice([0, 0, 80, 300])] + [rng.randrange(vocab) for _ in range(n)]
        kind = rng.choice([dict(temperature=0.0), dict(temperature=0.0), dict(temperature=0.8, seed=i), dict(temperature=1.0, top_k=20, seed=i),
                           dict(temperature=0.7, top_p=0.9, seed=i), dict(temperature=0.9, top_k=50, top_p=0.95, seed=i)])
        limit = rng.choice([1, 2, 8, 40])
        pending.append((f"r{i}", prompt, SamplingParams(max_tokens=limit, ignore_eos=True, **kind)))
        asked[f"r{i}"], prompts[f"r{i}"] = (limit, kind["temperature"] == 0.0), prompt
    done = {}
    while pending or eng.has_unfinished_requests():
        for _ in range(rng.choice([0, 0, 1, 3])):
            if pending:
                rid, prompt, params = pending.pop()
                eng.add_request(rid, prompt_token_ids=prompt, sampling_params=params)
        for out in eng.step():
            if out.finished:
                done[out.request_id] = list(out.token_ids)
    eng.runner.check_status()
    assert set(done) == set(asked) and all(len(done[rid]) == asked[rid][0] for rid in asked)
    assert eng.cache.requests == {} and eng.cache.state.num_free == 12
    assert eng.runner.portion_graph_steps > 20 and eng.runner.graphs
    greedy = [rid for rid in sorted(asked) if asked[rid][1] and len(prompts[rid]) <= 400][:5]
    for rid in greedy:
        assert_greedy(plain_models[name], prompts[rid], done[rid], exact=False)
