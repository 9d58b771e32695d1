"""Trace replay of a third, still small configuration with the head size of the real model (128) and
contexts of more than a thousand tokens, so that the kernels the product path takes at that size run
inside the engine and are compared with the plain implementation: the tcgen05 prefill attention over
many key tiles (with long rows of keys cut into parts, since the few work items leave SMs idle),
decode attention with its context splits and fused rotation, decoded tokens riding in a step beside
another request's prompt portion, and the tensor-core products with their split norm.  The tiny
configurations (head sizes 16 and 32) never reach those kernels."""

import json

import pytest
import torch

from tests.plain import qwen2_plain as plain
from tests.test_replay_gpu import check
from tests.trace_tools import TraceBuilder, cut, round_up, run_trace

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 384, "vocab_size": 512, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 4096,
    "hidden_act": "silu", "use_sliding_window": False,
}
PAGE = 16


def tokens(n: int, salt: int) -> list[int]:
    state, out = (2654435761 * (salt + 1) + 97 * n) & 0x7FFFFFFF, []
    for _ in range(n):
        state = (1103515245 * state + 12345) & 0x7FFFFFFF
        out.append((state >> 8) % CONFIG["vocab_size"])
    return out


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    """Random weights with the q and k projections scaled up, so that attention is peaked and a key
    that is missed, misplaced or weighted wrongly in a merge moves the logits beyond the tolerance."""
    from clockwork_b200.weights import save_safetensors, write_random_model

    plain_dir = write_random_model(tmp_path_factory.mktemp("head128"), CONFIG, seed=5)
    config, weights = plain.read_model_dir(plain_dir, dtype=torch.float32)
    sharp = {k: ((w * 6.0) if (".q_proj." in k or ".k_proj." in k) else w).to(torch.bfloat16) for k, w in weights.items()}
    target = tmp_path_factory.mktemp("head128_sharp")
    (target / "config.json").write_text(json.dumps(config))
    save_safetensors(target / "model.safetensors", sharp)
    return target


@pytest.fixture(scope="module")
def references(model_dir):
    """(exact, rounded as a bfloat16 run stores activations).  The exact logits are computed in float64:
    over 1,500 tokens of peaked attention the plain implementation's own float32 rounding reaches the
    1e-5 that the float32 engine is held to, and the gate is against the exact result."""
    config, weights = plain.read_model_dir(model_dir)
    weights64 = {k: v.double() for k, v in weights.items()}

    def get(toks):
        return (plain.all_position_logits(config, weights64, toks).float(),
                plain.all_position_logits(config, weights, toks, rnd=plain.to_bfloat16_and_back))

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_contexts_at_head_size_128(dtype, model_dir, references, tmp_path):
    from clockwork_b200.ops import attention_fast

    a, b = tokens(1500, 1), tokens(700, 2)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert attention_fast.prefill_tc_takes(CONFIG["head_dim"], PAGE)
    words = attention_fast.prefill_work_items([1300], [1300], CONFIG["num_attention_heads"], sms)[2]
    assert max(w & 0xFF for w in words) > 1  # the first step's long rows of keys are cut
    tb = TraceBuilder()
    tb.step([("a", a[:1300], True)])                          # many key tiles, few work items: cut rows
    tb.step([("a", a[1300:1468], True), ("b", b[:300], True)])  # a portion deep in a context beside a new prompt
    portions = cut(b[300:], [70, 2, 129, 40, 3, 17])
    assert len(portions) < 32
    for i, t in enumerate(a[1468:]):                          # 32 decoded tokens, b's portions riding along at first
        step, end = [("a", [t], True)], []
        if i < len(portions):
            step.append(("b", portions[i], True))
            if i == len(portions) - 1:
                end.append("b")
        if i == 31:
            end.append("a")
        tb.step(step, end=end)
    out = run_trace(model_dir, dtype, round_up(1500, 64) + round_up(700, 64), tb.steps, tmp_path / "out",
                    CONFIG["vocab_size"], PAGE)
    check(tb.gather(out, "a", len(a)), references(a), dtype, f"head size 128, {dtype}, the long request")
    check(tb.gather(out, "b", len(b)), references(b), dtype, f"head size 128, {dtype}, the request beside it")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_at_4400_tokens_beside_a_short_request(dtype, model_dir, references, tmp_path):
    """A context long enough that the captured decode step of the 8,192-token tier cuts it into many
    splits (merged in rounds), fetches its tiles by TMA and sizes its page list by the bound on the
    split, decoded beside a request of a few hundred tokens whose rows ride in the same graph."""
    a, b = tokens(4440, 3), tokens(260, 4)
    tb = TraceBuilder()
    tb.step([("a", a[:2048], False)])
    tb.step([("a", a[2048:4096], False)])
    tb.step([("a", a[4096:4400], True), ("b", b[:220], True)])
    for i in range(40):
        tb.step([("a", [a[4400 + i]], True), ("b", [b[220 + i]], True)], end=["a", "b"] if i == 39 else [])
    out = run_trace(model_dir, dtype, round_up(4440, 64) + round_up(260, 64), tb.steps, tmp_path / "out",
                    CONFIG["vocab_size"], PAGE)
    exact, rounded = references(a)
    check(tb.gather(out, "a", len(a), first=4096), (exact[4096:], rounded[4096:]), dtype, f"head size 128, {dtype}, 4,400 tokens")
    check(tb.gather(out, "b", len(b)), references(b), dtype, f"head size 128, {dtype}, the short request beside them")


@pytest.mark.parametrize("dtype,seed", [("bfloat16", 0), ("bfloat16", 1), ("float32", 0)])
def test_random_compositions_of_steps_at_head_size_128(dtype, seed, model_dir, references):
    """Nine requests of 1 to 2,300 tokens, at most six live, every step a random choice of who takes part
    and with how many tokens (one, a few, a query tile, over a thousand), through the step function with
    its captured steps: logits at a few places of every portion against the plain implementation."""
    import random

    from clockwork_b200 import EngineConfig
    from clockwork_b200.engine import LLMEngine, StepEntry, load_model

    rng = random.Random(seed)
    cfg = EngineConfig.defaults(str(model_dir), dtype=dtype, block_size=PAGE, num_blocks=900, max_model_len=4096, max_num_seqs=12,
                                max_num_batched_tokens=8192, enable_prefix_cache=False)
    eng = LLMEngine(cfg, model=load_model(model_dir, cfg.model.dtype))
    runner, cache = eng.runner, eng.cache
    total = {f"q{i}": tokens(rng.choice([1, 5, 127, 128, 129, 300, 640, 1100, 1500, 2300]), seed * 20 + i) for i in range(9)}
    waiting, live = list(total), {}
    got = {rid: [] for rid in total}
    places = {rid: [] for rid in total}
    while waiting or live:
        while waiting and len(live) < 6 and rng.random() < 0.6:
            rid = waiting.pop()
            cache.open(rid)
            live[rid] = 0
        entries = []
        for rid in list(live):
            if rng.random() < 0.15:
                continue  # sits this step out
            n = min(len(total[rid]) - live[rid], rng.choice([1, 1, 1, 1, 2, 7, 16, 100, 128, 130, 400, 700, 1300]))
            entries.append(StepEntry(rid, total[rid][live[rid] : live[rid] + n], sorted(set(rng.sample(range(n), min(n, 3)) + [n - 1]))))
        if not entries:
            continue
        out = runner.step(entries).float().cpu()
        row = 0
        for e in entries:
            for w in e.want:
                got[e.request_id].append(out[row].clone())
                places[e.request_id].append(live[e.request_id] + w)
                row += 1
            live[e.request_id] += len(e.tokens)
            if live[e.request_id] == len(total[e.request_id]):
                cache.close(e.request_id)
                del live[e.request_id]
        runner.check_status()
    for rid, toks in total.items():
        exact, rounded = references(toks)
        check(torch.stack(got[rid]), (exact[places[rid]], rounded[places[rid]]), dtype, f"{dtype} seed {seed} {rid} ({len(toks)} tokens)")
    assert (runner.portion_graph_steps > 3) == (dtype == "bfloat16")


@pytest.mark.parametrize("captured", [True, False])
def test_portions_behind_a_long_context_with_rows_cut_for_even_rounds(captured, model_dir, references, monkeypatch):
    """More query tiles x heads than SMs, all with long rows of keys: the work list cuts the rows so that the
    rounds of CTAs come out even.  With four heads that takes more tokens than a step holds, so the policy is
    told of 20 SMs and of parts that cost nothing; the cuts it then makes (three parts per row from the
    third portion on) go through the captured step's arrays of fixed length, or the uncaptured step's own,
    and the logits are held against the plain implementation."""
    from clockwork_b200 import EngineConfig
    from clockwork_b200.engine import LLMEngine, StepEntry, load_model
    from clockwork_b200.ops import attention_fast

    monkeypatch.setattr(attention_fast, "_sm_count", lambda device=None: 20)
    for name, value in (("ROUNDS_MIN_CTX", 1024), ("ROUNDS_CTA_TILES", 0), ("ROUNDS_MERGE_TILES", 0), ("ROUNDS_MIN_PART_TILES", 2)):
        monkeypatch.setattr(attention_fast, name, value)
    seen = []
    inner = attention_fast.prefill_work_items

    def spy(*args, **kwargs):
        result = inner(*args, **kwargs)
        seen.append((len(result[0]), max((w & 0xFF for w in result[2]), default=1)))
        return result

    monkeypatch.setattr(attention_fast, "prefill_work_items", spy)
    cfg = EngineConfig.defaults(str(model_dir), dtype="bfloat16", block_size=PAGE, num_blocks=300, max_model_len=4096, max_num_seqs=8,
                                max_num_batched_tokens=4096, enable_prefix_cache=False)
    eng = LLMEngine(cfg, model=load_model(model_dir, cfg.model.dtype))
    runner, cache = eng.runner, eng.cache
    runner.portions_captured = captured
    toks = tokens(4024, 77)
    cache.open("r")
    got, places, done = [], [], 0
    for n in (1024, 1024, 1024, 952):
        want = [0, 63, 64, 500, n - 1]
        out = runner.step([StepEntry("r", toks[done : done + n], want)]).float().cpu()
        runner.check_status()
        got += list(out)
        places += [done + w for w in want]
        done += n
    assert (runner.portion_graph_steps == 4) == captured
    assert max(parts for _, parts in seen) >= 3 and max(items for items, _ in seen) * CONFIG["num_attention_heads"] > 20, seen
    exact, rounded = references(toks)
    check(torch.stack(got), (exact[places], rounded[places]), "bfloat16", f"rows cut for even rounds, captured={captured}")
