"""The plain implementation against the reference's own model code, through the outputs that
tests/golden/make_golden.py stored (and against the reference directly when its checkout is present)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from tests.golden.make_golden import GREEDY_NEW, GREEDY_PROMPT, weight_checksum
from tests.plain import qwen2_plain as plain
from tests.tiny_configs import TINY

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", sorted(TINY))
def test_plain_matches_golden(name, tiny_dirs):
    gold = np.load(GOLDEN / f"tiny_{name.lower()}.npz")
    config, weights = plain.read_model_dir(tiny_dirs[name])
    assert weight_checksum(weights) == pytest.approx(float(gold["checksum"]), rel=1e-12), "weights differ from the golden run's"
    tokens = gold["tokens"].tolist()
    logits = plain.all_position_logits(config, weights, tokens)
    torch.testing.assert_close(logits, torch.from_numpy(gold["logits"]), rtol=1e-5, atol=1e-5)
    assert plain.greedy_generate(config, weights, tokens[:GREEDY_PROMPT], GREEDY_NEW) == gold["greedy"].tolist()


def test_negative_control(tiny_dirs):
    """A 1e-3 change of one weight must break the 1e-5 match (after the reference's
    tests/test_hf_equivalence.py:141-153), so the gate is not vacuous."""
    gold = np.load(GOLDEN / "tiny_a.npz")
    config, weights = plain.read_model_dir(tiny_dirs["A"])
    # (a v_proj weight: with N(0, 0.02) weights attention is nearly uniform and a q_proj change
    # of 1e-3 moves the logits by only 4e-6)
    weights["model.layers.0.self_attn.v_proj.weight"][0, 0] += 1e-3
    logits = plain.all_position_logits(config, weights, gold["tokens"].tolist())
    assert not torch.allclose(logits, torch.from_numpy(gold["logits"]), rtol=1e-5, atol=1e-5)


def test_plain_parts():
    x = torch.randn(5, 8)
    w = torch.rand(8) + 0.5
    y = plain.rms_norm(x, w, 1e-6)
    torch.testing.assert_close(y, w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6))
    cos, sin = plain.rope_cos_sin(torch.tensor([0, 3]), 8, 100.0, torch.float32)
    assert torch.allclose(cos[0], torch.ones(8)) and torch.allclose(sin[0], torch.zeros(8))
    q = torch.randn(2, 3, 8)
    r = plain.apply_rope(q, cos, sin)
    torch.testing.assert_close(r.norm(dim=-1), q.norm(dim=-1))  # a rotation
    # causal: the first query sees only the first key
    q, k, v = torch.randn(4, 2, 8), torch.randn(4, 1, 8), torch.randn(4, 1, 8)
    out = plain.causal_attention(q, k, v, 0.3)
    torch.testing.assert_close(out[0, 0], v[0, 0])
    # a window of one sees only itself
    out = plain.causal_attention(q, k, v, 0.3, window=1)
    torch.testing.assert_close(out[:, 1], v[:, 0])
    # decoding one token against a longer context aligns the query with the context's end
    full = plain.causal_attention(q, k, v, 0.3)
    last = plain.causal_attention(q[3:], k, v, 0.3)
    torch.testing.assert_close(last[0], full[3])


def test_sampling_rules():
    logits = torch.tensor([1.0, 3.0, 2.0, 0.5])
    p = plain.sampling_probs(logits, 1.0, top_k=2)
    assert p[0] == 0 and p[3] == 0 and p[1] > p[2] > 0
    p = plain.sampling_probs(logits, 1.0, top_p=0.5)  # the token that crosses the threshold stays
    assert (p > 0).tolist() == [False, True, False, False]
    p = plain.sampling_probs(logits, 1.0, top_p=0.7)
    assert (p > 0).tolist() == [False, True, True, False]
    assert plain.sample_with_uniform(logits, 0.0, -1, 1.0, 0.9) == 1
    assert plain.sample_with_uniform(logits, 1.0, -1, 1.0, 0.0) == 0
    assert plain.sample_with_uniform(logits, 1.0, -1, 1.0, 0.999999) == 3


def test_plain_matches_reference_checkout_directly(tiny_dirs):
    import sys
    from types import SimpleNamespace

    from tests.tiny_configs import reference_checkout

    ref = str(reference_checkout())
    if not Path(ref, "clockwork/engine/model.py").is_file():
        pytest.skip("reference checkout not present")
    sys.path.insert(0, ref)
    try:
        from clockwork.engine.model import Qwen2ForCausalLM
    finally:
        sys.path.remove(ref)
    config, weights = plain.read_model_dir(tiny_dirs["B"])
    model = Qwen2ForCausalLM(SimpleNamespace(**config))
    model.load_state_dict(weights, strict=False)
    tokens = list(range(5, 30))
    with torch.inference_mode():
        want = model(torch.tensor(tokens), torch.arange(len(tokens)), None, None)  # last row
    got = plain.all_position_logits(config, weights, tokens)[-1:]
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
