"""Generality of the parts: a toy architecture defined in this file only — a mixer with a state of
fixed size per request, a windowed attention layer with pages of its own, and a run order that names
a layer twice and lets it read the cache it wrote the first time — is registered, written as a
random model folder, loaded, and stepped in several cuts and batches, without any change to the
framework's files.  It is a toy, not any real model."""

import pytest
import torch

from clockwork_b200.config import ExecStep, LayerSpec, ModelSpec, PartSpec, register_architecture
from clockwork_b200.engine import LLMEngine, ModelRunner, StepEntry, load_model
from clockwork_b200.cache import CacheManager
from clockwork_b200.parts import Mixer, SlotStateNeed, register_mixer
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights import TensorDecl, write_random_model
from clockwork_b200 import EngineConfig
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class DecayingSumMixer(Mixer):
    """state <- decay * state + x W_in (per token, in order); out = state W_out.  The state
    ([state_size] float32 per request) lives in the cache manager's fixed-size slots."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.h, self.d, self.decay = spec["hidden_size"], spec["state_size"], spec["decay"]

    def cache_need(self):
        return SlotStateNeed((self.d,))

    def tensor_decls(self):
        yield TensorDecl(self.name("w_in"), (self.d, self.h), "matrix", "linear")
        yield TensorDecl(self.name("w_out"), (self.h, self.d), "matrix", "linear")

    def load_weights(self, fetch):
        self.w_in, self.w_out = fetch(self.name("w_in")), fetch(self.name("w_out"))

    def forward(self, ctx, x, view, stream):
        u = x.float() @ self.w_in.float().T  # [N, d]
        out = torch.empty_like(u)
        start = 0
        for s, n in enumerate(ctx.q_lens_host):  # portions of a request arrive in order
            state = view.state[view.slots_host[s]]
            for t in range(start, start + n):
                state.mul_(self.decay).add_(u[t])
                out[t] = state
            start += n
        return (out @ self.w_out.float().T).to(self.dtype)  # a delta: the next norm adds it


class CapturedDecayingSumMixer(DecayingSumMixer):
    """The same mixer, able to run inside a captured single-token step: there it finds its rows through the
    view's device-side slot list (padding rows of the captured batch land in the scratch row) and uses no
    host-side list.  Steps with prompt portions take the loop above."""

    graph_safe = True

    def forward(self, ctx, x, view, stream):
        if not ctx.all_single_token:
            return super().forward(ctx, x, view, stream)
        u = x.float() @ self.w_in.float().T  # [S, d]: one token per request
        state = view.state.index_select(0, view.slots) * self.decay + u
        view.state.index_copy_(0, view.slots, state)
        return (state @ self.w_out.float().T).to(self.dtype)


class ToyArchitecture:
    name = "ToyStateLM"

    def parse_config(self, raw):
        return raw

    def model_spec(self, raw):
        h = raw["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]})
        ffn = PartSpec("swiglu", {"hidden_size": h, "intermediate_size": raw["ffn"]})

        def attention(window):
            return PartSpec("attention", dict(hidden_size=h, num_heads=4, num_kv_heads=2, head_dim=16, qkv_bias=False,
                                              o_bias=True, scale=0.3, window=window,
                                              position=PartSpec("rope_neox", {"theta": 100.0, "rotary_dim": 8})))

        mixers = [attention(None), PartSpec(raw.get("mixer_kind", "toy_decaying_sum"), dict(hidden_size=h, state_size=raw["state"], decay=0.9)),
                  attention(raw["window"])]
        layers = [LayerSpec("prenorm_residual", m, ffn, norm, norm, f"model.layers.{i}") for i, m in enumerate(mixers)]
        schedule = [ExecStep(0), ExecStep(1), ExecStep(2), ExecStep(0, cache_layer=0, write_cache=False)]
        return ModelSpec(self.name, raw["vocab_size"], h, layers, schedule, norm, tie_word_embeddings=True, raw=raw)


RAW = dict(architectures=["ToyStateLM"], hidden_size=48, vocab_size=90, eps=1e-5, ffn=72, state=20, window=6)


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    register_mixer("toy_decaying_sum", DecayingSumMixer, replace=True)
    register_mixer("toy_decaying_sum_captured", CapturedDecayingSumMixer, replace=True)
    register_architecture(ToyArchitecture(), replace=True)
    import json

    from clockwork_b200.weights import save_safetensors

    plain_dir = write_random_model(tmp_path_factory.mktemp("toy_flat"), RAW, seed=5)
    # peaked attention (q and k projections scaled up), so that the window's edge and the cache that the
    # last layer reads again matter: with plain random weights every softmax is nearly uniform
    config, weights = plain.read_model_dir(plain_dir, dtype=torch.float32)
    sharp = {k: ((w * 12.0) if (".q_proj." in k or ".k_proj." in k) else w).to(torch.bfloat16) for k, w in weights.items()}
    target = tmp_path_factory.mktemp("toy")
    (target / "config.json").write_text(json.dumps(config))
    save_safetensors(target / "model.safetensors", sharp)
    return target


def plain_toy_logits(folder, tokens, rnd=plain.exact):
    """The same model, whole sequence, no cache, from the plain implementation's functions.  ``rnd``
    rounds activations where a bfloat16 run stores them (the yardstick of the bfloat16 comparison)."""
    _, w = plain.read_model_dir(folder)
    t = len(tokens)
    positions = torch.arange(t)
    eps = RAW["eps"]

    def attention(x, prefix, window):
        q = rnd(x @ w[f"{prefix}.q_proj.weight"].T).view(t, 4, 16)
        k = rnd(x @ w[f"{prefix}.k_proj.weight"].T).view(t, 2, 16)
        v = rnd(x @ w[f"{prefix}.v_proj.weight"].T).view(t, 2, 16)
        cos, sin = plain.rope_cos_sin(positions, 8, 100.0, torch.float32)
        q = rnd(torch.cat([plain.apply_rope(q[..., :8], cos, sin), q[..., 8:]], dim=-1))
        k = rnd(torch.cat([plain.apply_rope(k[..., :8], cos, sin), k[..., 8:]], dim=-1))
        out = rnd(plain.causal_attention(q, k, v, 0.3, window=window))
        return out.reshape(t, 64) @ w[f"{prefix}.o_proj.weight"].T + w[f"{prefix}.o_proj.bias"], (k, v)

    def block(h, i, mixer):
        p = f"model.layers.{i}"
        h = h + mixer(rnd(plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)))
        return h + plain.swiglu_mlp(rnd(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)), w, f"{p}.mlp", rnd=rnd)

    kv0 = {}

    def first(x):
        out, kv0["kv"] = attention(x, "model.layers.0.self_attn", None)
        return out

    def decaying_sum(x):
        u = x @ w["model.layers.1.self_attn.w_in"].T
        state, rows = torch.zeros(RAW["state"]), []
        for row in u:
            state = 0.9 * state + row
            rows.append(state)
        return rnd(torch.stack(rows) @ w["model.layers.1.self_attn.w_out"].T)

    def again(x):  # layer 0's weights on new activations, but keys and values of its first run
        q = rnd(x @ w["model.layers.0.self_attn.q_proj.weight"].T).view(t, 4, 16)
        cos, sin = plain.rope_cos_sin(positions, 8, 100.0, torch.float32)
        q = rnd(torch.cat([plain.apply_rope(q[..., :8], cos, sin), q[..., 8:]], dim=-1))
        out = rnd(plain.causal_attention(q, *kv0["kv"], 0.3))
        return out.reshape(t, 64) @ w["model.layers.0.self_attn.o_proj.weight"].T + w["model.layers.0.self_attn.o_proj.bias"]

    h = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    h = block(h, 0, first)
    h = block(h, 1, decaying_sum)
    h = block(h, 2, lambda x: attention(x, "model.layers.2.self_attn", RAW["window"])[0])
    h = block(h, 0, again)
    return rnd(plain.rms_norm(h, w["model.norm.weight"], eps)) @ w["model.embed_tokens.weight"].T


def tokens(n, salt):
    return [(salt * 31 + i * i * 7 + i) % RAW["vocab_size"] for i in range(n)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_steps_like_its_plain_form(toy_dir, dtype):
    from tests.test_replay_gpu import check  # float32: 1e-5; bfloat16: 2.5 x what bfloat16 storage alone moves the logits

    model = load_model(toy_dir, dtype)
    needs = model.cache_needs()
    assert isinstance(needs[1], SlotStateNeed) and needs[2].window == 6 and needs[0].window is None
    cache = CacheManager(needs, num_pages=24, page_size=4, dtype=model.dtype, device=DEV, num_state_slots=3)
    assert [g.cache_layers for g in cache.groups] == [[0], [2]]  # the windowed layer has pages of its own
    runner = ModelRunner(model, cache)
    a, b = tokens(37, 1), tokens(22, 2)
    want_a = (plain_toy_logits(toy_dir, a), plain_toy_logits(toy_dir, a, rnd=plain.to_bfloat16_and_back))
    want_b = (plain_toy_logits(toy_dir, b), plain_toy_logits(toy_dir, b, rnd=plain.to_bfloat16_and_back))

    def run(plan):
        got = {"a": [], "b": []}
        pos = {"a": 0, "b": 0}
        data = {"a": a, "b": b}
        for step in plan:
            entries = []
            for rid, n in step.items():
                if rid not in cache.requests:
                    cache.open(rid)
                entries.append(StepEntry(rid, data[rid][pos[rid] : pos[rid] + n], list(range(n))))
                pos[rid] += n
            logits = runner.step(entries).cpu()
            runner.check_status()
            row = 0
            for rid, n in step.items():
                got[rid].append(logits[row : row + n])
                row += n
        for rid in list(cache.requests):
            cache.close(rid)
        cache.check_invariants()
        return {rid: torch.cat(rows) for rid, rows in got.items() if rows}

    whole = run([{"a": 37}, {"b": 22}])
    check(whole["a"].float(), want_a, dtype, f"toy {dtype} a whole")
    check(whole["b"].float(), want_b, dtype, f"toy {dtype} b whole")
    mixed = run([{"a": 9}, {"a": 2, "b": 13}, {"b": 1}, {"a": 20, "b": 1}, {"a": 1, "b": 7}, {"a": 5}])
    check(mixed["a"].float(), want_a, dtype, f"toy {dtype} a mixed")
    check(mixed["b"].float(), want_b, dtype, f"toy {dtype} b mixed")
    assert cache.num_free_pages() == [24, 24] and cache.state.num_free == 3


def test_toy_model_generates_through_the_engine(toy_dir):
    cfg = EngineConfig.defaults(str(toy_dir), dtype="float32", block_size=4, num_blocks=32, max_num_seqs=2,
                                max_num_batched_tokens=16, max_model_len=128)
    eng = LLMEngine(cfg)
    assert not eng.prefix_cache.enabled  # fixed-size state and windows cannot be shared by pages
    prompts = [tokens(19, 3), tokens(6, 4), tokens(11, 5)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=7, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for _ in range(7):
            ids.append(int(plain_toy_logits(toy_dir, ids)[-1].argmax()))
        assert out.token_ids == ids[len(prompt):]
    assert eng.cache.state.num_free == 2


def test_toy_model_with_state_runs_in_captured_steps(toy_dir, tmp_path):
    """A mixer with state of its own whose single-token path uses device-side data only is captured in the
    decode graphs like the framework's own parts (its state rows follow the requests' slots, padding rows
    use the scratch row), steps run ahead of the host, and the tokens are those of the plain form."""
    import json
    import shutil

    config = json.loads((toy_dir / "config.json").read_text())
    config["mixer_kind"] = "toy_decaying_sum_captured"
    (tmp_path / "config.json").write_text(json.dumps(config))
    shutil.copy(toy_dir / "model.safetensors", tmp_path / "model.safetensors")
    cfg = EngineConfig.defaults(str(tmp_path), dtype="float32", block_size=4, num_blocks=48, max_num_seqs=4,
                                max_num_batched_tokens=16, max_model_len=128)
    eng = LLMEngine(cfg)
    assert eng.uses_graphs and not eng.prefix_cache.enabled
    prompts = [tokens(19, 3), tokens(6, 4), tokens(11, 5)]
    outs = eng.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True) for n in (9, 14, 6)])
    assert eng.runner.graphs and eng.steps_run_ahead > 0
    # (its steps with prompt portions ran uncaptured: the toy mixer walks the step's host-side lists there
    # and does not declare ``graph_safe_portions``)
    assert not eng.runner.portions_captured and eng.runner.portion_graph_steps == 0
    for prompt, out in zip(prompts, outs):
        ids = list(prompt)
        for _ in range(out.num_generated_tokens):
            ids.append(int(plain_toy_logits(toy_dir, ids)[-1].argmax()))
        assert out.token_ids == ids[len(prompt):]
    assert eng.cache.state.num_free == 4 and eng.cache.requests == {}
