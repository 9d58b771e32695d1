"""Each part alone (norm, position encoding, attention mixer, feed-forward, block) against the
plain implementation's function for the same part, at sizes of its own, through the cache and in
two ways of cutting where the part has a cache."""

import pytest
import torch

from clockwork_b200.config import LayerSpec, PartSpec
from clockwork_b200.parts import ResidualStream, build_block, build_part
from tests.gpu_tools import DEV, PartHarness
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(rtol=1e-5, atol=1e-5 * scale) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2 * scale)


def close(got, want, dtype):
    """Elementwise, with the absolute part scaled by the size of the values compared."""
    torch.testing.assert_close(got, want, **tol(dtype, max(1.0, float(want.abs().max()))))


def weights(decls, dtype, seed=0, scale=None):
    """float32 CPU tensors for the declarations (rounded to the run's storage precision)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in decls:
        t = torch.randn(d.shape, generator=g)
        t = 1 + 0.1 * t if d.init == "norm" else (scale or 0.1) * t
        out[d.name] = t.to(dtype).float()
    return out


def load(part, w):
    from clockwork_b200.weights.loader import kept_dtype

    decls = {d.name: d for d in part.tensor_decls()}
    part.load_weights(lambda name: w[name].to(DEV, kept_dtype(decls[name].role, part.dtype)).contiguous())


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    h, eps = 200, 3e-5
    norm = build_part("norm", PartSpec("rmsnorm", {"size": h, "eps": eps}), "n", dtype, DEV)
    w = weights(norm.tensor_decls(), dtype)
    load(norm, w)
    harness = PartHarness({}, dtype)
    resid = torch.randn(6, h) * 2
    delta = torch.randn(6, h).to(dtype)
    stream = ResidualStream(resid.to(DEV).clone())
    stream.push(delta.to(DEV))
    out = norm.forward(stream, harness.status)
    assert stream.pending is None
    want_resid = resid + delta.float()
    torch.testing.assert_close(stream.residual.cpu(), want_resid, rtol=0, atol=0)
    torch.testing.assert_close(out.float().cpu(), plain.rms_norm(want_resid, w["n.weight"], eps), **tol(dtype, 2))
    rows = torch.tensor([5, 1], dtype=torch.int32, device=DEV)
    out_rows = norm.forward_rows(stream, rows, harness.status)
    assert torch.equal(out_rows, out[[5, 1]])


ATTN = dict(hidden_size=80, num_heads=6, num_kv_heads=2, head_dim=48, qkv_bias=True, o_bias=False,
            scale=48**-0.5, window=None, position=PartSpec("rope_neox", {"theta": 5000.0, "rotary_dim": 48}))


def plain_attention(x, w, prefix, p, positions, window=None):
    config = dict(num_attention_heads=p["num_heads"], num_key_value_heads=p["num_kv_heads"], head_dim=p["head_dim"],
                  rope_theta=p["position"]["theta"])
    return plain.attention_block(x, w, prefix, config, positions, window=window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 11])
def test_attention_part_whole_and_cut(dtype, window):
    params = dict(ATTN, window=window)
    mixer = build_part("mixer", PartSpec("attention", params), "a", dtype, DEV)
    w = weights(mixer.tensor_decls(), dtype, scale=0.2)  # q/k weights large enough for peaked attention
    load(mixer, w)
    t_total, h = 37, params["hidden_size"]
    x = torch.randn(t_total, h).to(dtype).float()
    want = plain_attention(x, w, "a", params, torch.arange(t_total), window=window)
    for cuts in ([t_total], [9, 2, 1, 1, 13, 11]):
        harness = PartHarness({0: mixer.cache_need()}, dtype, page_size=8)
        got, pos = [], 0
        for n in cuts:
            prepared = harness.prepare({"r": n})
            stream = ResidualStream(torch.zeros(n, h, device=DEV))
            assert mixer.forward(prepared.ctx, x[pos : pos + n].to(dtype).to(DEV), prepared.ctx.views[0], stream) is None
            got.append(stream.residual.cpu())
            harness.commit(prepared)
            pos += n
        close(torch.cat(got), want, dtype)
        if window is not None:  # pages behind the window were given back on the way
            assert -1 in harness.cache.get("r").tables[0] or len(cuts) == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_two_requests_in_one_batch(dtype):
    mixer = build_part("mixer", PartSpec("attention", ATTN), "a", dtype, DEV)
    w = weights(mixer.tensor_decls(), dtype, scale=0.2, seed=3)
    load(mixer, w)
    h = ATTN["hidden_size"]
    xa, xb = torch.randn(21, h).to(dtype).float(), torch.randn(14, h).to(dtype).float()
    want_a = plain_attention(xa, w, "a", ATTN, torch.arange(21))
    want_b = plain_attention(xb, w, "a", ATTN, torch.arange(14))
    harness = PartHarness({0: mixer.cache_need()}, dtype, page_size=4)
    outs = {"a": [], "b": []}
    # step 1: 20 tokens of a with 5 of b; step 2: a's last token (a decode) beside 9 more of b
    for take_a, take_b, pa, pb in ((20, 5, 0, 0), (1, 9, 20, 5)):
        prepared = harness.prepare({"a": take_a, "b": take_b})
        x = torch.cat([xa[pa : pa + take_a], xb[pb : pb + take_b]]).to(dtype).to(DEV)
        stream = ResidualStream(torch.zeros(take_a + take_b, h, device=DEV))
        mixer.forward(prepared.ctx, x, prepared.ctx.views[0], stream)
        outs["a"].append(stream.residual[:take_a].cpu())
        outs["b"].append(stream.residual[take_a:].cpu())
        harness.commit(prepared)
    close(torch.cat(outs["a"]), want_a, dtype)
    close(torch.cat(outs["b"]), want_b, dtype)


def test_attention_part_refuses_sizes_it_cannot_run():
    with pytest.raises(ValueError, match="multiples of 16"):
        build_part("mixer", PartSpec("attention", dict(ATTN, head_dim=40)), "a", torch.float32, DEV)
    with pytest.raises(ValueError, match="not a multiple"):
        build_part("mixer", PartSpec("attention", dict(ATTN, num_kv_heads=4)), "a", torch.float32, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_position_parts(dtype):
    """Rotary with a rotary span shorter than the head, and the encoding that leaves q and k alone."""
    nh, nkv, hd = 3, 1, 32
    harness = PartHarness({}, dtype)
    from clockwork_b200.parts.base import PagedView, StepContext

    n = 5
    positions = torch.tensor([0, 7, 100, 3, 2999], dtype=torch.int32, device=DEV)
    ctx = StepContext(dtype=dtype, device=torch.device(DEV), status=harness.status, num_tokens=n, num_seqs=1,
                      positions=positions, tok_seq=torch.zeros(n, dtype=torch.int32, device=DEV), q_start=None,
                      ctx_lens=None, q_lens_host=[n], ctx_lens_host=[n], max_q_len=n, max_ctx_len=n)
    view = PagedView(torch.zeros(2, 4, nkv, hd, dtype=dtype, device=DEV), torch.zeros(2, 4, nkv, hd, dtype=dtype, device=DEV),
                     torch.zeros(1, 2, dtype=torch.int32, device=DEV), torch.arange(n, dtype=torch.int32, device=DEV))
    qkv = torch.randn(n, (nh + 2 * nkv) * hd).to(dtype)
    rope = build_part("position", PartSpec("rope_neox", {"theta": 1e4, "rotary_dim": 16}), "p", dtype, DEV)
    x = qkv.to(DEV).clone()
    rope.apply_and_store(ctx, x, view, nh, nkv, hd)
    cos, sin = plain.rope_cos_sin(positions.cpu(), 16, 1e4, torch.float32)
    q = qkv.float()[:, : nh * hd].view(n, nh, hd)
    want = q.clone()
    want[..., :16] = plain.apply_rope(q[..., :16], cos, sin)
    torch.testing.assert_close(x.float().cpu()[:, : nh * hd].view(n, nh, hd), want, **tol(dtype, 3))
    k = qkv.float()[:, nh * hd : (nh + nkv) * hd].view(n, nkv, hd)
    want_k = k.clone()
    want_k[..., :16] = plain.apply_rope(k[..., :16], cos, sin)
    torch.testing.assert_close(view.k_cache.float().cpu().view(-1, nkv, hd)[:n], want_k, **tol(dtype, 3))
    none = build_part("position", PartSpec("none", {}), "p", dtype, DEV)
    y = qkv.to(DEV).clone()
    none.apply_and_store(ctx, y, view, nh, nkv, hd)
    assert torch.equal(y.cpu(), qkv)
    assert torch.equal(view.k_cache.cpu().view(-1, nkv * hd)[:n], qkv[:, nh * hd : (nh + nkv) * hd])
    assert torch.equal(view.v_cache.cpu().view(-1, nkv * hd)[:n], qkv[:, (nh + nkv) * hd :])


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    h, i = 72, 200
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": h, "intermediate_size": i}), "m", dtype, DEV)
    w = weights(ffn.tensor_decls(), dtype, scale=0.2)
    load(ffn, w)
    x = torch.randn(11, h).to(dtype).float()
    base = torch.randn(11, h)
    stream = ResidualStream(base.to(DEV).clone())
    assert ffn.forward(None, x.to(dtype).to(DEV), stream) is None
    torch.testing.assert_close(stream.residual.cpu(), base + plain.swiglu_mlp(x, w, "m"), **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block(dtype):
    """The pre-norm residual arrangement over its parts == the plain decoder layer."""
    h, eps = 80, 1e-5
    norm = PartSpec("rmsnorm", {"size": h, "eps": eps})
    layer = LayerSpec("prenorm_residual", PartSpec("attention", ATTN), PartSpec("swiglu", {"hidden_size": h, "intermediate_size": 136}),
                      norm, norm, "model.layers.0")
    block = build_block(layer, dtype, DEV)
    w = weights(list(block.tensor_decls()), dtype, scale=0.2)
    load(block, w)
    config = dict(num_attention_heads=6, num_key_value_heads=2, head_dim=48, rope_theta=5000.0, rms_norm_eps=eps)
    t = 19
    x0 = torch.randn(t, h)
    want = plain.decoder_layer(x0, w, 0, config, torch.arange(t))
    harness = PartHarness({0: block.mixer.cache_need()}, dtype)
    got, pos = [], 0
    for n in (12, 1, 6):
        prepared = harness.prepare({"r": n})
        stream = ResidualStream(x0[pos : pos + n].to(DEV).clone())
        block.forward(prepared.ctx, stream, prepared.ctx.views[0])
        stream.flush()
        got.append(stream.residual.cpu())
        harness.commit(prepared)
        pos += n
    close(torch.cat(got), want, dtype)
