"""Each CUDA kernel alone against a plain torch computation of the same operation, at sizes other
than the engine's tiny models (widths and vocabularies that are no power of two, odd head counts
and group sizes, head sizes in steps of 16), in float32 and bfloat16."""

import math

import pytest
import torch

from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(rtol=1e-5, atol=1e-5 * scale) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2 * scale)


@pytest.fixture(scope="module")
def ops():
    from clockwork_b200 import ops

    return ops


@pytest.fixture()
def status(ops):
    return ops.new_status(DEV)


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, status, dtype):
    table = rand(1000, 200, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32)
    out = ops.embed(table.to(DEV), ids.to(DEV), status)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), table.float()[ids.long()], rtol=0, atol=0)
    ops.raise_on_status(status)
    out = ops.embed(table.to(DEV), torch.tensor([3, 1000], dtype=torch.int32, device=DEV), status)
    assert float(out[1].abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="token id outside the vocabulary"):
        ops.raise_on_status(status)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,h", [(5, 7), (5, 200), (5, 1536), (5, 3000),
                                 # many rows: the warp-per-row kernel (row widths that fill, and do not fill, its vectors)
                                 (300, 1536), (257, 200), (300, 3000), (260, 4096), (260, 4100), (300, 6)])
def test_add_rmsnorm(ops, status, dtype, n, h):
    eps = 1e-5
    resid = rand(n, h, scale=3.0)
    delta = rand(n, h, dtype=dtype, seed=1)
    weight = (1 + 0.1 * rand(h, seed=2)).float()
    r = resid.to(DEV).clone()
    out = ops.add_rmsnorm(r, delta.to(DEV), weight.to(DEV), eps, dtype, status)
    want_resid = resid + delta.float()
    torch.testing.assert_close(r.cpu(), want_resid, rtol=0, atol=0)  # one float32 add per element
    torch.testing.assert_close(out.float().cpu(), plain.rms_norm(want_resid, weight, eps), **tol(dtype, 3))
    # without a delta the residual is left alone
    r2 = resid.to(DEV).clone()
    out2 = ops.add_rmsnorm(r2, None, weight.to(DEV), eps, dtype, status)
    assert torch.equal(r2.cpu(), resid)
    torch.testing.assert_close(out2.float().cpu(), plain.rms_norm(resid, weight, eps), **tol(dtype, 3))
    # selected rows
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    out3 = ops.rmsnorm_rows(r2, rows, weight.to(DEV), eps, dtype, status)
    assert torch.equal(out3, out2[[4, 0, 4]])
    ops.raise_on_status(status)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_ref_shapes_epilogues_and_row_independence(ops, dtype):
    m, n, k = 37, 129, 200
    a, w, bias = rand(m, k, dtype=dtype), rand(n, k, dtype=dtype, scale=0.1, seed=1), rand(n, seed=2)
    want = a.float() @ w.float().T + bias
    ad, wd, bd = a.to(DEV), w.to(DEV), bias.to(DEV)
    out = ops.gemm_ref(ad, wd, bd)
    assert out.dtype == dtype
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype, 4))
    # float32 output, and accumulation into a float32 matrix
    out32 = ops.gemm_ref(ad, wd, bd, epilogue=ops.EPILOGUE_STORE_F32)
    torch.testing.assert_close(out32.cpu(), want, rtol=1e-5, atol=5e-5)
    base = rand(m, n, seed=3)
    acc = base.to(DEV).clone()
    ops.gemm_ref(ad, wd, bd, out=acc, epilogue=ops.EPILOGUE_ADD_F32)
    torch.testing.assert_close(acc.cpu(), base + want, rtol=1e-5, atol=5e-5)
    # a row's result does not depend on the rest of the batch (bitwise)
    single = ops.gemm_ref(ad[11:12].contiguous(), wd, bd, epilogue=ops.EPILOGUE_STORE_F32)
    assert torch.equal(single[0], out32[11])
    # a column slice of a wider matrix as the left operand
    wide = rand(m, k + 24, dtype=dtype, seed=4).to(DEV)
    sliced = ops.gemm_ref(wide[:, 8 : 8 + k], wd, None, epilogue=ops.EPILOGUE_STORE_F32)
    torch.testing.assert_close(sliced.cpu(), wide[:, 8 : 8 + k].float().cpu() @ w.float().T, rtol=1e-5, atol=5e-5)
    with pytest.raises(ValueError, match="inner sizes differ"):
        ops.gemm_ref(ad, wd[:, :-1].contiguous())


def test_gemm_ref_is_true_float32(ops):
    """Operands that need 13 mantissa bits, chosen so that every product and every partial sum is
    exact in float32 (22 bits at most) whatever the order of summation: the result must equal the
    float64 one bit for bit.  TF32 (10 bits) or bfloat16 (8 bits) operands could not give that."""
    m, n, k = 8, 16, 256
    g = torch.Generator().manual_seed(0)
    a = 1 + torch.randint(0, 4096, (m, k), generator=g).float() / 4096
    w = torch.randint(1, 3, (n, k), generator=g).float()
    got = ops.gemm_ref(a.to(DEV), w.to(DEV)).double().cpu()
    assert torch.equal(got, a.double() @ w.double().T)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_ref_swiglu_and_silu_mul(ops, dtype):
    m, n, k = 9, 200, 96
    a, wg, wu = rand(m, k, dtype=dtype), rand(n, k, dtype=dtype, scale=0.2, seed=1), rand(n, k, dtype=dtype, scale=0.2, seed=2)
    g, u = a.float() @ wg.float().T, a.float() @ wu.float().T
    want = torch.nn.functional.silu(g) * u
    got = ops.gemm_ref_swiglu(a.to(DEV), wg.to(DEV), wu.to(DEV))
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype, 2))
    gu = torch.cat([g, u], dim=1).to(dtype)
    got2 = ops.silu_mul(gu.to(DEV))
    torch.testing.assert_close(got2.float().cpu(), torch.nn.functional.silu(gu[:, :n].float()) * gu[:, n:].float(), **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot", [(5, 1, 48, 48), (4, 2, 64, 32), (3, 3, 16, 16), (12, 2, 128, 128),
                                           # sizes that the 16-byte kernel does not take (scalar kernel)
                                           (3, 1, 20, 10), (2, 2, 24, 8)])
def test_rope_store(ops, status, dtype, nh, nkv, hd, rot):
    n, pages, ps, theta = 6, 5, 4, 1e6
    qkv = rand(n, (nh + 2 * nkv) * hd, dtype=dtype)
    positions = torch.tensor([0, 1, 4000, 17, 2, 3], dtype=torch.int32)
    slots = torch.tensor([19, 0, 7, -1, 12, 3], dtype=torch.int32)  # -1: not stored
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    k_cache = torch.full((pages, ps, nkv, hd), 100.0, dtype=dtype, device=DEV)
    v_cache = torch.full((pages, ps, nkv, hd), 100.0, dtype=dtype, device=DEV)
    x = qkv.to(DEV).clone()
    ops.rope_store(x, positions.to(DEV), slots.to(DEV), inv_freq.to(DEV), k_cache, v_cache, nh, nkv, hd, rot, status)
    ops.raise_on_status(status)
    q = qkv.float()[:, : nh * hd].view(n, nh, hd)
    k = qkv.float()[:, nh * hd : (nh + nkv) * hd].view(n, nkv, hd)
    v = qkv.float()[:, (nh + nkv) * hd :].view(n, nkv, hd)
    cos, sin = plain.rope_cos_sin(positions, rot, theta, torch.float32)

    def rotate(t):
        out = t.clone()
        out[..., :rot] = plain.apply_rope(t[..., :rot], cos, sin)
        return out

    t = tol(dtype, 3)
    got = x.float().cpu()
    torch.testing.assert_close(got[:, : nh * hd].view(n, nh, hd), rotate(q), **t)
    flat_k, flat_v = k_cache.float().cpu().view(-1, nkv, hd), v_cache.float().cpu().view(-1, nkv, hd)
    stored = slots >= 0
    torch.testing.assert_close(flat_k[slots[stored].long()], rotate(k)[stored], **t)
    torch.testing.assert_close(flat_v[slots[stored].long()], v[stored].to(dtype).float(), rtol=0, atol=0)
    untouched = torch.ones(pages * ps, dtype=torch.bool)
    untouched[slots[stored].long()] = False
    assert bool((flat_k[untouched] == 100.0).all()) and bool((flat_v[untouched] == 100.0).all())
    # a slot outside the pool is reported, not written
    bad = torch.tensor([pages * ps] + [0] * (n - 1), dtype=torch.int32, device=DEV)
    ops.rope_store(qkv.to(DEV), positions.to(DEV), bad, inv_freq.to(DEV), k_cache, v_cache, nh, nkv, hd, rot, status)
    with pytest.raises(RuntimeError, match="cache slot outside the pool"):
        ops.raise_on_status(status)


def paged_setup(seq_lens, nkv, hd, ps, dtype, seed=0, extra_pages=3, fill=100.0):
    """Random K/V for several requests scattered over shuffled pages; padding filled with 100.0
    (the reference's poison trick, tests/test_triton_kernel.py:33-34) or with ``fill``."""
    g = torch.Generator().manual_seed(seed)
    blocks = [(n + ps - 1) // ps for n in seq_lens]
    total = sum(blocks) + extra_pages
    order = torch.randperm(total, generator=g).tolist()
    k_cache = torch.full((total, ps, nkv, hd), fill)
    v_cache = torch.full((total, ps, nkv, hd), fill)
    tables = torch.full((len(seq_lens), max(blocks) + 1), -1, dtype=torch.int32)
    ks, vs = [], []
    for s, n in enumerate(seq_lens):
        k, v = torch.randn(n, nkv, hd, generator=g), torch.randn(n, nkv, hd, generator=g)
        k, v = k.to(dtype).float(), v.to(dtype).float()
        ks.append(k)
        vs.append(v)
        for b in range(blocks[s]):
            page = order.pop()
            tables[s, b] = page
            chunk = slice(b * ps, min((b + 1) * ps, n))
            k_cache[page, : chunk.stop - chunk.start] = k[chunk]
            v_cache[page, : chunk.stop - chunk.start] = v[chunk]
    return k_cache.to(dtype), v_cache.to(dtype), tables, ks, vs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(6, 2, 128, 16, None), (5, 5, 48, 8, None), (8, 1, 16, 4, 37), (3, 1, 256, 16, None)])
def test_attention_ref_mixed_batch(ops, status, dtype, nh, nkv, hd, ps, window):
    # three requests: a prompt portion in the middle of a context, a single decoded token, a whole prompt
    ctx_lens, q_lens = [150, 333, 41], [23, 1, 41]
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype)
    scale = hd**-0.5
    g = torch.Generator().manual_seed(5)
    qs = [torch.randn(q, nh, hd, generator=g).to(dtype).float() * 2 for q in q_lens]
    n = sum(q_lens)
    q_flat = torch.cat(qs).view(n, nh * hd)
    wide = torch.zeros(n, (nh + 2 * nkv) * hd)  # queries live inside a [q|k|v] row
    wide[:, : nh * hd] = q_flat
    tok_seq = torch.cat([torch.full((q,), s, dtype=torch.int32) for s, q in enumerate(q_lens)])
    positions = torch.cat([torch.arange(c - q, c, dtype=torch.int32) for c, q in zip(ctx_lens, q_lens)])
    out = ops.attention_ref(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV), tok_seq.to(DEV),
                            positions.to(DEV), nh, nkv, hd, scale, window, status)
    ops.raise_on_status(status)
    want = torch.cat([plain.causal_attention(q, k, v, scale, window=window) for q, k, v in zip(qs, ks, vs)])
    torch.testing.assert_close(out.float().cpu().view(n, nh, hd), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_ref_finds_one_far_key_and_the_windows_edge(ops, status, dtype):
    """One key among hundreds gets a score that stands out; the output must be that key's value.
    Then a window that ends exactly one short of it: the output must not contain it."""
    nh, nkv, hd, ps, ctx = 2, 1, 32, 16, 700
    k_cache, v_cache, tables, ks, vs = paged_setup([ctx], nkv, hd, ps, dtype, seed=3)
    far = 37  # in the third page
    q = torch.zeros(1, nh, hd)
    q[0, :, 0] = 30.0
    kc = k_cache.float()
    page, off = int(tables[0, far // ps]), far % ps
    kc[page, off, 0, :] = 0.0
    kc[page, off, 0, 0] = 30.0  # score 900 * scale, everything else ~ N(0, 30^2) * scale
    ks[0][far] = kc[page, off]
    wide = torch.zeros(1, (nh + 2) * hd)
    wide[0, : nh * hd] = q.view(-1)
    args = (kc.to(dtype).to(DEV), v_cache.to(DEV), tables.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
            torch.tensor([ctx - 1], dtype=torch.int32, device=DEV), nh, nkv, hd, hd**-0.5)
    out = ops.attention_ref(wide.to(dtype).to(DEV), *args, None, status)
    torch.testing.assert_close(out.float().cpu().view(nh, hd)[0], vs[0][far, 0], **tol(dtype))
    for window, sees in ((ctx - far, True), (ctx - far - 1, False)):
        out = ops.attention_ref(wide.to(dtype).to(DEV), *args, window, status)
        want = plain.causal_attention(q, ks[0], vs[0], hd**-0.5, window=window)
        torch.testing.assert_close(out.float().cpu().view(1, nh, hd), want, **tol(dtype))
        close = torch.allclose(out.float().cpu().view(nh, hd)[0], vs[0][far, 0], atol=0.05)
        assert close == sees
    ops.raise_on_status(status)


def test_attention_ref_reports_pages_outside_the_pool(ops, status):
    k_cache, v_cache, tables, _, _ = paged_setup([20], 1, 16, 4, torch.float32)
    tables[0, 2] = 999
    q = torch.zeros(1, 3 * 16, device=DEV)
    ops.attention_ref(q, k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                      torch.tensor([19], dtype=torch.int32, device=DEV), 1, 1, 16, 0.25, None, status)
    with pytest.raises(RuntimeError, match="page id outside the pool"):
        ops.raise_on_status(status)


def test_copy_pages(ops, status):
    cache = torch.randn(6, 9, 4, 2, 16, device=DEV)  # [planes, pages, page_size, kv_heads, head_dim]
    before = cache.clone()
    pairs = torch.tensor([[2, 7], [0, 5]], dtype=torch.int32, device=DEV)
    ops.copy_pages(cache, pairs, status)
    assert torch.equal(cache[:, 7], before[:, 2]) and torch.equal(cache[:, 5], before[:, 0])
    keep = [0, 1, 2, 3, 4, 6, 8]
    assert torch.equal(cache[:, keep], before[:, keep])
    ops.raise_on_status(status)


def test_argmax_first_maximum_and_odd_vocabulary(ops):
    logits = rand(7, 1003)
    logits[2, 500] = logits[2, 17] = 50.0  # a tie: the first index wins (model_runner.py:136-137)
    logits[5] = -1e30
    got = ops.argmax(logits.to(DEV)).cpu()
    want = logits.argmax(dim=-1)
    want[2] = 17
    want[5] = 0
    assert got.tolist() == want.tolist()


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, -1, 1.0), (1.3, 5, 1.0), (0.7, -1, 0.6), (1.0, 40, 0.9), (0.0, 3, 0.5)])
def test_sample_matches_the_plain_rule(ops, temperature, top_k, top_p):
    r, v = 24, 1003
    logits = rand(r, v, scale=2.0, seed=4)
    u = (torch.arange(r, dtype=torch.float32) + 0.37) / r
    dev = lambda t: t.to(DEV)
    got = ops.sample(dev(logits), dev(torch.full((r,), temperature)), dev(torch.full((r,), max(top_k, 0), dtype=torch.int32)),
                     dev(torch.full((r,), top_p)), dev(u)).cpu().tolist()
    want = [plain.sample_with_uniform(logits[i], temperature, top_k, top_p, float(u[i])) for i in range(r)]
    assert got == want


def test_sample_over_many_blocks_per_row_at_the_real_vocabulary(ops):
    """The chain of kernels that cuts a row over many thread blocks (radix selections over integer
    histograms) against the kernel that walks it with one block, at 151,936 logits: rows with every mix
    of parameters (greedy rows among them, top-k of one and of nearly all, a top-p that keeps one token, a
    peaked and a flat row); the same tokens, and the same again on a second run."""
    r, v = 20, 151936
    logits = rand(r, v, scale=3.0, seed=21)
    logits[3] *= 4.0          # peaked
    logits[4] *= 0.01         # nearly flat
    logits[5, 777] = 60.0     # one token holds all the mass
    temps = torch.tensor([0.0, 0.7, 1.0, 0.9, 1.0, 0.8, 1.3, 0.5, 1.0, 0.0, 0.6, 1.0, 2.0, 0.7, 1.0, 0.9, 1.1, 0.3, 1.0, 0.85])
    ks = torch.tensor([0, 0, 50, 0, 5, 0, 1, 100000, 0, 7, 40, 1000, 0, 3, 151935, 0, 20, 0, 64, 0], dtype=torch.int32)
    ps = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 0.3, 1.0, 0.95, 0.999, 0.5, 0.9, 0.8, 0.7, 1.0, 0.6, 1e-6, 0.99, 0.2, 1.0, 0.0])
    dev = lambda t: t.to(DEV)
    for salt in (0.123, 0.5, 0.987):
        u = ((torch.arange(r, dtype=torch.float32) * 0.61803 + salt) % 1.0)
        args = (dev(logits), dev(temps), dev(ks), dev(ps), dev(u))
        many = ops.sample(*args).cpu().tolist()
        one = ops.sample(*args, one_block=True).cpu().tolist()
        assert many == one, [(i, a, b) for i, (a, b) in enumerate(zip(many, one)) if a != b]
        assert ops.sample(*args).cpu().tolist() == many
    assert many[0] == int(logits[0].argmax()) and many[9] == int(logits[9].argmax()) and many[5] == 777


def test_step_inputs_from_the_request_state_table(ops, status):
    """``step_from_state``: rows name slots of the state table; fresh rows overwrite their column first;
    token, position, context length, cache slot (through the row's block table, two page groups) and the
    sampling parameters come out of the table; the uniform number is the host's ``uniform_for`` of the
    column's seed and draw counter, bit for bit; padding rows and a page outside the pool are handled.
    Then ``argmax`` with the table: the token lands in the column and position and draws advance."""
    import numpy as np

    from clockwork_b200.engine.step import fresh_row
    from clockwork_b200.sampling import uniform_for

    slots, b, ps, max_blocks, pages = 7, 5, 8, 6, 40
    fields = len(ops.REQUEST_STATE_FIELDS)
    state = torch.zeros(fields, slots, dtype=torch.int32)
    # slot 3 goes on from what the table holds; slots 5 and 0 get fresh columns; row 3 is padding; slot 6 has a bad page
    held = fresh_row(position=19, last_token=77, draws=4, seed=(1 << 63) + 12345, temperature=0.7, top_k=11, top_p=0.9)
    state[:, 3] = torch.tensor(held, dtype=torch.int64).to(torch.int32)
    state[:, 6] = torch.tensor(fresh_row(position=9, last_token=5), dtype=torch.int64).to(torch.int32)
    rows = [3, 5, 0, -1, 6]
    fresh_cols = {1: fresh_row(33, 1234, 2, 99, 1.25, 0, 1.0), 2: fresh_row(0, 9)}
    fresh = torch.tensor([0, 1, 1, 0, 0], dtype=torch.int32)
    fresh_values = torch.zeros(fields, b, dtype=torch.int32)
    for r, col in fresh_cols.items():
        fresh_values[:, r] = torch.tensor(col, dtype=torch.int64).to(torch.int32)
    g = torch.Generator().manual_seed(3)
    tables = [torch.randint(0, pages, (b, max_blocks), generator=g, dtype=torch.int32) for _ in range(2)]
    tables[1][4, 1] = pages + 3  # the page of row 4's position 9 in group 1 lies outside the pool
    dev = lambda t: t.to(DEV)  # noqa: E731
    state_d, fresh_d = dev(state), dev(fresh)
    out_i = {k: torch.full((b,), -7, dtype=torch.int32, device=DEV) for k in ("tokens", "positions", "ctx_lens", "tok_seq", "top_k")}
    out_f = {k: torch.full((b,), -7.0, device=DEV) for k in ("temperature", "top_p", "uniform")}
    kv = [torch.full((b,), -7, dtype=torch.int32, device=DEV) for _ in range(2)]
    ops.step_from_state(dev(torch.tensor(rows, dtype=torch.int32)), fresh_d, dev(fresh_values), state_d, [dev(t) for t in tables], kv,
                        ps, pages, out_i["tokens"], out_i["positions"], out_i["ctx_lens"], out_i["tok_seq"],
                        out_f["temperature"], out_i["top_k"], out_f["top_p"], out_f["uniform"], status)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="page id outside the pool"):
        ops.raise_on_status(status)
    assert fresh_d.tolist() == [0, 0, 0, 0, 0]  # used and cleared
    cols = {0: held, 1: fresh_cols[1], 2: fresh_cols[2], 4: fresh_row(9, 5)}
    for r, col in cols.items():
        pos, tok, draws, lo, hi, temp_bits, top_k, top_p_bits = col
        seed = ((hi & 0xFFFFFFFF) << 32) | (lo & 0xFFFFFFFF)
        assert out_i["tokens"][r].item() == tok and out_i["positions"][r].item() == pos and out_i["ctx_lens"][r].item() == pos + 1
        assert out_i["tok_seq"][r].item() == r and out_i["top_k"][r].item() == top_k
        assert out_f["temperature"][r].item() == np.array([temp_bits], dtype=np.int32).view(np.float32)[0]
        assert out_f["top_p"][r].item() == np.array([top_p_bits], dtype=np.int32).view(np.float32)[0]
        assert out_f["uniform"][r].item() == np.float32(uniform_for(seed, draws))
        for grp in range(2):
            page = int(tables[grp][r, pos // ps])
            want = page * ps + pos % ps if page < pages else -1
            assert kv[grp][r].item() == want
    assert out_i["tok_seq"][3].item() == -1 and out_i["ctx_lens"][3].item() == 0 and kv[0][3].item() == -1
    assert state_d[:, 5].tolist() == list(fresh_cols[1]) and state_d[:, 0].tolist() == list(fresh_cols[2])
    # sampling writes back: the token becomes the column's last token, position and draws advance
    logits = torch.randn(b, 50, generator=g).to(DEV)
    before = state_d.clone()
    picked = ops.argmax(logits, into_state=(dev(torch.tensor(rows, dtype=torch.int32)), state_d))
    assert picked.tolist() == logits.argmax(dim=1).tolist()
    for r, slot in enumerate(rows):
        if slot < 0:
            continue
        assert state_d[1, slot].item() == picked[r].item()
        assert state_d[0, slot].item() == before[0, slot].item() + 1 and state_d[2, slot].item() == before[2, slot].item() + 1
        assert state_d[3:, slot].tolist() == before[3:, slot].tolist()
    assert state_d[:, [1, 2, 4]].tolist() == before[:, [1, 2, 4]].tolist()  # slots of no row are untouched


def test_sample_rows_carry_their_own_parameters(ops):
    r, v = 6, 320
    logits = rand(r, v, scale=3.0, seed=9)
    temps = torch.tensor([0.0, 0.5, 1.0, 0.0, 2.0, 0.9])
    ks = torch.tensor([0, 0, 7, 0, 0, 2], dtype=torch.int32)
    ps = torch.tensor([1.0, 0.8, 1.0, 1.0, 0.3, 1.0])
    u = torch.tensor([0.5, 0.1, 0.99, 0.2, 0.6, 0.45])
    got = ops.sample(logits.to(DEV), temps.to(DEV), ks.to(DEV), ps.to(DEV), u.to(DEV)).cpu().tolist()
    want = [plain.sample_with_uniform(logits[i], float(temps[i]), int(ks[i]) or -1, float(ps[i]), float(u[i])) for i in range(r)]
    assert got == want


@pytest.mark.parametrize("v", [3, 33, 4097])
def test_sample_with_equal_logits_and_zeros_of_both_signs(ops, v):
    """Logits rounded to halves, so that many are equal and some are -0.0 beside +0.0 (equal as floats,
    different as bits): a greedy row takes the first of the largest, and top-k keeps every logit that is
    not below the k-th largest (model_runner.py:136-137, :150-152).  Both forms of the sampler against
    the plain rule."""
    r = 12
    logits = (rand(r, v, scale=1.5, seed=40 + v) * 2).round() / 2
    logits[0, 0], logits[0, 1:] = -0.0, 0.0                    # greedy: index 0 although the bits of -0.0 are `smaller'
    logits[1] = -logits[1].abs() - 0.5
    logits[1, v // 2], logits[1, v - 1] = -0.0, 0.0            # the largest value twice, -0.0 first
    logits[2] = 1.5                                            # all equal
    assert v < 33 or (logits[3:] == 0).logical_and(torch.signbit(logits[3:])).any()
    temps = torch.tensor([0.0, 0.0, 0.0, 1.0, 0.7, 1.0, 0.0, 1.3, 1.0, 0.5, 1.0, 2.0])
    ks = torch.tensor([0, 0, 0, 1, 2, v, 5, 3, v + 5, 1, 0, max(v - 1, 1)], dtype=torch.int32)
    ps = torch.ones(r)
    dev = lambda t: t.to(DEV)  # noqa: E731
    for salt in (0.05, 0.51, 0.93):
        u = (torch.arange(r, dtype=torch.float32) * 0.61803 + salt) % 1.0
        args = (dev(logits), dev(temps), dev(ks), dev(ps), dev(u))
        many = ops.sample(*args).cpu().tolist()
        one = ops.sample(*args, one_block=True).cpu().tolist()
        want = [plain.sample_with_uniform(logits[i], float(temps[i]), int(ks[i]) or -1, float(ps[i]), float(u[i])) for i in range(r)]
        assert many == want and one == want, (many, one, want)
    assert many[0] == 0 and many[1] == v // 2 and many[2] == 0


def _draw_keeping_equal_logits_together(logits, temperature, top_k, top_p, u):
    """The rule of model_runner.py:147-164 where equal logits are told apart by nothing: a token stays under
    top-p iff the softmax mass of the logits strictly above it does not exceed top_p (the reference's sort puts
    equal logits in an order it does not define and may cut between them; the kernels keep or drop them
    together, which keeps every token the reference could keep)."""
    l = (logits.to(torch.float32) / temperature).double()
    if 0 < top_k < l.numel():
        l = l.masked_fill(l < torch.topk(l, top_k).values[-1], float("-inf"))
    probs = torch.softmax(l, dim=-1)
    if top_p < 1.0:
        values, inverse = torch.unique(l, return_inverse=True)              # ascending
        mass = torch.zeros_like(values).index_add_(0, inverse, probs)
        above = mass.flip(0).cumsum(0).flip(0) - mass                          # mass strictly above each value
        probs = probs.masked_fill((above > top_p)[inverse], 0.0)
    cdf = probs.cumsum(0)
    return int((cdf > u * float(cdf[-1])).nonzero()[0])


@pytest.mark.parametrize("v", [33, 1003, 50000])
def test_sample_top_p_with_equal_logits(ops, v):
    """Top-p over logits rounded to halves: the cut falls inside a group of equal logits in most rows."""
    r = 16
    logits = (rand(r, v, scale=1.5, seed=70 + v) * 2).round() / 2
    logits[1] = 1.5
    temps = torch.tensor([1.0, 1.0, 0.7, 1.3, 1.0, 0.5, 2.0, 1.0, 0.9, 1.0, 1.5, 0.7, 1.0, 1.0, 0.8, 1.0])
    ks = torch.tensor([0, 0, 0, 10, v, 0, 0, 3, 0, v // 2, 0, 0, 7, 0, 0, 1], dtype=torch.int32)
    ps = torch.tensor([0.9, 0.5, 0.0, 0.8, 0.999, 1e-4, 0.3, 0.6, 0.95, 0.7, 0.1, 0.99, 0.2, 0.4, 0.85, 0.5])
    dev = lambda t: t.to(DEV)  # noqa: E731
    for salt in (0.05, 0.51, 0.93):
        u = (torch.arange(r, dtype=torch.float32) * 0.61803 + salt) % 1.0
        args = (dev(logits), dev(temps), dev(ks), dev(ps), dev(u))
        many = ops.sample(*args).cpu().tolist()
        one = ops.sample(*args, one_block=True).cpu().tolist()
        want = [_draw_keeping_equal_logits_together(logits[i], float(temps[i]), int(ks[i]), float(ps[i]), float(u[i])) for i in range(r)]
        assert many == want and one == want, (many, one, want)


# ---- tcgen05 matrix products -------------------------------------------------------------------------
TC_SHAPES = [
    # T, N, K: decode sizes (inner dimension split over CTAs), ragged edges, prefill sizes
    (1, 2048, 1536), (8, 1536, 8960), (8, 200, 72), (16, 1536, 1536), (17, 384, 200), (64, 2048, 1536),
    (100, 130, 264), (300, 1000, 512), (512, 1536, 1536), (2048, 2048, 1536),
    # more tiles than SMs: the persistent kernel, two to three tiles per CTA, ragged in both directions
    (2100, 3000, 264), (2048, 5000, 512), (2048, 1536, 8960), (1000, 130, 200), (260, 2048, 1536),
]


@pytest.fixture(scope="module")
def gemm_tc():
    from clockwork_b200.ops import gemm_tc

    return gemm_tc


def bf16_product(x, w):
    return (x.double() @ w.double().T).float()


@pytest.mark.parametrize("t,n,k", [(300, 1000, 512), (2100, 3000, 264), (2048, 5000, 512)])
def test_gemm_tc_single_cta_persistent_kernel(ops, gemm_tc, t, n, k):
    """Prompt portions run on CTA pairs by default; the single-CTA persistent kernel stays reachable."""
    gemm_tc.set_pair_kernel(False)
    try:
        test_gemm_tc_against_float64(ops, gemm_tc, t, n, k)
    finally:
        gemm_tc.set_pair_kernel(True)


@pytest.mark.parametrize("t,n,k", [(300, 1536, 8960), (1056, 1536, 8960), (520, 1000, 2048), (700, 300, 4104), (2048, 1536, 8960)])
def test_gemm_tc_pair_kernel_adds_in_split_order(ops, gemm_tc, t, n, k):
    """Prompt-portion products that add into the residual: with few tiles and a long inner dimension
    the CTA-pair kernel splits K over pairs, whose partial tiles add into the output in split order.
    Against float64, and bit for bit the same on every run."""
    g = torch.Generator().manual_seed(t + n + k)
    x = torch.randn(t, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    bias = torch.randn(n, generator=g)
    res0 = torch.randn(t, n, generator=g)
    want = (res0.double() + x.double() @ w.double().T + bias.double()).float()
    xd, wd, bd = x.to(DEV), w.to(DEV), bias.to(DEV)
    outs = []
    for _ in range(4):
        out = res0.to(DEV).clone()
        gemm_tc.gemm(xd, wd, bd, out=out, epilogue=ops.EPILOGUE_ADD_F32)
        outs.append(out.cpu())
    torch.testing.assert_close(outs[0], want, rtol=1e-4, atol=1e-5 * max(1.0, float(want.abs().max())))
    assert all(torch.equal(o, outs[0]) for o in outs[1:])
    assert int(gemm_tc._device_state(torch.device(DEV))["split_flags"].abs().sum()) == 0  # left at zero for the next launch
    ops.raise_on_status(gemm_tc.status(DEV))


@pytest.mark.parametrize("t,n,k", [(1, 57000, 128), (8, 56840, 264), (50, 57096, 136), (64, 60000, 64)])
def test_gemm_tc_few_tokens_over_many_weight_tiles(ops, gemm_tc, t, n, k):
    """A logits-like product (three rounds of weight tiles or more) walks its tiles with one CTA per
    SM; the same sizes with a CTA per tile give the same bits."""
    test_gemm_tc_against_float64(ops, gemm_tc, t, n, k)
    x, w = rand(t, k, dtype=torch.bfloat16).to(DEV), rand(n, k, dtype=torch.bfloat16, scale=0.1, seed=1).to(DEV)
    walked = gemm_tc.gemm(x, w, epilogue=ops.EPILOGUE_STORE_F32)
    gemm_tc.set_stream_kernel(False)
    try:
        per_tile = gemm_tc.gemm(x, w, epilogue=ops.EPILOGUE_STORE_F32)
    finally:
        gemm_tc.set_stream_kernel(True)
    assert torch.equal(walked, per_tile)


@pytest.mark.parametrize("t,n,k", TC_SHAPES)
def test_gemm_tc_against_float64(ops, gemm_tc, t, n, k):
    x, w, bias = rand(t, k, dtype=torch.bfloat16), rand(n, k, dtype=torch.bfloat16, scale=0.1, seed=1), rand(n, seed=2)
    xd, wd, bd = x.to(DEV), w.to(DEV), bias.to(DEV)
    assert gemm_tc.accepts(xd, wd)
    want = bf16_product(x, w) + bias
    scale = max(1.0, float(want.abs().max()))
    out32 = gemm_tc.gemm(xd, wd, bd, epilogue=ops.EPILOGUE_STORE_F32)
    torch.testing.assert_close(out32.cpu(), want, rtol=1e-4, atol=1e-5 * scale)
    out = gemm_tc.gemm(xd, wd, bd)
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.float().cpu(), want, rtol=1e-2, atol=1e-2 * scale)
    base = rand(t, n, seed=3)
    acc = base.to(DEV).clone()
    gemm_tc.gemm(xd, wd, None, out=acc, epilogue=ops.EPILOGUE_ADD_F32)
    torch.testing.assert_close(acc.cpu(), base + bf16_product(x, w), rtol=1e-4, atol=1e-5 * scale)
    # twice in a row gives the same bits
    again = gemm_tc.gemm(xd, wd, bd, epilogue=ops.EPILOGUE_STORE_F32)
    assert torch.equal(again, out32)
    ops.raise_on_status(gemm_tc.status(DEV))


@pytest.mark.parametrize("t,n,k", [(256, 1536, 8960), (300, 520, 4480), (1000, 1536, 8960), (129, 264, 1024)])
def test_gemm_tc_partial_sums_and_the_norm_that_adds_them(ops, gemm_tc, t, n, k):
    """A product split over K with the splits kept apart: the slabs' sum is the product, twice in a row
    the same bits; the RMSNorm kernel that takes the slabs adds them into the residual in slab order
    and normalises, as the plain formulas say; without a norm the slabs are only added."""
    x, w = rand(t, k, dtype=torch.bfloat16), rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=1)
    xd, wd = x.to(DEV), w.to(DEV)
    splits = gemm_tc.partial_sums_splits(t, n, k, DEV)
    assert splits >= 1 and (k < 4096 or splits > 1), splits
    if splits == 1:
        return
    parts = gemm_tc.gemm_partial_sums(xd, wd, splits)
    assert parts.slabs.shape[0] == splits and parts.rows == t
    want = bf16_product(x, w)
    total = parts.slabs[:, :t].double().sum(0).float().cpu()
    torch.testing.assert_close(total, want, rtol=1e-4, atol=1e-5 * max(1.0, float(want.abs().max())))
    assert torch.equal(gemm_tc.gemm_partial_sums(xd, wd, splits).slabs[:, :t], parts.slabs[:, :t])
    base, g = rand(t, n, seed=3), rand(n, seed=4) + 1.0
    resid = base.to(DEV).clone()
    out = ops.add_rmsnorm(resid, parts, g.to(DEV), 1e-6, torch.bfloat16, gemm_tc.status(DEV))
    summed = base.clone()
    for s in range(splits):  # (float32 additions in slab order, as the kernel does them)
        summed += parts.slabs[s, :t].cpu()
    assert torch.equal(resid.cpu(), summed)
    normed = summed * torch.rsqrt((summed.double() ** 2).mean(-1, keepdim=True) + 1e-6).float() * g
    torch.testing.assert_close(out.float().cpu(), normed, rtol=1e-2, atol=1e-2)
    again = base.to(DEV).clone()
    ops.add_to_residual(again, parts)
    assert torch.equal(again.cpu(), summed)
    ops.raise_on_status(gemm_tc.status(DEV))


@pytest.mark.parametrize("t,n,k", [(8, 8960, 1536), (33, 200, 96), (64, 1000, 1536), (700, 520, 256),
                                   (2100, 5000, 264), (300, 8960, 1536), (129, 130, 72)])
def test_gemm_tc_swiglu(ops, gemm_tc, t, n, k):
    """Above 128 tokens the product runs on CTA pairs (two weight tiles per stage, two accumulators) or,
    switched, on the single-CTA persistent kernel: both against the formula."""
    x = rand(t, k, dtype=torch.bfloat16)
    wg, wu = rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=1), rand(n, k, dtype=torch.bfloat16, scale=0.05, seed=2)
    want = torch.nn.functional.silu(bf16_product(x, wg)) * bf16_product(x, wu)
    xd, gd, ud = x.to(DEV), wg.to(DEV), wu.to(DEV)
    try:
        for pairs in (True, False):
            gemm_tc.set_pair_swiglu(pairs)
            got = gemm_tc.gemm_swiglu(xd, gd, ud)
            torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2, atol=1e-2 * max(1.0, float(want.abs().max())),
                                       msg=lambda m: f"on CTA pairs: {pairs}: {m}")
            assert torch.equal(gemm_tc.gemm_swiglu(xd, gd, ud), got)  # twice in a row gives the same bits
    finally:
        gemm_tc.set_pair_swiglu(False)
    ops.raise_on_status(gemm_tc.status(DEV))


@pytest.mark.parametrize("t,n,k,n2", [(1, 1536, 8960, 2048), (8, 1536, 1536, 8960), (37, 200, 264, 130), (128, 1536, 512, 384),
                                      (64, 384, 8960, 1000)])
def test_gemm_tc_splits_a_norm_over_two_products(ops, gemm_tc, t, n, k, n2):
    """The product that adds into the residual also writes bf16(residual * g) and per-tile sums of
    squares; the next product, fed with that, finishes the RMSNorm in its epilogue."""
    eps = 1e-5
    x, w = rand(t, k, dtype=torch.bfloat16), rand(n, k, dtype=torch.bfloat16, scale=0.1, seed=1)
    base, g = rand(t, n, seed=3, scale=2.0), (1 + 0.1 * rand(n, seed=4)).float()
    resid = base.to(DEV).clone()
    xg = torch.full((t, n), 7.0, dtype=torch.bfloat16, device=DEV)
    parts = torch.full((t, gemm_tc.norm_tiles(n)), -1.0, device=DEV)
    gemm_tc.gemm(x.to(DEV), w.to(DEV), None, out=resid, epilogue=ops.EPILOGUE_ADD_F32, emit=(g.to(DEV), xg, parts))
    want_resid = base + bf16_product(x, w)
    scale = max(1.0, float(want_resid.abs().max()))
    torch.testing.assert_close(resid.cpu(), want_resid, rtol=1e-4, atol=1e-5 * scale)
    got_resid = resid.cpu()
    assert torch.equal(xg.cpu(), (got_resid * g).bfloat16())  # from the very values that were stored
    torch.testing.assert_close(parts.sum(1).cpu(), (got_resid.double() ** 2).sum(1).float(), rtol=1e-5, atol=0)
    # the consumer: plain with bias, and SwiGLU
    w2, bias2 = rand(n2, n, dtype=torch.bfloat16, scale=0.05, seed=5), rand(n2, seed=6)
    inv = 1.0 / torch.sqrt((got_resid.double() ** 2).mean(1, keepdim=True) + eps)
    want = ((xg.cpu().double() @ w2.double().T) * inv).float() + bias2
    got = gemm_tc.gemm(xg, w2.to(DEV), bias2.to(DEV), epilogue=ops.EPILOGUE_STORE_F32, row_scale=(parts, eps, n))
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-5 * max(1.0, float(want.abs().max())))
    w3 = rand(n2, n, dtype=torch.bfloat16, scale=0.05, seed=7)
    gate, up = ((xg.cpu().double() @ w2.double().T) * inv).float(), ((xg.cpu().double() @ w3.double().T) * inv).float()
    want_act = torch.nn.functional.silu(gate) * up
    got_act = gemm_tc.gemm_swiglu(xg, w2.to(DEV), w3.to(DEV), row_scale=(parts, eps, n))
    torch.testing.assert_close(got_act.float().cpu(), want_act, rtol=1e-2, atol=1e-2 * max(1.0, float(want_act.abs().max())))
    ops.raise_on_status(gemm_tc.status(DEV))


def test_gemm_tc_rows_do_not_depend_on_the_batch(ops, gemm_tc):
    """The same token gives the same bits alone, in a batch of 8 and in a batch of 64 (the split of
    the inner dimension may differ between those, the order of the float32 sums inside a split does not)."""
    k, n = 1536, 2048
    x, w = rand(64, k, dtype=torch.bfloat16).to(DEV), rand(n, k, dtype=torch.bfloat16, scale=0.1, seed=1).to(DEV)
    full = gemm_tc.gemm(x, w, epilogue=ops.EPILOGUE_STORE_F32)
    for rows in (1, 8):
        part = gemm_tc.gemm(x[:rows].contiguous(), w, epilogue=ops.EPILOGUE_STORE_F32)
        torch.testing.assert_close(part, full[:rows], rtol=1e-5, atol=1e-5)


def test_gemm_tc_refuses_what_tma_cannot_address(ops, gemm_tc):
    x, w = rand(4, 100, dtype=torch.bfloat16).to(DEV), rand(32, 100, dtype=torch.bfloat16).to(DEV)
    assert not gemm_tc.accepts(x, w)  # rows of 200 bytes are no multiple of 16
    from clockwork_b200.ops import gemm as dispatch

    out = dispatch.linear(x, w, None)  # the product path falls back to the plain kernel
    torch.testing.assert_close(out.float().cpu(), bf16_product(x.cpu(), w.cpu()), rtol=1e-2, atol=1e-2)
    wide = rand(4, 128, dtype=torch.bfloat16).to(DEV)
    assert gemm_tc.accepts(wide[:, 8:72], rand(32, 64, dtype=torch.bfloat16).to(DEV))  # an aligned column slice
    assert not gemm_tc.accepts(wide[:, 4:68], rand(32, 64, dtype=torch.bfloat16).to(DEV))


# ---- bfloat16 attention kernels ------------------------------------------------------------------------
@pytest.fixture(scope="module")
def fast():
    from clockwork_b200.ops import attention_fast

    return attention_fast


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (5, 5, 48, 8, None), (32, 1, 64, 16, None),
                                                (6, 2, 16, 4, None), (4, 2, 32, 8, 300), (3, 1, 256, 16, None)])
def test_attention_decode_kernel(ops, status, fast, nh, nkv, hd, ps, window):
    """Contexts that end inside the first tile, on a tile's edge, one past a split's edge and deep
    into several splits; padding filled with 100.0 must not leak; a request of length 0 is padding."""
    ctx_lens = [1, 17, 64, 256, 257, 700, 1300, 0]
    dtype = torch.bfloat16
    real = [c for c in ctx_lens if c > 0]
    k_cache, v_cache, tables, ks, vs = paged_setup(real, nkv, hd, ps, dtype, seed=11)
    tables = torch.cat([tables, torch.full((1, tables.shape[1]), -1, dtype=torch.int32)])
    g = torch.Generator().manual_seed(2)
    scale = hd**-0.5
    qs = [(torch.randn(1, nh, hd, generator=g) * 2).to(dtype).float() for _ in ctx_lens]
    wide = torch.zeros(len(ctx_lens), (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(len(ctx_lens), -1)
    out = fast.attention_decode(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
                                torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window,
                                max(ctx_lens), status, split=256).float().cpu().view(len(ctx_lens), nh, hd)
    ops.raise_on_status(status)
    for i, n in enumerate(real):
        want = plain.causal_attention(qs[i], ks[i], vs[i], scale, window=window)[0]
        torch.testing.assert_close(out[i], want, rtol=2e-2, atol=2e-2, msg=lambda m: f"context {n}: {m}")
    assert float(out[-1].abs().max()) == 0.0
    # the grid's bound on the context changes nothing
    again = fast.attention_decode(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
                                  torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window,
                                  4096, status, split=256).float().cpu().view(len(ctx_lens), nh, hd)
    assert torch.equal(again, out)
    # other ways of cutting the contexts (coarser, whole, chosen by the policy, given on the device)
    # ... and the other variants of the kernel: two tiles in flight, padded and swizzled K/V tiles
    # ... and the splits meeting through thread-block clusters of 16, 8 and 2 CTAs instead of the workspace
    # (a cluster of 2 over contexts bounded by 2,048 makes the kernel cut no finer than 1,024 tokens)
    cl = fast.CLUSTER_SHIFT
    for kw in (dict(split=512), dict(split=1344), dict(), dict(split_dev=torch.tensor([320], dtype=torch.int32, device=DEV)),
               dict(split=128, stages=2), dict(split=128, stages=2 | fast.SWIZZLED), dict(split=384, stages=2 | fast.SWIZZLED),
               dict(stages=2 | fast.SWIZZLED), dict(split=128, stages=16 << cl), dict(split=128, stages=2 | 16 << cl),
               dict(split=256, stages=2 | fast.SWIZZLED | 8 << cl), dict(stages=4 | 2 << cl),
               dict(split_dev=torch.tensor([192], dtype=torch.int32, device=DEV), stages=2 | 16 << cl)):
        other = fast.attention_decode(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
                                      torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window,
                                      2048, status, **kw).float().cpu().view(len(ctx_lens), nh, hd)
        for i, n in enumerate(real):
            want = plain.causal_attention(qs[i], ks[i], vs[i], scale, window=window)[0]
            torch.testing.assert_close(other[i], want, rtol=2e-2, atol=2e-2, msg=lambda m: f"{kw}, context {n}: {m}")
    # a bound far beyond the contexts only adds idle CTAs
    far = fast.attention_decode(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
                                torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window,
                                6000, status, split=256).float().cpu().view(len(ctx_lens), nh, hd)
    assert torch.equal(far, out)
    ops.raise_on_status(status)


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (32, 1, 64, 8, None), (4, 2, 128, 32, 300),
                                                (3, 1, 256, 64, None), (6, 3, 192, 16, 500), (8, 2, 64, 64, 70)])
def test_attention_decode_tiles_by_tma(ops, status, fast, nh, nkv, hd, ps, window):
    """K/V tiles fetched by TMA (a copy per page and operand, the hardware's swizzle) against the plain
    formula, and bit for bit against the same variant fed by cp.async: only the way into shared memory
    differs.  What the pages hold beyond a context is NaN here: a whole page arrives, and nothing of
    its unused rows may reach a result."""
    ctx_lens = [1, 17, 64, 65, 256, 257, 700, 1300, 0]
    dtype = torch.bfloat16
    real = [c for c in ctx_lens if c > 0]
    k_cache, v_cache, tables, ks, vs = paged_setup(real, nkv, hd, ps, dtype, seed=13, fill=float("nan"))
    tables = torch.cat([tables, torch.full((1, tables.shape[1]), -1, dtype=torch.int32)])
    g = torch.Generator().manual_seed(4)
    scale = hd**-0.5
    qs = [(torch.randn(1, nh, hd, generator=g) * 2).to(dtype).float() for _ in ctx_lens]
    wide = torch.zeros(len(ctx_lens), (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(len(ctx_lens), -1)
    args = (wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
            torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window, 2048, status)
    deep = 4 if hd <= 128 else 2  # (the larger heads have two tiles in flight whatever is asked for)
    for kw in (dict(split=128, stages=2), dict(split=384, stages=2 | fast.SWIZZLED), dict(stages=2 | fast.SWIZZLED),
               dict(split=256, stages=deep), dict(split=1344, stages=deep), dict(stages=deep),
               dict(split_dev=torch.tensor([192], dtype=torch.int32, device=DEV), stages=2)):
        by_tma = fast.attention_decode(*args, **{**kw, "stages": kw["stages"] | fast.TMA_TILES}).float().cpu().view(len(ctx_lens), nh, hd)
        by_cp_async = fast.attention_decode(*args, **kw).float().cpu().view(len(ctx_lens), nh, hd)
        ops.raise_on_status(status)
        assert torch.isfinite(by_tma).all(), kw
        for i, n in enumerate(real):
            want = plain.causal_attention(qs[i], ks[i], vs[i], scale, window=window)[0]
            torch.testing.assert_close(by_tma[i], want, rtol=2e-2, atol=2e-2, msg=lambda m: f"{kw}, context {n}: {m}")
        assert torch.equal(by_tma, by_cp_async), kw
        assert float(by_tma[-1].abs().max()) == 0.0
    # a split read from the device may come with a bound that sizes the page list in shared memory ...
    on_device = torch.tensor([192], dtype=torch.int32, device=DEV)
    bounded = fast.attention_decode(*args, split=256, split_dev=on_device, stages=2 | fast.TMA_TILES).float().cpu().view(len(ctx_lens), nh, hd)
    free = fast.attention_decode(*args, split_dev=on_device, stages=2 | fast.TMA_TILES).float().cpu().view(len(ctx_lens), nh, hd)
    ops.raise_on_status(status)
    assert torch.equal(bounded, free)
    # ... and a split beyond the bound is refused by the kernel, loudly
    fast.attention_decode(*args, split=128, split_dev=on_device, stages=2 | fast.TMA_TILES)
    with pytest.raises(RuntimeError, match="longer than the bound"):
        ops.raise_on_status(status)


@pytest.mark.parametrize("window", [None, 5000])
def test_attention_decode_merges_many_splits_in_two_levels(ops, status, fast, window):
    """Contexts cut into 51, 37 and 36 splits of 128 tokens: more than 36 meet in two levels (twelve
    splits share a counter, their last merges them, the last merger merges the results; the last group
    of the 37 holds a single split), 36 at one counter.  With a window the first splits hold no key
    and the groups of twelve start at the first split that does.  A second call gives the same bits:
    every counter is back at zero."""
    nh, nkv, hd, ps = 12, 2, 128, 16
    ctx_lens = [6500, 4700, 4608, 1]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=17)
    g = torch.Generator().manual_seed(6)
    scale = hd**-0.5
    qs = [(torch.randn(1, nh, hd, generator=g) * 2).to(dtype).float() for _ in ctx_lens]
    wide = torch.zeros(len(ctx_lens), (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(len(ctx_lens), -1)
    args = (wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV),
            torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), nh, nkv, hd, scale, window, 8192, status)
    outs = []
    for stages in (2, 2 | fast.SWIZZLED | fast.TMA_TILES, 2):
        out = fast.attention_decode(*args, split=128, stages=stages).float().cpu().view(len(ctx_lens), nh, hd)
        ops.raise_on_status(status)
        for i, n in enumerate(ctx_lens):
            want = plain.causal_attention(qs[i], ks[i], vs[i], scale, window=window)[0]
            torch.testing.assert_close(out[i], want, rtol=2e-2, atol=2e-2, msg=lambda m: f"stages {stages:#x}, context {n}: {m}")
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_attention_decode_scratch_outlives_captured_graphs(ops, status, fast):
    """A captured graph has the addresses of the split-merge scratch baked in.  A later, larger call
    makes the module take a larger scratch set; the set the graph points at must stay alive and its
    counters intact, so that replaying the older graph still merges its splits (contexts spanning
    several splits) and equals the uncaptured call."""
    nh, nkv, hd, ps = 12, 2, 128, 16
    ctx_lens = [900, 130, 517, 1024]
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, torch.bfloat16, seed=21)
    g = torch.Generator().manual_seed(5)
    q = (torch.randn(len(ctx_lens), (nh + 2 * nkv) * hd, generator=g) * 2).bfloat16().to(DEV)
    kc, vc, tb = k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)

    def call():
        return fast.attention_decode(q, kc, vc, tb, ctx, nh, nkv, hd, hd**-0.5, None, 1024, status, split=128)

    eager = call().clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = call()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    # a call that needs more scratch than any before it: 64 requests whose contexts are bounded (the
    # bound sizes the grid and the scratch, the contexts themselves stay short) beyond what is there
    before = fast._scratch[torch.cuda.current_device()]
    bound = (before["part_o"].numel() // (64 * nh * hd) + 2) * fast.MIN_SPLIT
    big_ctx = [100] * 64
    bk, bv, bt, _, _ = paged_setup(big_ctx, nkv, hd, ps, torch.bfloat16, seed=22)
    bq = torch.randn(64, (nh + 2 * nkv) * hd, generator=g).bfloat16().to(DEV)
    fast.attention_decode(bq, bk.to(DEV), bv.to(DEV), bt.to(DEV), torch.tensor(big_ctx, dtype=torch.int32, device=DEV),
                          nh, nkv, hd, hd**-0.5, None, bound, status)
    assert fast._scratch[torch.cuda.current_device()] is not before, "the larger call was meant to outgrow the scratch"
    # whatever the allocator hands out now must not be the memory the graph still uses
    junk = [torch.full((1 << 20,), 7.0, device=DEV) for _ in range(12)] + [torch.full((1 << 14,), 3, dtype=torch.int32, device=DEV) for _ in range(8)]
    torch.cuda.synchronize()
    captured.zero_()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)
    assert all(float(t.float().min()) == float(t.float().max()) for t in junk)  # and the graph wrote into none of it
    ops.raise_on_status(status)


def test_attention_decode_finds_one_far_key(ops, status, fast):
    nh, nkv, hd, ps, ctx = 4, 1, 64, 16, 1000
    for far in (3, 255, 256, 777, 999):
        k_cache, v_cache, tables, ks, vs = paged_setup([ctx], nkv, hd, ps, torch.bfloat16, seed=far)
        q = torch.zeros(1, nh, hd)
        q[0, :, 5] = 24.0
        kc = k_cache.float()
        page, off = int(tables[0, far // ps]), far % ps
        kc[page, off, 0, :] = 0.0
        kc[page, off, 0, 5] = 24.0
        wide = torch.zeros(1, (nh + 2) * hd)
        wide[0, : nh * hd] = q.view(-1)
        out = fast.attention_decode(wide.bfloat16().to(DEV), kc.bfloat16().to(DEV), v_cache.to(DEV), tables.to(DEV),
                                    torch.tensor([ctx], dtype=torch.int32, device=DEV), nh, nkv, hd, hd**-0.5, None, ctx, status)
        torch.testing.assert_close(out.float().cpu().view(nh, hd)[2], vs[0][far, 0], rtol=2e-2, atol=2e-2)
    ops.raise_on_status(status)


@pytest.mark.parametrize("kernel,nh,nkv,hd,ps,window", [
    ("mma", 12, 2, 128, 16, None), ("mma", 5, 5, 48, 8, None), ("mma", 8, 1, 16, 4, 37), ("mma", 4, 2, 32, 8, 100),
    ("mma", 6, 3, 64, 16, None),
    ("tc", 12, 2, 128, 16, None), ("tc", 6, 3, 64, 16, None), ("tc", 4, 2, 64, 8, 100), ("tc", 3, 1, 128, 32, 300),
    ("tc", 2, 1, 64, 128, None), ("tc", 5, 5, 128, 64, 37)])
def test_attention_prefill_kernel_mixed_batch(ops, status, fast, kernel, nh, nkv, hd, ps, window):
    """Portions in the middle of a context, whole prompts (shorter and longer than a tile, ending on
    and off tile edges), and single decoded tokens, all in one launch; the mma.sync kernel and the
    tcgen05 kernel."""
    assert kernel == "mma" or fast.prefill_tc_takes(hd, ps)
    ctx_lens, q_lens = [150, 333, 41, 200, 1000, 64, 65, 129], [23, 1, 41, 200, 130, 64, 2, 128]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=5)
    scale = hd**-0.5
    g = torch.Generator().manual_seed(6)
    qs = [(torch.randn(q, nh, hd, generator=g) * 2).to(dtype).float() for q in q_lens]
    n = sum(q_lens)
    wide = torch.zeros(n, (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(n, nh * hd)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)
    items = [(s, q0) for s, q in enumerate(q_lens) for q0 in range(0, q, fast.QUERY_TILE)]
    item_seq = torch.tensor([i[0] for i in items], dtype=torch.int32)
    item_q0 = torch.tensor([i[1] for i in items], dtype=torch.int32)
    out = fast.attention_prefill(wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV), q_start.to(DEV),
                                 torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), item_seq.to(DEV), item_q0.to(DEV),
                                 len(items), nh, nkv, hd, scale, window, status, use_tc=kernel == "tc").float().cpu().view(n, nh, hd)
    ops.raise_on_status(status)
    row = 0
    for i, (q, k, v) in enumerate(zip(qs, ks, vs)):
        want = plain.causal_attention(q, k, v, scale, window=window)
        torch.testing.assert_close(out[row : row + q.shape[0]], want, rtol=2e-2, atol=2e-2,
                                   msg=lambda m: f"request {i} (context {ctx_lens[i]}, {q_lens[i]} queries): {m}")
        row += q.shape[0]


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (5, 5, 48, 8, None), (8, 1, 16, 4, 37), (28, 4, 128, 16, None)])
def test_single_tokens_of_a_mixed_batch_go_to_the_decode_kernel(ops, status, fast, nh, nkv, hd, ps, window):
    """A flat batch of prompt portions and requests that bring one token: the prefill kernel takes the
    portions (its work items leave the single tokens out), the decode kernel takes the requests with
    exactly one row (it finds their rows through q_start and leaves the others' rows alone), and the two
    fill one output tensor.  Single tokens first, last and between portions; contexts of one token, of a
    few splits and of many."""
    ctx_lens, q_lens = [700, 150, 1, 333, 41, 1300, 2000, 64, 129], [1, 23, 1, 1, 41, 1, 130, 1, 128]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=15)
    scale = hd**-0.5
    g = torch.Generator().manual_seed(16)
    qs = [(torch.randn(q, nh, hd, generator=g) * 2).to(dtype).float() for q in q_lens]
    n = sum(q_lens)
    wide = torch.zeros(n, (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(n, nh * hd)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32).to(DEV)
    seqs, q0s, _ = fast.prefill_work_items(q_lens, ctx_lens, skip_single=True)
    assert sorted(set(seqs)) == [i for i, q in enumerate(q_lens) if q > 1]
    qd, kd, vd, td = wide.to(dtype).to(DEV), k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV)
    cd = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    out = fast.attention_prefill(qd, kd, vd, td, q_start, cd, torch.tensor(seqs, dtype=torch.int32, device=DEV),
                                 torch.tensor(q0s, dtype=torch.int32, device=DEV), len(seqs), nh, nkv, hd, scale, window, status)
    single_rows = [int(q_start[i]) for i, q in enumerate(q_lens) if q == 1]
    out[single_rows] = 77.0  # whatever the prefill kernel left there must be overwritten
    longest = max(c for c, q in zip(ctx_lens, q_lens) if q == 1)
    for kw in (dict(split=128), dict(split=256, stages=2), dict()):
        got = fast.attention_decode(qd, kd, vd, td, cd, nh, nkv, hd, scale, window, longest, status, q_start=q_start,
                                    out=out.clone(), **kw).float().cpu().view(n, nh, hd)
        ops.raise_on_status(status)
        row = 0
        for i, (q, k, v) in enumerate(zip(qs, ks, vs)):
            want = plain.causal_attention(q, k, v, scale, window=window)
            torch.testing.assert_close(got[row : row + q.shape[0]], want, rtol=2e-2, atol=2e-2,
                                       msg=lambda m: f"{kw} request {i} (context {ctx_lens[i]}, {q_lens[i]} queries): {m}")
            row += q.shape[0]


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (3, 1, 64, 32, None), (4, 2, 128, 8, 200)])
def test_attention_prefill_cuts_long_rows_of_keys(ops, status, fast, nh, nkv, hd, ps, window):
    """Query tiles with long rows of keys can be walked by several CTAs, whose partial results the
    last one merges: the same values as uncut, the same bits on every run (the counters return to
    zero), parts without a visible key (a window) included; and one far key that outweighs all
    others is found from whichever part holds it."""
    ctx_lens, q_lens = [2500, 1100, 3000, 4200, 600], [300, 1100, 1, 129, 600]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=15)
    scale = hd**-0.5
    g = torch.Generator().manual_seed(16)
    qs = [(torch.randn(q, nh, hd, generator=g) * 2).to(dtype).float() for q in q_lens]
    # request 3: key 70 (in the first part of every tile's keys) scores far above the rest for head 0
    kc = k_cache.float()
    page, off = int(tables[3, 70 // ps]), 70 % ps
    kc[page, off, 0, :] = 0.0
    kc[page, off, 0, 3] = 24.0
    qs[3][:, 0, :] = 0.0
    qs[3][:, 0, 3] = 24.0
    ks[3][70, 0, :] = kc[page, off, 0, :]
    n = sum(q_lens)
    wide = torch.zeros(n, (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(n, nh * hd)
    q_start = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32)

    def run(split):
        seqs, q0s, words = fast.prefill_work_items(q_lens, ctx_lens, nh if split else 0, 148 * 4)  # (room for many parts)
        assert (max(w & 0xFF for w in words) > 3) == split
        dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
        out = fast.attention_prefill(wide.to(dtype).to(DEV), kc.to(dtype).to(DEV), v_cache.to(DEV), tables.to(DEV), q_start.to(DEV),
                                     dev(ctx_lens), dev(seqs), dev(q0s), len(seqs), nh, nkv, hd, scale, window, status,
                                     item_split=dev(words) if split else None)
        ops.raise_on_status(status)
        return out

    cut, again, whole = run(True), run(True), run(False)
    assert torch.equal(cut, again)
    torch.testing.assert_close(cut.float(), whole.float(), rtol=2e-2, atol=2e-2)
    out = cut.float().cpu().view(n, nh, hd)
    row = 0
    for i, (q, k, v) in enumerate(zip(qs, ks, vs)):
        want = plain.causal_attention(q, k, v, scale, window=window)
        torch.testing.assert_close(out[row : row + q.shape[0]], want, rtol=2e-2, atol=2e-2,
                                   msg=lambda m: f"request {i} (context {ctx_lens[i]}, {q_lens[i]} queries): {m}")
        if i == 3 and window is None:
            torch.testing.assert_close(out[row : row + q.shape[0], 0], vs[3][70, 0].expand(q.shape[0], hd), rtol=2e-2, atol=2e-2)
        row += q.shape[0]


def test_attention_prefill_with_rows_cut_to_even_out_rounds_of_ctas(ops, status, fast):
    """A portion behind a long context has more tiles x heads than SMs, all of about the same length; the
    work list cuts every row into parts so that the rounds of CTAs come out even (here 13 tiles x 12 heads
    in three parts each).  The same values as plain attention, and one far key per head is found."""
    nh, nkv, hd, ps = 12, 2, 128, 16
    ctx_lens, q_lens = [9000], [1600]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, ks, vs = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=25)
    scale = hd**-0.5
    g = torch.Generator().manual_seed(26)
    qs = [(torch.randn(q, nh, hd, generator=g) * 2).to(dtype).float() for q in q_lens]
    kc = k_cache.float()
    far = 5000  # (in the second of three parts) outweighs all other keys for the first head of KV head 1
    page, off = int(tables[0, far // ps]), far % ps
    kc[page, off, 1, :] = 0.0
    kc[page, off, 1, 9] = 24.0
    qs[0][:, 6, :] = 0.0
    qs[0][:, 6, 9] = 24.0
    ks[0][far, 1, :] = kc[page, off, 1, :]
    n = sum(q_lens)
    wide = torch.zeros(n, (nh + 2 * nkv) * hd)
    wide[:, : nh * hd] = torch.cat(qs).view(n, nh * hd)
    q_start = torch.tensor([0, n], dtype=torch.int32)
    seqs, q0s, words = fast.prefill_work_items(q_lens, ctx_lens, nh, 148)
    assert len(seqs) * nh > 148 and {w & 0xFF for w in words} == {3}
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    out = fast.attention_prefill(wide.to(dtype).to(DEV), kc.to(dtype).to(DEV), v_cache.to(DEV), tables.to(DEV), q_start.to(DEV),
                                 dev(ctx_lens), dev(seqs), dev(q0s), len(seqs), nh, nkv, hd, scale, None, status,
                                 item_split=dev(words))
    ops.raise_on_status(status)
    out = out.float().cpu().view(n, nh, hd)
    want = plain.causal_attention(qs[0], ks[0], vs[0], scale)
    torch.testing.assert_close(out, want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:, 6], vs[0][far, 1].expand(n, hd), rtol=2e-2, atol=2e-2)


def test_attention_prefill_refuses_a_bad_cut(ops, status, fast):
    nh, nkv, hd, ps = 2, 1, 64, 16
    k_cache, v_cache, tables, _, _ = paged_setup([200], nkv, hd, ps, torch.bfloat16, seed=1)
    wide = torch.zeros(200, (nh + 2) * hd, dtype=torch.bfloat16, device=DEV)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    fast.attention_prefill(wide, k_cache.to(DEV), v_cache.to(DEV), tables.to(DEV), dev([0, 200]), dev([200]), dev([0, 0]),
                           dev([0, 128]), 2, nh, nkv, hd, 1.0, None, status, item_split=dev([0 << 8 | 1, 1 << 8 | 9]))
    with pytest.raises(RuntimeError, match="cut of its keys"):
        ops.raise_on_status(status)


@pytest.mark.parametrize("hd,n", [(32, 150), (64, 150), (128, 300)])
def test_attention_prefill_sees_the_diagonal_and_nothing_after_it(ops, status, fast, hd, n):
    """Each query's own key carries a score that stands out, so each output must be its own value;
    if the mask were off by one either way the output would be a neighbour's.  (Head size 32 runs the
    mma.sync kernel, 64 and 128 the tcgen05 kernel.)"""
    nh, nkv, ps = 2, 1, 16
    k_cache, v_cache, tables, ks, vs = paged_setup([n], nkv, hd, ps, torch.bfloat16, seed=9)
    kc = k_cache.float()
    q = torch.zeros(n, nh, hd)
    for pos in range(n):
        page, off = int(tables[0, pos // ps]), pos % ps
        code = torch.tensor([1.0 if (pos >> b) & 1 else -1.0 for b in range(9)]) * 6.0
        kc[page, off, 0, :] = 0.0
        kc[page, off, 0, :9] = code
        q[pos, :, :9] = code
    wide = torch.zeros(n, (nh + 2) * hd)
    wide[:, : nh * hd] = q.view(n, -1)
    items = list(range(0, n, fast.QUERY_TILE))
    out = fast.attention_prefill(wide.bfloat16().to(DEV), kc.bfloat16().to(DEV), v_cache.to(DEV), tables.to(DEV),
                                 torch.tensor([0, n], dtype=torch.int32, device=DEV), torch.tensor([n], dtype=torch.int32, device=DEV),
                                 torch.zeros(len(items), dtype=torch.int32, device=DEV), torch.tensor(items, dtype=torch.int32, device=DEV),
                                 len(items), nh, nkv, hd, 1.0, None, status).float().cpu().view(n, nh, hd)
    ops.raise_on_status(status)
    # own score 9*36 = 324; any other key differs in at least one bit: at most 324 - 72
    torch.testing.assert_close(out[:, 0], vs[0][:, 0], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nh,nkv,hd,ps,rot", [(12, 2, 128, 16, 128), (5, 5, 48, 8, 32), (32, 1, 64, 16, 64), (4, 2, 32, 8, 0)])
def test_attention_decode_fused_position_and_store(ops, status, fast, nh, nkv, hd, ps, rot):
    """The decode kernel doing the rotation of q and the new k and the cache write itself == the
    position kernel followed by the plain decode kernel, bit for bit, cache included."""
    ctx_lens = [1, 17, 64, 256, 257, 700, 1300]
    dtype = torch.bfloat16
    k_cache, v_cache, tables, _, _ = paged_setup(ctx_lens, nkv, hd, ps, dtype, seed=21)
    n = len(ctx_lens)
    qkv = rand(n, (nh + 2 * nkv) * hd, dtype=dtype, scale=2.0, seed=3).to(DEV)
    positions = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(tables[i, (c - 1) // ps]) * ps + (c - 1) % ps for i, c in enumerate(ctx_lens)],
                         dtype=torch.int32, device=DEV)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV) if rot else None
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    scale = hd**-0.5
    # the two-kernel way
    k1, v1, x1 = k_cache.to(DEV).clone(), v_cache.to(DEV).clone(), qkv.clone()
    ops.rope_store(x1, positions, slots, inv_freq, k1, v1, nh, nkv, hd, rot, status)
    want = fast.attention_decode(x1, k1, v1, tables.to(DEV), ctx, nh, nkv, hd, scale, None, max(ctx_lens), status, split=256)
    # the fused way
    k2, v2 = k_cache.to(DEV).clone(), v_cache.to(DEV).clone()
    got = fast.attention_decode(qkv, k2, v2, tables.to(DEV), ctx, nh, nkv, hd, scale, None, max(ctx_lens), status, split=256,
                                fused=(inv_freq, rot, slots))
    ops.raise_on_status(status)
    assert torch.equal(k2, k1) and torch.equal(v2, v1)
    assert torch.equal(got, want)
