"""Each kernel alone against a plain torch float32 reference of the same operation, at
sizes other than the tiny models': head sizes in steps of 16, odd head and group counts,
widths and vocabularies that are no power of two."""

import math

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab, width", [(37, 24), (1000, 520)])
def test_embedding(dtype, vocab, width):
    from yalis_b200.ops.elementwise import embedding
    table = rnd(vocab, width, dtype=dtype)
    ids = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = embedding(table, ids, bad_flag=flag)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())
    assert int(flag) == 0
    embedding(table, torch.tensor([vocab], dtype=torch.int32, device=DEV), bad_flag=flag)
    assert int(flag) == 1                                   # an id out of range is flagged, not read
    # a scale; and ids taken from the per-slot array of chosen tokens where a token names a slot
    assert torch.equal(embedding(table, ids, scale=2.5), table[ids.long()].float() * 2.5)
    chosen = torch.tensor([9, 3, 30, 1], dtype=torch.int32, device=DEV)
    from_slot = torch.tensor([-1, 2, -1, 0, 3], dtype=torch.int32, device=DEV)
    want = torch.tensor([0, 30, 5, 9, 1], device=DEV)
    assert torch.equal(embedding(table, ids, from_slot=from_slot, chosen=chosen), table[want].float())


def test_softcap_and_chosen_tokens_per_slot():
    from yalis_b200.ops.elementwise import softcap_
    from yalis_b200.ops.sampling import argmax, sample
    x = rnd(7, 1000, seed=3, scale=20.0)
    torch.testing.assert_close(softcap_(x.clone(), 8.0), 8.0 * torch.tanh(x / 8.0), rtol=1e-5, atol=1e-5)
    for vocab in (1000, 40000):                            # one block per row; 32 blocks per row and a merge
        logits = rnd(5, vocab, seed=4)
        where = torch.tensor([3, -1, 0, 6, -1], dtype=torch.int32, device=DEV)
        kept = torch.full((8,), -7, dtype=torch.int32, device=DEV)
        got = argmax(logits, scatter_index=where, scatter=kept)
        best = logits.argmax(dim=-1).tolist()
        assert got.tolist() == best
        assert kept.tolist() == [best[2], -7, -7, best[0], -7, -7, best[3], -7]
        kept.fill_(-7)
        zeros = torch.zeros(5, device=DEV)
        got = sample(logits, zeros, torch.zeros(5, dtype=torch.int32, device=DEV), zeros, torch.zeros(5, dtype=torch.int64, device=DEV),
                     torch.zeros(5, dtype=torch.int64, device=DEV), scatter_index=where, scatter=kept)
        assert got.tolist() == best and kept.tolist() == [best[2], -7, -7, best[0], -7, -7, best[3], -7]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, width, eps", [(5, 96, 1e-6), (3, 4100, 1e-5), (1, 16, 1e-2)])
def test_add_rmsnorm(dtype, n, width, eps):
    from yalis_b200.ops.elementwise import add_rmsnorm
    x = rnd(n, width, seed=1, scale=3.0)
    delta = rnd(n, width, dtype=dtype, seed=2)
    w = rnd(width, seed=3).abs() + 0.5
    h = x + delta.float()
    ref = plain.rms_norm(h, w, eps)
    x1 = x.clone()
    y = add_rmsnorm(x1, delta, w, eps, dtype)
    torch.testing.assert_close(x1, h, rtol=1e-6, atol=1e-6)              # the stream got the sum
    torch.testing.assert_close(y.float(), ref.to(dtype).float(), **tol(dtype))
    # without delta; and on chosen rows only (stream untouched)
    y0 = add_rmsnorm(x.clone(), None, w, eps, dtype)
    torch.testing.assert_close(y0.float(), plain.rms_norm(x, w, eps).to(dtype).float(), **tol(dtype))
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
    x2 = x.clone()
    yr = add_rmsnorm(x2, delta, w, eps, dtype, rows=rows)
    assert torch.equal(x2, x)
    torch.testing.assert_close(yr.float(), ref[rows.long()].to(dtype).float(), **tol(dtype))
    # split partial sums [S, n, width] are added in order
    parts = torch.stack([delta.float() * 0.25, delta.float() * 0.75]).contiguous()
    x3 = x.clone()
    add_rmsnorm(x3, parts, w, eps, dtype)
    torch.testing.assert_close(x3, x + parts[0] + parts[1], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, inter", [(4, 176), (3, 1000), (5, 100), (300, 14336 // 8)])
def test_silu_mul(dtype, n, inter):
    from yalis_b200.ops.elementwise import silu_mul
    x = rnd(n, 2 * inter, dtype=dtype, scale=2.0)
    xf = x.float()
    ref = torch.nn.functional.silu(xf[:, :inter]) * xf[:, inter:]
    torch.testing.assert_close(silu_mul(x).float(), ref.to(dtype).float(), **tol(dtype))
    ref_i = torch.nn.functional.silu(xf[:, 0::2]) * xf[:, 1::2]          # the reference's interleaved layout
    torch.testing.assert_close(silu_mul(x, interleaved=True).float(), ref_i.to(dtype).float(), **tol(dtype))


def paged_setup(n_req, lens, g, hs, page, dtype, seed=0, extra_pages=3):
    """Random K/V for requests of the given lengths scattered into shuffled pages."""
    gen = torch.Generator().manual_seed(seed)
    pages_per = [-(-l // page) for l in lens]
    num_pages = sum(pages_per) + extra_pages
    perm = torch.randperm(num_pages, generator=gen).tolist()
    width = max(pages_per) + 1
    table = torch.full((n_req, width), -1, dtype=torch.int32)
    k_pool = torch.full((num_pages, g, page, hs), float("nan"))          # unwritten places must never be read
    v_pool = torch.full((num_pages, g, page, hs), float("nan"))
    ks, vs = [], []
    it = iter(perm)
    for r, l in enumerate(lens):
        k = torch.randn(l, g, hs, generator=gen)
        v = torch.randn(l, g, hs, generator=gen)
        ks.append(k); vs.append(v)
        for i in range(pages_per[r]):
            p = next(it)
            table[r, i] = p
            n = min(page, l - i * page)
            k_pool[p, :, :n] = k[i * page:i * page + n].transpose(0, 1)
            v_pool[p, :, :n] = v[i * page:i * page + n].transpose(0, 1)
    return ks, vs, k_pool.to(dtype).to(DEV), v_pool.to(dtype).to(DEV), table.to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, g, hs, page, window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, None), (5, 5, 80, 16, None),
    (8, 2, 128, 16, None), (2, 1, 256, 32, None), (4, 2, 64, 16, 7), (4, 4, 96, 8, 33),
])
def test_paged_attention_generic(dtype, nh, g, hs, page, window):
    from yalis_b200.ops.attention import paged_attention_generic
    lens = [1, 37, 130]
    q_lens = [1, 5, 130]                                     # a decode, a portion at an offset, a whole prompt
    ks, vs, k_pool, v_pool, table = paged_setup(3, lens, g, hs, page, dtype, seed=hs)
    gen = torch.Generator().manual_seed(1)
    qs, pos, req = [], [], []
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        qs.append(torch.randn(ql, nh, hs, generator=gen))
        pos += list(range(l - ql, l))
        req += [r] * ql
    q = torch.cat(qs).to(dtype)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    req_of_token = torch.tensor(req, dtype=torch.int32, device=DEV)
    out = paged_attention_generic(q.view(-1, nh * hs).to(DEV), k_pool, v_pool, positions, req_of_token, table, nh, g, hs,
                                  window=window)
    o = 0
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        kk, vv = ks[r].to(dtype).float(), vs[r].to(dtype).float()
        ref = plain.causal_attention(q[o:o + ql].float(), kk, vv, torch.arange(l - ql, l), torch.arange(l), window=window)
        got = out[o:o + ql].float().cpu().view(ql, nh, hs)
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got, ref.to(dtype).float(), **tol(dtype))
        o += ql


def test_paged_attention_far_key_stands_out():
    """One key among hundreds, scaled so that it takes nearly all the weight, for a query far
    behind it and across many pages: the output must be that key's value."""
    from yalis_b200.ops.attention import paged_attention_generic
    nh, g, hs, page, l = 2, 1, 32, 8, 777
    ks, vs, k_pool, v_pool, table = paged_setup(1, [l], g, hs, page, torch.float32, seed=9)
    for target in (0, 7, 8, 391, l - 1):                     # first key, page edges, middle, the query itself
        q = ks[0][target, 0] * 8.0                           # aligned with that key, large
        qq = q.repeat(nh).view(1, nh * hs).to(DEV)
        out = paged_attention_generic(qq, k_pool, v_pool, torch.tensor([l - 1], dtype=torch.int32, device=DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV), table, nh, g, hs)
        ref = plain.causal_attention(q.repeat(nh).view(1, nh, hs), ks[0], vs[0], torch.tensor([l - 1]), torch.arange(l))
        torch.testing.assert_close(out.cpu().view(1, nh, hs), ref, rtol=1e-4, atol=1e-4)
        assert torch.allclose(out.cpu().view(nh, hs)[0], vs[0][target, 0], atol=5e-2)


def test_window_edge_is_exact():
    """With a window of W the key at distance W-1 is seen and the one at distance W is not."""
    from yalis_b200.ops.attention import paged_attention_generic
    nh, g, hs, page, l, w = 1, 1, 16, 4, 40, 9
    ks, vs, k_pool, v_pool, table = paged_setup(1, [l], g, hs, page, torch.float32, seed=2)
    p = l - 1
    for target, seen in ((p - w + 1, True), (p - w, False)):
        q = (ks[0][target, 0] * 20.0).view(1, hs).to(DEV)
        out = paged_attention_generic(q, k_pool, v_pool, torch.tensor([p], dtype=torch.int32, device=DEV),
                                      torch.zeros(1, dtype=torch.int32, device=DEV), table, nh, g, hs, window=w)
        close = torch.allclose(out.cpu()[0], vs[0][target, 0], atol=5e-2)
        assert close == seen


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, g, hs, page", [(4, 2, 16, 16), (3, 1, 32, 8), (5, 5, 80, 4), (8, 2, 128, 16)])
@pytest.mark.parametrize("scaled", [False, True])
def test_rope_kv_write(dtype, nh, g, hs, page, scaled):
    from yalis_b200.ops.elementwise import rope_kv_write
    from yalis_b200.parts.rotary import inverse_frequencies
    scaling = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=32) if scaled else None
    theta = 500000.0 if scaled else 10000.0
    inv = inverse_frequencies(hs, theta, scaling)
    torch.testing.assert_close(inv, plain.rope_inverse_frequencies(hs, theta, None if not scaled else scaling), rtol=0, atol=0)
    pos_list = [0, 1, 7, 8, 100, 4095, 3, 4]
    req_list = [0, 0, 0, 0, 0, 0, 1, 1]
    n = len(pos_list)
    qkv = rnd(n, (nh + 2 * g) * hs, dtype=dtype, seed=4)
    num_pages = 4096 // page + 4
    table = torch.full((2, 4096 // page), -1, dtype=torch.int32)
    gen = torch.Generator().manual_seed(0)
    perm = torch.randperm(num_pages, generator=gen)
    for i, (p, r) in enumerate(zip(pos_list, req_list)):
        table[r, p // page] = perm[(p // page) * 2 + r] if (p // page) * 2 + r < num_pages else perm[i]
    table = table.to(DEV)
    k_pool = torch.zeros(num_pages, g, page, hs, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    reqs = torch.tensor(req_list, dtype=torch.int32, device=DEV)
    before = qkv.clone()
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = rope_kv_write(qkv, positions, reqs, inv.to(DEV), k_pool, v_pool, table, nh, g, hs, bad_flag=flag)
    assert int(flag) == 0
    cos, sin = plain.rope_tables(torch.tensor(pos_list), inv)
    bq = before[:, :nh * hs].float().cpu().view(n, nh, hs)
    bk = before[:, nh * hs:(nh + g) * hs].float().cpu().view(n, g, hs)
    bv = before[:, (nh + g) * hs:].float().cpu().view(n, g, hs)
    t = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_out.float().cpu().view(n, nh, hs), plain.apply_rope(bq, cos, sin).to(dtype).float(), **t)
    assert torch.equal(qkv, before)                                       # the source row is left alone
    # the same from float32 partial sums of a split product
    parts = torch.stack([before.float() * 0.5, before.float() * 0.25, before.float() * 0.25]).contiguous()
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    q2 = rope_kv_write(parts, positions, reqs, inv.to(DEV), k2, v2, table, nh, g, hs, out_dtype=dtype, bad_flag=flag)
    torch.testing.assert_close(q2.float(), q_out.float(), **t)
    torch.testing.assert_close(k2.float(), k_pool.float(), **t)
    assert torch.equal(v2, v_pool)
    rk = plain.apply_rope(bk, cos, sin)
    for i, (p, r) in enumerate(zip(pos_list, req_list)):
        page_id, off = int(table[r, p // page]), p % page
        torch.testing.assert_close(k_pool[page_id, :, off].float().cpu(), rk[i].to(dtype).float(), **t)
        assert torch.equal(v_pool[page_id, :, off].float().cpu(), bv[i])
    assert int((k_pool != 0).any(dim=-1).sum()) <= n * g                  # nothing else was written
    # an unmapped page is flagged and skipped
    rope_kv_write(before.clone(), torch.tensor([9 * page], dtype=torch.int32, device=DEV).repeat(n)[:n], reqs * 0 + 1,
                  inv.to(DEV), k_pool, v_pool, table, nh, g, hs, bad_flag=flag)
    assert int(flag) == 2                                   # YALIS_FLAG_BAD_PAGE


def test_rope_large_positions_match_float32_table():
    """Angles are float32 products as in the reference's table: at position 100000 a float64
    angle would differ visibly; the kernel must agree with the float32 table."""
    from yalis_b200.ops.elementwise import rope_kv_write
    from yalis_b200.parts.rotary import inverse_frequencies
    nh, g, hs, page = 1, 1, 64, 16
    inv = inverse_frequencies(hs, 500000.0, None)
    pos = [100000, 131071]
    qkv = rnd(2, 3 * hs, seed=6)
    before = qkv.clone()
    table = torch.zeros(1, 131072 // page, dtype=torch.int32, device=DEV)
    pool = torch.zeros(1, g, page, hs, device=DEV)
    q = rope_kv_write(qkv, torch.tensor(pos, dtype=torch.int32, device=DEV), torch.zeros(2, dtype=torch.int32, device=DEV),
                      inv.to(DEV), pool, pool.clone(), table, nh, g, hs)
    cos, sin = plain.rope_tables(torch.tensor(pos), inv)
    ref = plain.apply_rope(before[:, :hs].cpu().view(2, 1, hs), cos, sin)
    torch.testing.assert_close(q.cpu().view(2, 1, hs), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("m, n, k", [(1, 7, 5), (33, 130, 96), (70, 64, 1000), (5, 300, 17)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(m, n, k, dtype):
    from yalis_b200.ops.linear import gemm_simt
    x, w = rnd(m, k, dtype=dtype, seed=1), rnd(n, k, dtype=dtype, seed=2)
    ref = x.double() @ w.double().T
    out = gemm_simt(x, w, out_dtype=torch.float32)
    torch.testing.assert_close(out.double(), ref, rtol=1e-5, atol=1e-4)
    out = gemm_simt(x, w)
    torch.testing.assert_close(out.double(), ref.to(dtype).double(), **(dict(rtol=1e-5, atol=1e-4) if dtype == torch.float32
                                                                        else dict(rtol=2e-2, atol=2e-2)))


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    from yalis_b200.ops.linear import gemm_simt
    x, w = rnd(67, 200, seed=1), rnd(150, 200, seed=2)
    full = gemm_simt(x, w)
    for rows in ([0], [3, 66], list(range(20, 41))):
        part = gemm_simt(x[rows].contiguous(), w)
        assert torch.equal(part, full[rows])                               # the same bits


@pytest.mark.parametrize("m, n, k", [(1, 512, 96), (24, 300, 64), (130, 1000, 256)])
def test_linear_bf16_against_float32(m, n, k):
    from yalis_b200.ops.linear import linear
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=1), rnd(n, k, dtype=torch.bfloat16, seed=2)
    ref = x.float() @ w.float().T
    torch.testing.assert_close(linear(x, w, out_dtype=torch.float32), ref, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(linear(x, w).float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("rows, vocab", [(1, 5), (3, 1000), (2, 128256)])
def test_argmax_ties_go_to_the_lowest_index(rows, vocab):
    from yalis_b200.ops.sampling import argmax
    x = rnd(rows, vocab, seed=3)
    assert argmax(x).tolist() == x.argmax(dim=-1).tolist()
    x[:, :] = 0.0
    x[0, vocab // 2] = 1.0
    x[0, vocab - 1] = 1.0
    got = argmax(x).tolist()
    assert got[0] == vocab // 2 and all(g == 0 for g in got[1:])


def draws(logits_row, temperature, top_k, top_p, n, seed=77, rows_per_call=None):
    """n draws (draw numbers 0..n-1) from one row; in calls of rows_per_call rows each, since the
    number of rows decides how many blocks walk a wide row."""
    from yalis_b200.ops.sampling import sample
    vocab = logits_row.numel()
    per = rows_per_call or n
    logits = logits_row.view(1, vocab).repeat(per, 1).contiguous().to(DEV)
    f = lambda v, dt: torch.full((per,), v, dtype=dt, device=DEV)
    args = (f(temperature, torch.float32), f(top_k or 0, torch.int32), f(top_p, torch.float32), f(seed, torch.int64))
    out = [sample(logits, *args, torch.arange(at, at + per, dtype=torch.int64, device=DEV)) for at in range(0, n, per)]
    return torch.cat(out)[:n].cpu()


@pytest.mark.parametrize("temperature, top_k, top_p", [(1.0, None, 1.0), (0.7, None, 1.0), (1.0, 5, 1.0), (1.3, None, 0.8),
                                                       (0.9, 11, 0.6), (0.0, None, 0.9)])
def test_sampler_follows_the_reference_distribution(temperature, top_k, top_p):
    """Chi-square of 20000 draws against the probabilities the reference samples from."""
    vocab = 40
    logits = torch.randn(vocab, generator=torch.Generator().manual_seed(5)) * 2.0
    n = 20000
    out = draws(logits, temperature, top_k, top_p, n)
    p = plain.sampling_distribution(logits, temperature, top_k, top_p).double().numpy()
    counts = np.bincount(out.numpy(), minlength=vocab).astype(np.float64)
    assert counts[p == 0].sum() == 0                                        # nothing outside the kept set
    keep = p > 0
    chi2 = (((counts[keep] - n * p[keep]) ** 2) / (n * p[keep])).sum()
    dof = keep.sum() - 1
    assert chi2 < dof + 5 * math.sqrt(2 * max(dof, 1)) + 10, (chi2, dof)


def test_sampler_greedy_rule_and_reproducibility():
    from yalis_b200.ops.sampling import sample
    vocab = 1000
    logits = rnd(4, vocab, seed=1)
    f = lambda vals, dt: torch.tensor(vals, dtype=dt, device=DEV)
    temp, tk, tp = f([0.0, 1.0, 1.0, 0.0], torch.float32), f([0, 0, 1, 0], torch.int32), f([0.0, 0.0, 1.0, 1.0], torch.float32)
    seed, draw = f([1, 2, 3, 4], torch.int64), f([0, 0, 0, 0], torch.int64)
    a = sample(logits, temp, tk, tp, seed, draw).tolist()
    best = logits.argmax(dim=-1).tolist()
    assert a[0] == best[0]          # temperature 0 and top_p 0: greedy
    assert a[1] == best[1]          # top_p 0 keeps the first only
    assert a[2] == best[2]          # top_k 1
    b = sample(logits, temp, tk, tp, seed, draw).tolist()
    assert a == b                   # same seed and draw index: same token
    # a row's draw does not depend on the rest of the batch
    one = sample(logits[3:4].contiguous(), temp[3:4].contiguous(), tk[3:4].contiguous(), tp[3:4].contiguous(),
                 seed[3:4].contiguous(), draw[3:4].contiguous()).tolist()
    assert one[0] == a[3]
    many = {int(sample(logits[3:4].contiguous(), temp[3:4].contiguous(), tk[3:4].contiguous(), tp[3:4].contiguous(),
                       seed[3:4].contiguous(), f([d], torch.int64))) for d in range(30)}
    assert len(many) > 5            # other draw indices give other tokens


def test_top_k_and_top_p_cuts_on_clear_gaps():
    """Logits with wide gaps: the kept sets are exactly the reference's."""
    logits = torch.tensor([5.0, 4.0, 3.0, -2.0, -3.0, 1.0, 0.0, -9.0])
    for temperature, top_k, top_p in ((1.0, 3, 1.0), (1.0, None, 0.7), (1.0, None, 0.95), (2.0, 4, 0.9), (1.0, None, 0.2)):
        p = plain.sampling_distribution(logits, temperature, top_k, top_p)
        seen = set(draws(logits, temperature, top_k, top_p, 4000).tolist())
        assert seen == {i for i in range(8) if p[i] > 1e-4}, (temperature, top_k, top_p, seen)


def test_cuts_of_a_wide_row_whose_blocks_each_see_a_slice():
    """A row of 50,001 entries is walked by eight blocks: the entries that matter lie at the first
    and last index, on both sides of slice edges and in the ragged tail; the rest carry no mass."""
    vocab = 50001
    per = ((vocab + 7) // 8 + 3) & ~3
    at = [0, per - 1, per, 3 * per + 1, 4 * per - 1, 7 * per, vocab - 2, vocab - 1]
    values = [5.0, 4.0, 3.0, -2.0, -3.0, 1.0, 0.0, -9.0]
    logits = torch.randn(vocab, generator=torch.Generator().manual_seed(9)) * 0.5 - 40.0
    logits[at] = torch.tensor(values)
    for temperature, top_k, top_p in ((1.0, 3, 1.0), (1.0, None, 0.7), (1.0, None, 0.95), (2.0, 4, 0.9), (1.0, None, 0.2),
                                      (3.0, 7, 1.0)):
        p = plain.sampling_distribution(logits, temperature, top_k, top_p)
        one_block = draws(logits, temperature, top_k, top_p, 3000)
        seen = set(one_block.tolist())
        assert seen <= set(at), (temperature, top_k, top_p, seen - set(at))
        assert seen == {i for i in at if p[i] > 1e-4}, (temperature, top_k, top_p, seen)
        for rows in (16, 32, 64):                                           # eight, four and two blocks per row
            assert torch.equal(draws(logits, temperature, top_k, top_p, 3000, rows_per_call=rows), one_block), rows


@pytest.mark.parametrize("vocab, top_k, top_p, temperature", [(128256, 50, 0.9, 0.8), (16384, None, 0.6, 1.0),
                                                             (100003, 200, 1.0, 1.5)])
def test_wide_rows_draw_only_what_the_reference_keeps(vocab, top_k, top_p, temperature):
    logits = torch.randn(vocab, generator=torch.Generator().manual_seed(vocab)) * 3.0
    p = plain.sampling_distribution(logits, temperature, top_k, top_p)
    out = draws(logits, temperature, top_k, top_p, 1500)
    assert bool((p[out] > 0).all())
    likely = {int(i) for i in torch.nonzero(p > 0.02).flatten()}
    assert likely <= set(out.tolist())
    counts = torch.bincount(out, minlength=vocab).double() / out.numel()
    top = torch.topk(p, 5).indices
    assert float((counts[top] - p[top].double()).abs().max()) < 0.05
    for rows in (8, 24, 48):                                                # eight, four and two blocks per row
        assert torch.equal(draws(logits, temperature, top_k, top_p, 1500, rows_per_call=rows), out), rows


@pytest.mark.parametrize("nh, g, hs, page, window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, None), (5, 5, 80, 16, None), (8, 2, 128, 16, None),
    (2, 1, 256, 32, None), (4, 2, 64, 16, 7), (4, 4, 96, 8, 33), (32, 1, 64, 16, None), (12, 4, 112, 2, None),
    (6, 2, 160, 64, 100), (3, 3, 192, 16, None), (2, 2, 224, 16, None),
])
@pytest.mark.parametrize("mode", ["mixed", "decode", "decode_split"])
def test_paged_attention_mma_against_plain_and_generic(nh, g, hs, page, window, mode):
    """The tensor-core kernel: a decode, a portion at an offset and a whole prompt in one
    launch; decode-only batches with and without key splitting; against the plain float32
    attention and against the exact generic kernel."""
    from yalis_b200.ops.attention import paged_attention_generic, paged_attention_mma
    dtype = torch.bfloat16
    if mode == "mixed":
        lens, q_lens = [1, 37, 130, 300], [1, 5, 130, 67]
    else:
        lens, q_lens = [1, 64, 65, 130, 517], [1, 1, 1, 1, 1]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=hs + nh)
    gen = torch.Generator().manual_seed(1)
    qs, pos, req, q_start = [], [], [], [0]
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        qs.append(torch.randn(ql, nh, hs, generator=gen))
        pos += list(range(l - ql, l))
        req += [r] * ql
        q_start.append(q_start[-1] + ql)
    q = torch.cat(qs).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req_of_token, q_start_d = i32(pos), i32(req), i32(q_start)
    qd = q.view(-1, nh * hs).to(DEV)
    splits = 5 if mode == "decode_split" else 1
    if mode != "mixed" and nh // g > 16:
        splits = 1
    out = paged_attention_mma(qd, k_pool, v_pool, positions, q_start_d, req_of_token, table, max(q_lens), nh, g, hs,
                              window=window, n_splits=splits if nh // g <= 16 else 1)
    gen_out = paged_attention_generic(qd, k_pool, v_pool, positions, req_of_token, table, nh, g, hs, window=window)
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), gen_out.float(), rtol=2e-2, atol=2e-2)
    o = 0
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        kk, vv = ks[r].to(dtype).float(), vs[r].to(dtype).float()
        ref = plain.causal_attention(q[o:o + ql].float(), kk, vv, torch.arange(l - ql, l), torch.arange(l), window=window)
        torch.testing.assert_close(out[o:o + ql].float().cpu().view(ql, nh, hs), ref, rtol=2e-2, atol=2e-2)
        o += ql


def test_paged_attention_mma_far_key_and_padding_rows():
    """A far key that takes nearly all the weight, through the tensor-core kernel in split
    decode mode; and padding tokens (request index -1) are left alone."""
    from yalis_b200.ops.attention import paged_attention_mma
    nh, g, hs, page, l = 8, 2, 64, 16, 1500
    ks, vs, k_pool, v_pool, table = paged_setup(1, [l], g, hs, page, torch.bfloat16, seed=9)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for target in (0, 15, 16, 777, l - 1):
        q = torch.cat([ks[0][target, h // (nh // g)] * 6.0 for h in range(nh)]).view(1, nh * hs)
        qq = torch.cat([q, torch.zeros(3, nh * hs)]).to(torch.bfloat16).to(DEV)         # three padding rows behind
        out = torch.full((4, nh * hs), 7.0, dtype=torch.bfloat16, device=DEV)
        paged_attention_mma(qq, k_pool, v_pool, i32([l - 1, 0, 0, 0]), i32([0, 1]), i32([0, -1, -1, -1]), table, 1, nh, g, hs,
                            n_splits=7, out=out)
        got = out[0].float().cpu().view(nh, hs)
        for h in range(nh):
            assert torch.allclose(got[h], vs[0][target, h // (nh // g)].to(torch.bfloat16).float(), atol=6e-2), (target, h)
        assert torch.all(out[1:] == 7.0)


@pytest.mark.parametrize("m, n, k", [(1, 128, 64), (8, 384, 1024), (17, 200, 520), (64, 1000, 4096), (100, 130, 72),
                                     (256, 512, 2048), (3, 4096, 14336)])
def test_gemm_wstream_tcgen05(m, n, k):
    """The tcgen05 weight-streaming product against a float32 product of the same bfloat16
    operands: whole and as split partial sums; its rows do not depend on the batch."""
    from yalis_b200.ops.linear import gemm_simt, gemm_wstream, wstream_error_flag, wstream_splits
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=1, scale=0.5), rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.5)
    ref = gemm_simt(x, w, out_dtype=torch.float32)
    out32 = gemm_wstream(x, w, out_dtype=torch.float32)
    torch.testing.assert_close(out32, ref, rtol=1e-4, atol=1e-3 * math.sqrt(k / 64))
    out16 = gemm_wstream(x, w)
    torch.testing.assert_close(out16.float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2)
    parts = gemm_wstream(x, w, split=True)
    assert parts.shape == (wstream_splits(n, k), m, n) and parts.dtype == torch.float32
    torch.testing.assert_close(parts.sum(0), ref, rtol=1e-4, atol=1e-3 * math.sqrt(k / 64))
    one = gemm_wstream(x[m - 1:].contiguous(), w, out_dtype=torch.float32)
    assert torch.equal(one[0], out32[m - 1])                               # the same bits alone and in the batch
    assert int(wstream_error_flag(DEV)) == 0


@pytest.mark.parametrize("m, inter, k", [(1, 64, 64), (8, 448, 256), (5, 200, 136), (16, 1000, 72), (17, 130, 512), (64, 320, 192),
                                         (100, 96, 1024), (256, 192, 64)])
def test_gemm_wstream_silu_has_the_bits_of_product_then_activation(m, inter, k):
    """The gated activation fused into the weight-streaming product: tiles of 64 gate and 64 up rows,
    sizes that end inside a tile, against the unfused pair of kernels (same bits) and float32."""
    from yalis_b200.ops.linear import gemm_wstream, gemm_wstream_silu, wstream_error_flag
    from yalis_b200.ops.elementwise import silu_mul
    x = rnd(m, k, dtype=torch.bfloat16, seed=m + k)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=inter, scale=1.0 / math.sqrt(k))
    fused = gemm_wstream_silu(x, w)
    pair = silu_mul(gemm_wstream(x, w))
    assert fused.shape == (m, inter) and torch.equal(fused, pair)
    prod = x.float().cpu() @ w.float().cpu().t()
    gate, up = prod[:, :inter], prod[:, inter:]
    ref = gate / (1.0 + torch.exp(-gate)) * up        # the activation of plain.swiglu, written out
    torch.testing.assert_close(fused.float().cpu(), ref, rtol=3e-2, atol=3e-2)
    assert int(wstream_error_flag(DEV)) == 0


@pytest.mark.parametrize("nh, g, hs, page", [(32, 8, 128, 16), (8, 2, 64, 8), (4, 4, 64, 32), (16, 1, 128, 64), (6, 2, 192, 16),
                                             (2, 1, 256, 16), (5, 5, 128, 16)])
@pytest.mark.parametrize("splits, early", [(1, False), (3, True), (8, False), (8, True), (1, True), (11, True), (20, False)])
def test_decode_attention_tma_against_plain_and_generic(nh, g, hs, page, splits, early):
    """The TMA-fed decode kernel: lengths around tile and page edges, pools poisoned with NaN
    where nothing was written, against the plain float32 attention and the exact kernel."""
    from yalis_b200.ops.attention import decode_attention_tma, paged_attention_generic
    dtype = torch.bfloat16
    lens = [1, 15, 16, 17, 63, 64, 65, 130, 517, 1200]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=hs + nh + page)
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(len(lens), nh, hs, generator=gen).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, q_start, req = i32([l - 1 for l in lens]), i32(list(range(len(lens) + 1))), i32(list(range(len(lens))))
    qd = q.view(-1, nh * hs).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()      # early fetching wants the pool and the index arrays complete before the launch
    out = decode_attention_tma(qd, k_pool, v_pool, positions, q_start, table, nh, g, hs, n_splits=splits, error_flag=flag,
                               early_fetch=early)
    assert int(flag) == 0 and not torch.isnan(out.float()).any()
    ref_gen = paged_attention_generic(qd, k_pool, v_pool, positions, req, table, nh, g, hs)
    torch.testing.assert_close(out.float(), ref_gen.float(), rtol=2e-2, atol=2e-2)
    for r, l in enumerate(lens):
        ref = plain.causal_attention(q[r:r + 1].float(), ks[r].to(dtype).float(), vs[r].to(dtype).float(),
                                     torch.tensor([l - 1]), torch.arange(l))
        torch.testing.assert_close(out[r].float().cpu().view(1, nh, hs), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nh, g, hs, page", [(32, 8, 128, 16), (8, 2, 64, 8), (4, 4, 64, 32), (16, 1, 128, 64), (6, 2, 192, 16),
                                             (2, 1, 256, 16), (5, 5, 128, 16)])
@pytest.mark.parametrize("n_blocks", [1, 2, 5, 13, 64, 296, 5000])
def test_decode_attention_lean_against_plain_and_generic(nh, g, hs, page, n_blocks):
    """The decode kernel that deals the tiles of all (request, KV head) pairs to a fixed grid: one block that
    walks everything, a few blocks whose borders cut pairs (a long request spans several), about as many
    blocks as tiles, and more blocks than tiles; a request without a token in the middle; twice in a row
    (the tickets must come back to zero)."""
    from yalis_b200.ops.attention import decode_attention_lean, paged_attention_generic
    dtype = torch.bfloat16
    lens = [1, 15, 16, 17, 63, 64, 65, 130, 517, 1200, 2, 64]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=hs + nh + page)
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(len(lens), nh, hs, generator=gen).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req = i32([l - 1 for l in lens]), i32(list(range(len(lens))))
    q_start = i32(list(range(len(lens) + 1)))
    qd = q.view(-1, nh * hs).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref_gen = paged_attention_generic(qd, k_pool, v_pool, positions, req, table, nh, g, hs)
    early = n_blocks % 2 == 1     # fetching before the preceding kernel has finished wants everything complete: it is
    torch.cuda.synchronize()
    for _ in range(2):
        out = decode_attention_lean(qd, k_pool, v_pool, positions, q_start, table, nh, g, hs, n_blocks=n_blocks,
                                    error_flag=flag, early_fetch=early)
        assert int(flag) == 0 and not torch.isnan(out.float()).any()
        torch.testing.assert_close(out.float(), ref_gen.float(), rtol=2e-2, atol=2e-2)
    for r, l in enumerate(lens):
        ref = plain.causal_attention(q[r:r + 1].float(), ks[r].to(dtype).float(), vs[r].to(dtype).float(),
                                     torch.tensor([l - 1]), torch.arange(l))
        torch.testing.assert_close(out[r].float().cpu().view(1, nh, hs), ref, rtol=2e-2, atol=2e-2)
    # Requests 3 and 7 bring no token (padding of a captured batch): the others' results do not move.
    keep = [r for r in range(len(lens)) if r not in (3, 7)]
    starts, at = [], 0
    for r in range(len(lens)):
        starts.append(at)
        at += 1 if r in keep else 0
    starts.append(at)
    out2 = decode_attention_lean(qd[keep].contiguous(), k_pool, v_pool, positions[keep].contiguous(), i32(starts), table,
                                 nh, g, hs, n_blocks=n_blocks, error_flag=flag)
    assert int(flag) == 0
    if n_blocks in (1, 5000):       # every pair whole in both runs: the same bits
        assert torch.equal(out2, out[keep])
    torch.testing.assert_close(out2.float(), ref_gen[keep].float(), rtol=2e-2, atol=2e-2)


def test_decode_attention_lean_many_requests_and_a_far_key():
    """600 requests of mixed lengths on the engine's grid; in some, one far key is made to carry all the weight
    (a tile dropped or read from the wrong pair would show)."""
    from yalis_b200.ops.attention import decode_attention_lean, decode_lean_blocks, paged_attention_generic
    nh, g, hs, page, dtype = 8, 4, 128, 16, torch.bfloat16
    gen = torch.Generator().manual_seed(11)
    lens = [int(x) for x in torch.randint(1, 400, (600,), generator=gen)]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=5)
    q = torch.randn(len(lens), nh, hs, generator=gen).to(dtype)
    marked = {}
    for r in range(0, len(lens), 37):
        target = int(torch.randint(0, lens[r], (1,), generator=gen))
        marked[r] = target
        for h in range(nh):
            q[r, h] = (ks[r][target, h // (nh // g)] * 6.0).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req, q_start = i32([l - 1 for l in lens]), i32(list(range(len(lens)))), i32(list(range(len(lens) + 1)))
    qd = q.view(-1, nh * hs).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = decode_attention_lean(qd, k_pool, v_pool, positions, q_start, table, nh, g, hs, error_flag=flag)
    assert int(flag) == 0 and decode_lean_blocks(hs) < len(lens) * g
    ref = paged_attention_generic(qd, k_pool, v_pool, positions, req, table, nh, g, hs)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    for r, target in marked.items():
        got = out[r].float().cpu().view(nh, hs)
        for h in range(nh):
            assert torch.allclose(got[h], vs[r][target, h // (nh // g)].to(dtype).float(), atol=8e-2), (r, h)


@pytest.mark.parametrize("nh, g, hs, page", [(32, 8, 128, 64), (8, 2, 64, 8), (6, 2, 192, 16), (2, 1, 256, 32), (5, 5, 128, 16)])
@pytest.mark.parametrize("parts, splits, rotate", [(1, 1, True), (3, 4, True), (2, 8, False), (0, 3, True), (3, 11, True)])
def test_decode_attention_tma_fused_has_the_bits_of_rotary_kernel_then_attention(nh, g, hs, page, parts, splits, rotate):
    """The decode kernel that rotates Q and the new K itself and stores K, V: same output and same cache
    as the rotary / cache-write kernel followed by the plain decode kernel; lengths at page and tile edges;
    bfloat16 rows (parts 0) and float32 partial sums; and without storing (a cache that another layer filled)."""
    from yalis_b200.ops.attention import decode_attention_tma, decode_attention_tma_fused
    from yalis_b200.ops.elementwise import rope_kv_write
    from yalis_b200.parts.rotary import inverse_frequencies
    dtype = torch.bfloat16
    lens = [1, 16, 17, 64, 65, 128, 129, 517]
    n = len(lens)
    _, _, k_pool, v_pool, table = paged_setup(n, lens, g, hs, page, dtype, seed=hs + nh + page + parts)
    width = (nh + 2 * g) * hs
    if parts == 0:
        qkv = rnd(n, width, dtype=dtype, seed=5)
    else:
        qkv = rnd(parts, n, width, seed=5)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, q_start, req = i32([l - 1 for l in lens]), i32(list(range(n + 1))), i32(list(range(n)))
    inv = inverse_frequencies(hs, 10000.0, None).to(DEV) if rotate else None
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    k1, v1 = k_pool.clone(), v_pool.clone()
    q = rope_kv_write(qkv, positions, req, inv, k1, v1, table, nh, g, hs, out_dtype=dtype, bad_flag=flag)
    ref = decode_attention_tma(q, k1, v1, positions, q_start, table, nh, g, hs, n_splits=splits, error_flag=flag)
    k2, v2 = k_pool.clone(), v_pool.clone()
    torch.cuda.synchronize()
    out = decode_attention_tma_fused(qkv, inv, True, k2, v2, positions, q_start, table, nh, g, hs, n_splits=splits,
                                     error_flag=flag, early_fetch=True)
    assert int(flag) == 0
    assert torch.equal(out, ref)
    # pools: equal wherever something was written (both started from the same poisoned pools)
    assert torch.equal(torch.nan_to_num(k2.float(), nan=7.0), torch.nan_to_num(k1.float(), nan=7.0))
    assert torch.equal(torch.nan_to_num(v2.float(), nan=7.0), torch.nan_to_num(v1.float(), nan=7.0))
    # a cache that already holds this step's key and value (filled by another layer): nothing is stored
    k3, v3 = k1.clone(), v1.clone()
    out3 = decode_attention_tma_fused(qkv, inv, False, k3, v3, positions, q_start, table, nh, g, hs, n_splits=splits,
                                      error_flag=flag)
    assert int(flag) == 0 and torch.equal(out3, ref)
    assert torch.equal(torch.nan_to_num(k3.float(), nan=7.0), torch.nan_to_num(k1.float(), nan=7.0))


def test_decode_attention_tma_far_key_and_padding_requests():
    """A far key with nearly all the weight at page and tile edges; requests without tokens
    (padding of a captured batch) are left alone."""
    from yalis_b200.ops.attention import decode_attention_tma
    nh, g, hs, page, l = 8, 2, 128, 16, 2000
    ks, vs, k_pool, v_pool, table = paged_setup(1, [l], g, hs, page, torch.bfloat16, seed=11)
    table = torch.cat([table, torch.full_like(table, -1), torch.full_like(table, -1)])
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for target in (0, 15, 16, 63, 64, 1023, l - 1):
        q = torch.cat([ks[0][target, h // (nh // g)] * 4.0 for h in range(nh)]).view(1, nh * hs)
        qq = torch.cat([q, torch.zeros(2, nh * hs)]).to(torch.bfloat16).to(DEV)
        out = torch.full((3, nh * hs), 7.0, dtype=torch.bfloat16, device=DEV)
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        pos, qs = i32([l - 1, 0, 0]), i32([0, 1, 1, 1])
        torch.cuda.synchronize()
        decode_attention_tma(qq, k_pool, v_pool, pos, qs, table, nh, g, hs, n_splits=6, error_flag=flag, out=out,
                             early_fetch=target % 2 == 0)
        got = out[0].float().cpu().view(nh, hs)
        for h in range(nh):
            assert torch.allclose(got[h], vs[0][target, h // (nh // g)].to(torch.bfloat16).float(), atol=6e-2), (target, h)
        assert torch.all(out[1:] == 7.0) and int(flag) == 0


@pytest.mark.parametrize("hs", [48, 20, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_kv_write_many_tokens(dtype, hs):
    """Steps with many tokens take the one-block-per-token variants (four pairs per thread when the
    head size is a multiple of 8, else one): same results."""
    from yalis_b200.ops.elementwise import rope_kv_write
    from yalis_b200.parts.rotary import inverse_frequencies
    nh, g, page, n = 6, 2, 8, 333
    inv = inverse_frequencies(hs, 10000.0, None)
    qkv = rnd(n, (nh + 2 * g) * hs, dtype=dtype, seed=8)
    pos_list = list(range(5, 5 + n))
    num_pages = (5 + n) // page + 2
    table = torch.arange(num_pages, dtype=torch.int32).flip(0).view(1, -1).contiguous().to(DEV)
    k_pool = torch.zeros(num_pages, g, page, hs, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = rope_kv_write(qkv, torch.tensor(pos_list, dtype=torch.int32, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                          inv.to(DEV), k_pool, v_pool, table, nh, g, hs, bad_flag=flag)
    assert int(flag) == 0
    cos, sin = plain.rope_tables(torch.tensor(pos_list), inv)
    src = qkv.float().cpu()
    t = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(q_out.float().cpu().view(n, nh, hs), plain.apply_rope(src[:, :nh * hs].view(n, nh, hs), cos, sin).to(dtype).float(), **t)
    rk = plain.apply_rope(src[:, nh * hs:(nh + g) * hs].view(n, g, hs), cos, sin).to(dtype).float()
    tab = table.cpu()[0]
    for i in (0, 1, 7, 100, n - 1):
        p = pos_list[i]
        torch.testing.assert_close(k_pool[int(tab[p // page]), :, p % page].float().cpu(), rk[i], **t)
        assert torch.equal(v_pool[int(tab[p // page]), :, p % page].float().cpu(), src[i, (nh + g) * hs:].view(g, hs).to(dtype).float())
    # the same rows as three float32 partial sums of a split product
    parts = torch.stack([qkv.float() * 0.5, qkv.float() * 0.25, qkv.float() * 0.25]).contiguous()
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    q2 = rope_kv_write(parts, torch.tensor(pos_list, dtype=torch.int32, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV),
                       inv.to(DEV), k2, v2, table, nh, g, hs, out_dtype=dtype, bad_flag=flag)
    assert int(flag) == 0
    assert torch.equal(q2, q_out) and torch.equal(k2, k_pool) and torch.equal(v2, v_pool)   # the halves and quarters add exactly


@pytest.mark.parametrize("nh, g, hs, page", [(8, 2, 128, 16), (4, 4, 64, 8), (6, 2, 128, 32), (3, 1, 64, 64), (32, 8, 128, 16),
                                             (5, 1, 128, 128)])
@pytest.mark.parametrize("kv_splits, tiles_per_split", [(1, 1), (2, 1), (3, 2), (5, 1), (16, 1), (4, 3), (2, 5)])
def test_prefill_attention_tcgen05_against_plain_and_generic(nh, g, hs, page, kv_splits, tiles_per_split):
    """The tcgen05 prompt kernel: a whole prompt, a portion at an offset that ends inside a page,
    a short portion and a decode token in one launch; pools poisoned with NaN where nothing was
    written; against the plain float32 attention and the exact kernel.  With key splits: shares that end at
    causal edges, shares of a single tile, more room for shares than a request has tiles, and limits (3 or 5 key
    tiles per share) under which some tiles of queries are divided and others finished by one block."""
    from yalis_b200.ops.attention import paged_attention_generic, prefill_attention_tcgen05
    dtype = torch.bfloat16
    lens, q_lens = [300, 517, 40, 130, 1], [300, 67, 33, 128, 1]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=hs + nh)
    gen = torch.Generator().manual_seed(1)
    qs, pos, req, q_start = [], [], [], [0]
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        qs.append(torch.randn(ql, nh, hs, generator=gen))
        pos += list(range(l - ql, l))
        req += [r] * ql
        q_start.append(q_start[-1] + ql)
    q = torch.cat(qs).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req_of_token, q_start_d = i32(pos), i32(req), i32(q_start)
    qd = q.view(-1, nh * hs).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = prefill_attention_tcgen05(qd, k_pool, v_pool, positions, q_start_d, table, max(q_lens), nh, g, hs, error_flag=flag,
                                    kv_splits=kv_splits, tiles_per_split=tiles_per_split)
    torch.cuda.synchronize()
    assert int(flag) == 0
    assert not torch.isnan(out.float()).any()
    gen_out = paged_attention_generic(qd, k_pool, v_pool, positions, req_of_token, table, nh, g, hs)
    torch.testing.assert_close(out.float(), gen_out.float(), rtol=2e-2, atol=2e-2)
    o = 0
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        kk, vv = ks[r].to(dtype).float(), vs[r].to(dtype).float()
        ref = plain.causal_attention(q[o:o + ql].float(), kk, vv, torch.arange(l - ql, l), torch.arange(l))
        torch.testing.assert_close(out[o:o + ql].float().cpu().view(ql, nh, hs), ref, rtol=2e-2, atol=2e-2)
        o += ql


@pytest.mark.parametrize("nh, g, hs, page", [(8, 2, 128, 16), (6, 2, 64, 8), (32, 8, 128, 64)])
@pytest.mark.parametrize("kv_splits, tiles_per_split", [(1, 1), (3, 2)])
def test_mixed_step_with_its_decoding_requests_in_the_decode_kernel(nh, g, hs, page, kv_splits, tiles_per_split):
    """A step of prompt portions and decoding requests: the decode kernel that deals tiles to a fixed grid takes
    the requests that bring one token, the tcgen05 prompt kernel the others, both into one output; neither
    touches the other's rows (the output starts as NaN and ends without)."""
    from yalis_b200.ops.attention import decode_attention_lean, paged_attention_generic, prefill_attention_tcgen05
    dtype = torch.bfloat16
    lens, q_lens = [300, 517, 40, 700, 1, 90, 200], [300, 67, 33, 1, 1, 1, 2]
    ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, dtype, seed=hs + nh)
    gen = torch.Generator().manual_seed(1)
    qs, pos, req, q_start = [], [], [], [0]
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        qs.append(torch.randn(ql, nh, hs, generator=gen))
        pos += list(range(l - ql, l))
        req += [r] * ql
        q_start.append(q_start[-1] + ql)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req_of_token, q_start_d = i32(pos), i32(req), i32(q_start)
    qd = torch.cat(qs).to(dtype).view(-1, nh * hs).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((qd.shape[0], nh * hs), float("nan"), dtype=dtype, device=DEV)
    decode_attention_lean(qd, k_pool, v_pool, positions, q_start_d, table, nh, g, hs, n_blocks=5, error_flag=flag, out=out,
                          only_single=True)
    single_rows = [q_start[r] for r, ql in enumerate(q_lens) if ql == 1]
    written = ~torch.isnan(out.float()).any(dim=1).cpu()
    assert sorted(torch.nonzero(written).flatten().tolist()) == single_rows
    prefill_attention_tcgen05(qd, k_pool, v_pool, positions, q_start_d, table, max(q_lens), nh, g, hs, error_flag=flag, out=out,
                              kv_splits=kv_splits, tiles_per_split=tiles_per_split, skip_single=True)
    torch.cuda.synchronize()
    assert int(flag) == 0 and not torch.isnan(out.float()).any()
    ref = paged_attention_generic(qd, k_pool, v_pool, positions, req_of_token, table, nh, g, hs)
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("kv_splits, tiles_per_split, skip_single", [(1, 1, False), (1, 1, True), (2, 1, True), (3, 2, False)])
def test_prefill_attention_tcgen05_many_requests(kv_splits, tiles_per_split, skip_single):
    """75 requests in one launch (more than the 32 whose tiles a warp adds up at a time), some with one token, one
    with none: more work items than resident blocks, each block finding the request of its tile from the token
    ranges; against the exact kernel.  With ``skip_single`` the rows of one-token requests are left as they were."""
    from yalis_b200.ops.attention import paged_attention_generic, prefill_attention_tcgen05
    nh, g, hs, page, dtype = 8, 4, 64, 16, torch.bfloat16          # 75 tiles and more x 4 KV heads: over 296 items
    rng = torch.Generator().manual_seed(77)
    n_req = 75
    q_lens = [[1, 2, 17, 40, 33, 1][int(torch.randint(0, 6, (1,), generator=rng))] for _ in range(n_req)]
    q_lens[40] = 0                                           # a request that brings nothing (as padding does)
    lens = [ql + int(torch.randint(0, 180, (1,), generator=rng)) for ql in q_lens]
    lens[40] = 5
    ks, vs, k_pool, v_pool, table = paged_setup(n_req, lens, g, hs, page, dtype, seed=5)
    pos, req, q_start = [], [], [0]
    for r, (l, ql) in enumerate(zip(lens, q_lens)):
        pos += list(range(l - ql, l))
        req += [r] * ql
        q_start.append(q_start[-1] + ql)
    n = q_start[-1]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    positions, req_of_token, q_start_d = i32(pos), i32(req), i32(q_start)
    qd = torch.randn(n, nh * hs, generator=rng).to(dtype).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((n, nh * hs), 7.0, dtype=dtype, device=DEV)
    prefill_attention_tcgen05(qd, k_pool, v_pool, positions, q_start_d, table, max(q_lens), nh, g, hs, error_flag=flag, out=out,
                              kv_splits=kv_splits, tiles_per_split=tiles_per_split, skip_single=skip_single)
    torch.cuda.synchronize()
    assert int(flag) == 0
    ref = paged_attention_generic(qd, k_pool, v_pool, positions, req_of_token, table, nh, g, hs)
    single = torch.zeros(n, dtype=torch.bool)
    for r, ql in enumerate(q_lens):
        if ql == 1:
            single[q_start[r]] = True
    if skip_single:
        assert torch.all(out[single.to(DEV)] == 7.0)         # untouched
        keep = (~single).to(DEV)
        torch.testing.assert_close(out[keep].float(), ref[keep].float(), rtol=2e-2, atol=2e-2)
    else:
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_prefill_attention_tcgen05_random_steps(seed):
    """Random steps (head counts, page sizes, 1 to 90 requests of 1 to 700 tokens behind up to 3,000 cached ones,
    keys divided or not, one-token requests skipped or not), several launches each on the same counters of work
    items: every launch against the exact kernel, and no bounded wait may run out."""
    import random
    from yalis_b200.ops.attention import paged_attention_generic, prefill_attention_tcgen05
    rng = random.Random(seed)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    for trial in range(14):
        nh, g, hs = rng.choice([(32, 8, 128), (8, 2, 64), (24, 8, 128), (6, 2, 128), (4, 4, 64), (5, 1, 128)])
        page = rng.choice([8, 16, 32, 64, 128])
        q_lens = [rng.choice([1, 1, 2, 17, 33, 64, 200, 700]) for _ in range(rng.choice([1, 2, 5, 40, 90]))]
        if sum(q_lens) > 6000:
            q_lens = q_lens[:8]
        lens = [q + rng.choice([0, 0, 3, 100, 900, 3000]) for q in q_lens]
        ks, vs, k_pool, v_pool, table = paged_setup(len(lens), lens, g, hs, page, torch.bfloat16, seed=seed * 100 + trial)
        pos, req, q_start = [], [], [0]
        for r, (l, ql) in enumerate(zip(lens, q_lens)):
            pos += list(range(l - ql, l))
            req += [r] * ql
            q_start.append(q_start[-1] + ql)
        n = q_start[-1]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        positions, req_of_token, q_start_d = i32(pos), i32(req), i32(q_start)
        gen = torch.Generator().manual_seed(trial)
        qd = torch.randn(n, nh * hs, generator=gen).to(torch.bfloat16).to(DEV)
        splits, limit = rng.choice([(1, 1), (1, 1), (2, 1), (3, 2), (4, 16), (8, 4)])
        skip = rng.random() < 0.3
        ref = paged_attention_generic(qd, k_pool, v_pool, positions, req_of_token, table, nh, g, hs)
        keep = torch.tensor([not (skip and q_lens[r] == 1) for r in req], dtype=torch.bool, device=DEV)
        for launch in range(3):
            out = torch.full((n, nh * hs), 3.0, dtype=torch.bfloat16, device=DEV)
            prefill_attention_tcgen05(qd, k_pool, v_pool, positions, q_start_d, table, max(q_lens), nh, g, hs, error_flag=flag,
                                      out=out, kv_splits=splits, tiles_per_split=limit, skip_single=skip)
            assert int(flag) == 0, (seed, trial, launch)
            if bool(keep.any()):
                torch.testing.assert_close(out[keep].float(), ref[keep].float(), rtol=2e-2, atol=2e-2)
            assert torch.all(out[~keep] == 3.0)


def test_prefill_attention_tcgen05_far_key_and_causal_edge():
    """One key takes nearly all the weight: each query row must return that key's value if it
    can see the key, and must not if the key lies after it (causal edge inside a tile)."""
    from yalis_b200.ops.attention import prefill_attention_tcgen05
    nh, g, hs, page, l = 4, 1, 128, 16, 700
    ks, vs, k_pool, v_pool, table = paged_setup(1, [l], g, hs, page, torch.bfloat16, seed=21)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for target, kv_splits in ((0, 1), (127, 1), (128, 1), (300, 1), (555, 1), (0, 3), (128, 4), (555, 3), (300, 2)):
        q_len = 200                                          # queries at positions 500..699
        q = (ks[0][target, 0] * 4.0).repeat(q_len * nh).view(q_len, nh * hs).to(torch.bfloat16).to(DEV)
        out = prefill_attention_tcgen05(q, k_pool, v_pool, i32(list(range(l - q_len, l))), i32([0, q_len]), table, q_len,
                                        nh, g, hs, kv_splits=kv_splits, tiles_per_split=2)
        got = out.float().cpu().view(q_len, nh, hs)
        want = vs[0][target, 0].to(torch.bfloat16).float()
        for t in (0, 54, 55, 56, 199):
            sees = target <= l - q_len + t
            close = torch.allclose(got[t, 0], want, atol=8e-2)
            assert close == sees, (target, t, sees)
