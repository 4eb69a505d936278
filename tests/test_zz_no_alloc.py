"""The allocation-free entry point of the split-key decode attention, called through its
exported C symbol as a host program without an allocator would call it, against plain attention
in float32 over the gathered keys and against the regular entry point.

The caller of ``yalis_paged_attention_mma_noalloc`` owns inputs and output; the kernel's
temporary memory comes from a fixed array inside the library (csrc/attention_noalloc.h), so
nothing is allocated by the call.  Two calls in a row must give the regular result (the
array keeps the first call's contents), and a problem larger than the array is refused.
This file sorts last so that a run that stops at the first failure has run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ERR_SCRATCH = -5


def _case(batch, lens, nh, g, hs, page, seed):
    gen = torch.Generator().manual_seed(seed)
    pages_per = [-(-l // page) for l in lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=gen).tolist()
    table = torch.full((batch, max(pages_per)), -1, dtype=torch.int32)
    it = iter(perm)
    for r, n in enumerate(pages_per):
        for i in range(n):
            table[r, i] = next(it)
    k_pool = torch.randn(num_pages, g, page, hs, generator=gen).to(torch.bfloat16).to(DEV)
    v_pool = torch.randn(num_pages, g, page, hs, generator=gen).to(torch.bfloat16).to(DEV)
    q = torch.randn(batch, nh * hs, generator=gen).to(torch.bfloat16).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, i32([l - 1 for l in lens]), i32(list(range(batch + 1))), i32(list(range(batch))), table.to(DEV)


def _plain(q, k_pool, v_pool, lens, table, nh, g, hs):
    """Every request's single query over its own keys, gathered page by page, in float32."""
    page, rows = k_pool.shape[2], []
    for r, n in enumerate(lens):
        pages = table[r, :-(-n // page)].long()
        keys = k_pool[pages].permute(1, 0, 2, 3).reshape(g, -1, hs)[:, :n].float()
        values = v_pool[pages].permute(1, 0, 2, 3).reshape(g, -1, hs)[:, :n].float()
        query = q[r].view(g, nh // g, hs).float()
        weights = torch.softmax(torch.einsum("gpd,gkd->gpk", query, keys) / math.sqrt(hs), dim=-1)
        rows.append(torch.einsum("gpk,gkd->gpd", weights, values).reshape(nh * hs))
    return torch.stack(rows)


def _call_noalloc(lib, q, k_pool, v_pool, positions, q_start, req, table, nh, g, hs, splits, out):
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    ci = ctypes.c_int
    return lib.yalis_paged_attention_mma_noalloc(
        vp(q), ci(q.stride(0)), vp(out), ci(out.stride(0)), vp(k_pool), vp(v_pool), vp(positions), vp(q_start), vp(req),
        vp(table), ci(table.shape[1]), ci(k_pool.shape[2]), ci(k_pool.shape[0]), ci(q.shape[0]), ci(q_start.numel() - 1),
        ci(1), ci(nh), ci(g), ci(hs), ctypes.c_float(1.0 / math.sqrt(hs)), ci(0), ci(splits),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_entry_matches_regular_entry_twice():
    from yalis_b200 import native
    from yalis_b200.ops.attention import paged_attention_mma
    lib = native.load("cuda")
    nh, g, hs, page, splits = 8, 2, 64, 16, 4
    first_lens, second_lens = [1, 70, 129, 300, 1000], [513, 64, 2]
    first = _case(5, first_lens, nh, g, hs, page, seed=1)
    second = _case(3, second_lens, nh, g, hs, page, seed=2)             # another shape: the array holds stale data
    for lens, (q, k_pool, v_pool, positions, q_start, req, table) in ((first_lens, first), (second_lens, second)):
        want = paged_attention_mma(q, k_pool, v_pool, positions, q_start, req, table, 1, nh, g, hs, n_splits=splits)
        out = torch.zeros_like(want)                                      # the caller's own output buffer
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        status = _call_noalloc(lib, q, k_pool, v_pool, positions, q_start, req, table, nh, g, hs, splits, out)
        torch.cuda.synchronize()
        assert status == 0
        assert torch.cuda.memory_allocated() == before                   # nothing went through torch's allocator
        torch.testing.assert_close(out.float(), _plain(q, k_pool, v_pool, lens, table, nh, g, hs), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert not torch.isnan(out.float()).any()


def test_noalloc_entry_refuses_what_does_not_fit():
    from yalis_b200 import native
    lib = native.load("cuda")
    needed = lib.yalis_paged_attention_mma_noalloc_needed
    needed.restype = ctypes.c_longlong
    tb, pb = ctypes.c_longlong(0), ctypes.c_longlong(0)
    total = needed(64, 64, 32, 8, 128, 4, ctypes.byref(tb), ctypes.byref(pb))
    assert tb.value == 64 * 8 * 4 and pb.value == 64 * 32 * 4 * 130 * 4 and total == tb.value + pb.value
    nh, g, hs, page = 32, 8, 128, 16
    q, k_pool, v_pool, positions, q_start, req, table = _case(40, [20] * 40, nh, g, hs, page, seed=3)
    out = torch.full((40, nh * hs), 3.0, dtype=torch.bfloat16, device=DEV)
    # 40 tokens x 32 heads x 32 splits x 130 floats = 21 MB of partial results: over the 16 MiB limit
    status = _call_noalloc(lib, q, k_pool, v_pool, positions, q_start, req, table, nh, g, hs, 32, out)
    torch.cuda.synchronize()
    assert status == ERR_SCRATCH
    assert torch.all(out == 3.0)                                          # nothing was launched
    # and the same problem with fewer splits fits and runs
    assert _call_noalloc(lib, q, k_pool, v_pool, positions, q_start, req, table, nh, g, hs, 8, out) == 0
    torch.cuda.synchronize()
    assert not torch.all(out == 3.0)
