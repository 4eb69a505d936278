"""A hand-made step context and page pools for tests that run one part without an engine."""

import torch

from yalis_b200.engine.context import HostStep, StepContext
from yalis_b200.parts.base import PagedKVCache

DEV = "cuda:0"


def make_context(q_lens, ctx_before, page_size, group="kv_all", seed=0):
    """Requests i feeds q_lens[i] tokens after ctx_before[i] cached ones; pages are handed out shuffled."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    n, r = sum(q_lens), len(q_lens)
    pos, req, qs = [], [], [0]
    for i, (q, b) in enumerate(zip(q_lens, ctx_before)):
        pos += list(range(b, b + q))
        req += [i] * q
        qs.append(qs[-1] + q)
    kv = [b + q for q, b in zip(q_lens, ctx_before)]
    pages_per = [-(-l // page_size) for l in kv]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(pages_per)
    table = torch.full((r, width), -1, dtype=torch.int32)
    it = iter(perm)
    for i, pp in enumerate(pages_per):
        for j in range(pp):
            table[i, j] = next(it)
    ctx = StepContext(
        n_tokens=n, n_requests=r, token_ids=i32([0] * n), positions=i32(pos), req_of_token=i32(req), q_start=i32(qs),
        kv_len=i32(kv), slots=i32(list(range(r))), logit_rows=i32([]), block_tables={group: table.to(DEV)},
        host=HostStep(slots=list(range(r)), q_start=qs, ctx_before=list(ctx_before), max_q_len=max(q_lens), max_kv_len=max(kv)),
        error_flag=torch.zeros(1, dtype=torch.int32, device=DEV), decode_only=all(q == 1 for q in q_lens))
    return ctx, num_pages


def make_cache(num_pages, kv_heads, page_size, head_dim, dtype, group="kv_all"):
    k = torch.zeros(num_pages, kv_heads, page_size, head_dim, dtype=dtype, device=DEV)
    return PagedKVCache(k, torch.zeros_like(k), group)
