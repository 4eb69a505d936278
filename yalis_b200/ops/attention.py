"""Wrappers of the paged attention kernels."""

from __future__ import annotations

import collections
import ctypes
import math
import os
from typing import Optional

import numpy as np
import torch

from yalis_b200 import native

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream


def _check_common(name, q, k_pool, v_pool, positions, req_of_token, block_table, num_heads, num_kv_heads, head_dim):
    need_cuda(name, q, k_pool, v_pool, positions, req_of_token, block_table)
    n = q.shape[0]
    need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= num_heads * head_dim, name,
         "q must be [N, >= heads*head_dim] with unit inner stride")
    need(k_pool.shape == v_pool.shape and k_pool.dim() == 4 and k_pool.shape[1] == num_kv_heads
         and k_pool.shape[3] == head_dim and k_pool.is_contiguous() and v_pool.is_contiguous(), name,
         "pools must be contiguous [pages, kv_heads, page_size, head_dim]")
    need(k_pool.dtype == q.dtype == v_pool.dtype, name, "q and the pools must have one dtype")
    need(num_heads % num_kv_heads == 0, name, "heads must be a multiple of kv_heads")
    for t in (positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions/req_of_token: int32 [N]")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
         "block_table must be contiguous int32 [R, width]")


def paged_attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                            req_of_token: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                            num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                            window: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact attention of every token over the cached keys of its request.

    ``q`` may be the fused qkv matrix (only its first heads*head_dim columns are
    read).  Token t of request r at position p sees keys j of r with
    p - window < j <= p.  Returns [N, heads*head_dim] in q's dtype.
    """
    name = "paged_attention_generic"
    LAUNCHED["generic"] += 1
    _check_common(name, q, k_pool, v_pool, positions, req_of_token, block_table, num_heads, num_kv_heads, head_dim)
    need(head_dim % 2 == 0 and head_dim <= 256, name, f"head_dim {head_dim} must be even and at most 256")
    n = q.shape[0]
    if out is None:
        out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    need(out.shape == (n, num_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous(), name, "bad out tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    check(lib().yalis_paged_attention_generic(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), i32(dtype_code(q.dtype)),
        ptr(positions), ptr(req_of_token), ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]),
        i32(k_pool.shape[0]), i32(n), i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale),
        i32(window or 0), stream()), name)
    return out


SM_COUNT: Optional[int] = None    # set to override what the device reports (tests pretend a small GPU)
_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked of the driver once per device)."""
    if SM_COUNT is not None:
        return SM_COUNT
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


# How often each attention kernel was launched through these wrappers (tests read it to see which path a step took).
LAUNCHED = collections.Counter()
# YALIS_B200_NO_DECODE_TMA=1 keeps decode steps on the cp.async kernel (for comparisons).
# YALIS_B200_NO_FUSED_ROPE=1 keeps the rotary / cache-write kernel apart from the decode attention.
USE_FUSED_ROPE = os.environ.get("YALIS_B200_NO_FUSED_ROPE", "0") != "1"
USE_DECODE_TMA = os.environ.get("YALIS_B200_NO_DECODE_TMA", "0") != "1"
# YALIS_B200_NO_DECODE_LEAN=1 keeps large decode batches on one block per (request, KV head).
USE_DECODE_LEAN = os.environ.get("YALIS_B200_NO_DECODE_LEAN", "0") != "1"
# YALIS_B200_NO_PREFILL_TCGEN05=1 keeps prompt portions on the mma.sync kernel.
USE_PREFILL_TCGEN05 = os.environ.get("YALIS_B200_NO_PREFILL_TCGEN05", "0") != "1"


def mma_supports(head_dim: int) -> bool:
    """Whether the tensor-core kernel is built for this head size (multiples of 16 up to 128, of 32 up to 256)."""
    return bool(lib().yalis_attention_mma_supports(i32(head_dim)))


def decode_splits(n_requests: int, num_kv_heads: int) -> int:
    """How many blocks share the keys of one (request, KV head) in a decode step, so that
    few requests still fill the GPU: as many as fit in ONE wave of two blocks per SM (a second,
    nearly empty wave would double the kernel's time).  Depends on the batch shape only, never
    on lengths, so a captured step can be replayed."""
    blocks = max(1, n_requests * num_kv_heads)
    return max(1, min(32, (2 * sm_count()) // blocks))


LONG_CONTEXT = 8192     # beyond this many cached tokens a few requests cannot keep HBM busy with 8 splits each


def decode_tma_splits(n_requests: int, num_kv_heads: int, long_context: bool) -> int:
    """Splits of a (request, KV head) for the TMA-fed decode kernel: up to 8 merge inside a thread-block
    cluster (the cheaper merge); steps of the long-context kind take up to 32 and merge through global memory,
    so that a single long request still spreads over the whole GPU.  Clusters of more than four blocks are
    kept to 70 % of the places for blocks: a cluster starts only when all its blocks find room in one part of
    the GPU, and inside a step the kernel before still holds some (4 requests x 8 KV heads in 8 splits are 256
    blocks in 32 clusters: 5 % of a decode step slower than in 6 splits)."""
    n = decode_splits(n_requests, num_kv_heads)
    if long_context:
        return n
    n = min(8, n)
    if n > 4:
        pairs = max(1, n_requests * num_kv_heads)
        n = min(n, max(4, int(0.7 * 2 * sm_count()) // pairs))
    return n


_ticket_cache = {}


def _tickets(device, n: int) -> torch.Tensor:
    """Zeroed int32 counters, one per (request, KV head): every split launch leaves them zero,
    so one buffer per device is allocated once (outside any graph capture) and shared."""
    key = torch.device(device)
    t = _ticket_cache.get(key)
    if t is None or t.numel() < n:
        t = _ticket_cache[key] = torch.zeros(max(n, 4096), dtype=torch.int32, device=key)
    return t


_work_counter_cache = {}


def _work_counters(device) -> torch.Tensor:
    """Two zeroed int32 in which the prompt kernel counts its work items.  Every launch leaves them zero, so one
    pair per device is allocated once (outside any graph capture) and shared by launches that run one after the
    other; launches of this kernel on two streams at the same time would need a pair each."""
    key = torch.device(device)
    t = _work_counter_cache.get(key)
    if t is None:
        t = _work_counter_cache[key] = torch.zeros(2, dtype=torch.int32, device=key)
    return t


def paged_attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                        q_start: torch.Tensor, req_of_token: torch.Tensor, block_table: torch.Tensor, max_q_len: int,
                        num_heads: int, num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                        window: Optional[int] = None, n_splits: int = 1,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention (bfloat16) of the step's tokens over the cache; the same
    semantics as ``paged_attention_generic``.  ``q_start`` int32 [R+1] gives each request's
    token range; ``max_q_len`` bounds the launch grid.  ``n_splits`` > 1 divides the keys of
    a request among blocks (decode steps) and needs scratch memory for the partial results.
    """
    name = "paged_attention_mma"
    LAUNCHED["mma"] += 1
    _check_common(name, q, k_pool, v_pool, positions, req_of_token, block_table, num_heads, num_kv_heads, head_dim)
    need(q.dtype == torch.bfloat16, name, "bfloat16 only (float32 goes to the generic kernel)")
    need(mma_supports(head_dim), name, f"head_dim {head_dim} is not built (multiples of 16 to 128, of 32 to 256)")
    n, r = q.shape[0], q_start.numel() - 1
    need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.is_cuda, name, "q_start must be int32 [R+1]")
    need(block_table.shape[0] >= r, name, "block_table has fewer rows than requests")
    if out is None:
        out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    need(out.shape == (n, num_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous(), name, "bad out tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    scratch = tickets = None
    if n_splits > 1:
        need(max_q_len * (num_heads // num_kv_heads) <= 16, name, "splitting the keys is for decode steps only")
        floats = lib().yalis_attention_mma_scratch_floats
        floats.restype = ctypes.c_longlong
        scratch = torch.empty(int(floats(i32(n), i32(num_heads), i32(head_dim), i32(n_splits))), dtype=torch.float32,
                              device=q.device)
        tickets = _tickets(q.device, r * num_kv_heads)
    check(lib().yalis_paged_attention_mma(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(q_start),
        ptr(req_of_token), ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]), i32(k_pool.shape[0]),
        i32(n), i32(r), i32(max_q_len), i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale), i32(window or 0),
        i32(n_splits), ptr(scratch), ptr(tickets), stream()), name)
    return out


def decode_tma_supports(head_dim: int, page_size: int, heads_per_group: int) -> bool:
    """Whether the TMA-fed decode kernel takes this shape (head_dim 64/128/192/256, pages of 8..64, <= 16 heads per group)."""
    return bool(lib().yalis_decode_attention_tma_supports(i32(head_dim), i32(page_size), i32(heads_per_group)))


def decode_attention_tma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                         q_start: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                         head_dim: int, scale: Optional[float] = None, n_splits: int = 1,
                         error_flag: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                         early_fetch: bool = False) -> torch.Tensor:
    """Decode attention (one token per request, no window) with TMA-fed K/V tiles; same result as
    ``paged_attention_mma`` for such a step.  ``q`` is [R, heads*head_dim] (one row per request).

    ``early_fetch`` lets the kernel read keys below each query's position, ``positions``, ``q_start`` and the
    block table while the kernel before it on the stream is still running; pass it only when all of those
    were complete before that kernel began (inside a model step they are)."""
    name = "decode_attention_tma"
    LAUNCHED["decode_tma"] += 1
    n, r = q.shape[0], q_start.numel() - 1
    req_dummy = positions      # only shapes and dtypes are checked through the common helper
    _check_common(name, q, k_pool, v_pool, positions, req_dummy, block_table, num_heads, num_kv_heads, head_dim)
    need(q.dtype == torch.bfloat16, name, "bfloat16 only")
    need(decode_tma_supports(head_dim, k_pool.shape[2], num_heads // num_kv_heads), name,
         "needs head_dim 64/128/192/256, page_size 8/16/32/64 and at most 16 heads per KV head")
    need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.is_cuda, name, "q_start must be int32 [R+1]")
    need(block_table.shape[0] >= r, name, "block_table has fewer rows than requests")
    if out is None:
        out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    need(out.shape == (n, num_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous(), name, "bad out tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    scratch = tickets = None
    if n_splits > 8:            # up to 8 splits merge inside a thread-block cluster and need no scratch memory
        floats = lib().yalis_attention_mma_scratch_floats
        floats.restype = ctypes.c_longlong
        scratch = torch.empty(int(floats(i32(n), i32(num_heads), i32(head_dim), i32(n_splits))), dtype=torch.float32,
                              device=q.device)
        tickets = _tickets(q.device, r * num_kv_heads)
    check(lib().yalis_decode_attention_tma(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(q_start),
        ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]), i32(k_pool.shape[0]), i32(n), i32(r),
        i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale), i32(n_splits), i32(1 if early_fetch else 0),
        ptr(scratch), ptr(tickets), ptr(error_flag), stream()), name)
    return out


def decode_lean_blocks(head_dim: int) -> int:
    """Blocks of the evenly dealt decode kernel that are resident at once (its grid)."""
    return (2 if head_dim <= 128 else 1) * sm_count()


DEAL_MIN_LONGEST = 2048   # below this many cached tokens even a lone long request costs less than dealing tiles out


def deal_tiles_hint(lengths) -> bool:
    """Host-side choice for a decode step of requests holding ``lengths`` cached tokens: True when a block per
    (request, KV head) - or a fixed number of them - would leave the GPU waiting for the longest request, i.e.
    with two or more requests of which one is beyond the long-context mark, or is at least ``DEAL_MIN_LONGEST``
    long and twice the mean.  Depends on lengths only."""
    n = len(lengths)
    if n < 2:
        return False
    longest = max(lengths)
    return longest > LONG_CONTEXT or (longest >= DEAL_MIN_LONGEST and longest * n >= 2 * sum(lengths))


def decode_step_kind(lengths) -> tuple:
    """(deal_tiles, long_context) of a decode step whose requests hold ``lengths`` tokens after it: everything
    the decode kernels' launch depends on besides the shapes.  A recorded step is keyed by it, because a replay
    cannot look at lengths: dealt tiles for long or uneven batches, more key splits for one long request."""
    if not lengths:
        return (False, False)
    deal = deal_tiles_hint(lengths)
    return (deal, not deal and max(lengths) > LONG_CONTEXT)


def step_kind(ctx) -> tuple:
    """``decode_step_kind`` of the step, computed once (every layer asks)."""
    kind = ctx.extras.get("paged_attention.kind")
    if kind is None:
        host = ctx.host
        lengths = [b + (q1 - q0) for b, q0, q1 in zip(host.ctx_before, host.q_start[:-1], host.q_start[1:])]
        kind = ctx.extras["paged_attention.kind"] = decode_step_kind(lengths) if ctx.decode_only else (False, False)
    return kind


def decode_lean_preferred(n_requests: int, num_kv_heads: int, head_dim: int, deal_tiles: bool = False) -> bool:
    """Whether a decode step goes to the kernel that deals the key tiles of all (request, KV head) pairs to a fixed
    grid: with more pairs than blocks fit the GPU at once (a block per pair would run in waves, the last one
    mostly empty), or when the requests are long or uneven (``deal_tiles``)."""
    if not USE_DECODE_LEAN or n_requests > 4096:
        return False
    if deal_tiles and n_requests >= 2:
        return True
    return n_requests * num_kv_heads > decode_lean_blocks(head_dim)


def decode_attention_lean(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                          q_start: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                          head_dim: int, scale: Optional[float] = None, n_blocks: Optional[int] = None,
                          error_flag: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                          early_fetch: bool = False, only_single: bool = False) -> torch.Tensor:
    """Decode attention (one token per request, no window) by a fixed grid of blocks that share the key/value
    tiles of all (request, KV head) pairs evenly; same result as ``decode_attention_tma`` up to the order in which
    the pieces of a pair cut between blocks are added.  ``q`` is [N, >= heads*head_dim]; a request's token is the
    first of its range in ``q_start``.  ``early_fetch`` as for ``decode_attention_tma``.  With ``only_single``
    requests that bring more than one token are skipped and their rows of ``out`` left as they are (the decoding
    requests of a step that also holds prompt portions)."""
    name = "decode_attention_lean"
    LAUNCHED["decode_lean"] += 1
    n, r = q.shape[0], q_start.numel() - 1
    _check_common(name, q, k_pool, v_pool, positions, positions, block_table, num_heads, num_kv_heads, head_dim)
    need(q.dtype == torch.bfloat16, name, "bfloat16 only")
    need(decode_tma_supports(head_dim, k_pool.shape[2], num_heads // num_kv_heads), name,
         "needs head_dim 64/128/192/256, page_size 8/16/32/64 and at most 16 heads per KV head")
    need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.is_cuda, name, "q_start must be int32 [R+1]")
    need(block_table.shape[0] >= r, name, "block_table has fewer rows than requests")
    need(r <= 4096, name, "at most 4096 requests")
    if out is None:
        out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    need(out.shape == (n, num_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous(), name, "bad out tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    if n_blocks is None:
        n_blocks = decode_lean_blocks(head_dim)
    need(n_blocks >= 1, name, "n_blocks must be positive")
    floats = lib().yalis_decode_attention_lean_scratch_floats
    floats.restype = ctypes.c_longlong
    scratch = torch.empty(int(floats(i32(n_blocks), i32(head_dim))), dtype=torch.float32, device=q.device)
    tickets = _tickets(q.device, r * num_kv_heads)
    check(lib().yalis_decode_attention_lean(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(q_start),
        ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]), i32(k_pool.shape[0]), i32(n), i32(r),
        i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale), i32(n_blocks), i32(1 if early_fetch else 0),
        i32(1 if only_single else 0), ptr(scratch), ptr(tickets), ptr(error_flag), stream()), name)
    return out


def decode_attention_tma_fused(qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], store: bool, k_pool: torch.Tensor,
                               v_pool: torch.Tensor, positions: torch.Tensor, q_start: torch.Tensor,
                               block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                               scale: Optional[float] = None, n_splits: int = 1,
                               error_flag: Optional[torch.Tensor] = None, early_fetch: bool = False) -> torch.Tensor:
    """``decode_attention_tma`` with the rotary kernel's work done inside: ``qkv`` is the step's fused projection
    [N, (heads + 2 kv_heads) * head_dim] in bfloat16, or float32 partial sums [S, N, ...] that are added in order;
    queries and the new key are rotated by ``float(position) * inv_freq`` (None: not at all), and with ``store``
    the new key and value are written to the pools.  Same bits as ``rope_kv_write`` followed by
    ``decode_attention_tma``."""
    name = "decode_attention_tma_fused"
    LAUNCHED["decode_tma_fused"] += 1
    width = (num_heads + 2 * num_kv_heads) * head_dim
    need_cuda(name, qkv, inv_freq, k_pool, v_pool, positions, q_start, block_table, error_flag)
    need(qkv.is_contiguous() and qkv.shape[-1] == width and qkv.dim() in (2, 3), name,
         "qkv must be contiguous [N, (heads + 2*kv_heads) * head_dim] or [S, N, ...]")
    need((qkv.dim() == 2 and qkv.dtype == torch.bfloat16) or (qkv.dim() == 3 and qkv.dtype == torch.float32), name,
         "qkv must be bfloat16 rows or float32 partial sums")
    parts = qkv.shape[0] if qkv.dim() == 3 else 1
    n, r = qkv.shape[-2], q_start.numel() - 1
    need(k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16 and k_pool.shape == v_pool.shape
         and k_pool.dim() == 4 and k_pool.shape[1] == num_kv_heads and k_pool.shape[3] == head_dim
         and k_pool.is_contiguous() and v_pool.is_contiguous(), name, "pools must be contiguous bfloat16 [pages, kv_heads, page_size, head_dim]")
    need(decode_tma_supports(head_dim, k_pool.shape[2], num_heads // num_kv_heads), name,
         "needs head_dim 64/128/192/256, page_size 8/16/32/64 and at most 16 heads per KV head")
    for t in (positions,):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions: int32 [N]")
    need(q_start.dtype == torch.int32 and q_start.is_contiguous(), name, "q_start must be int32 [R+1]")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
         and block_table.shape[0] >= r, name, "block_table must be contiguous int32 [>= R, width]")
    if inv_freq is not None:
        need(inv_freq.dtype == torch.float32 and inv_freq.shape == (head_dim // 2,) and inv_freq.is_contiguous(), name,
             "inv_freq must be float32 [head_dim / 2]")
    out = torch.empty((n, num_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    scratch = tickets = None
    if n_splits > 8:
        floats = lib().yalis_attention_mma_scratch_floats
        floats.restype = ctypes.c_longlong
        scratch = torch.empty(int(floats(i32(n), i32(num_heads), i32(head_dim), i32(n_splits))), dtype=torch.float32,
                              device=qkv.device)
        tickets = _tickets(qkv.device, r * num_kv_heads)
    check(lib().yalis_decode_attention_tma_fused(
        ptr(qkv), i32(1 if qkv.dtype == torch.float32 else 0), i32(parts), i64(n * width), i32(width), ptr(inv_freq),
        i32(1 if store else 0), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(q_start),
        ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]), i32(k_pool.shape[0]), i32(n), i32(r),
        i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale), i32(n_splits), i32(1 if early_fetch else 0),
        ptr(scratch), ptr(tickets), ptr(error_flag), stream()), name)
    return out


def decode_tma_applicable(dtype: torch.dtype, ctx, head_dim: int, page_size: int, heads_per_group: int,
                          window: Optional[int]) -> bool:
    """Whether a step goes to the TMA-fed decode kernel: bfloat16, one token per request, no window, a shape it takes."""
    return (dtype == torch.bfloat16 and USE_DECODE_TMA and ctx.decode_only and ctx.host.max_q_len == 1 and window is None
            and decode_tma_supports(head_dim, page_size, heads_per_group))


def prefill_tcgen05_supports(head_dim: int, page_size: int, heads_per_group: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this shape (head_dim 64/128, pages of 8..128)."""
    return bool(lib().yalis_prefill_attention_tcgen05_supports(i32(head_dim), i32(page_size), i32(heads_per_group)))


def prefill_attention_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                              q_start: torch.Tensor, block_table: torch.Tensor, max_q_len: int, num_heads: int,
                              num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                              error_flag: Optional[torch.Tensor] = None,
                              out: Optional[torch.Tensor] = None, kv_splits: int = 1,
                              tiles_per_split: int = 1, skip_single: bool = False) -> torch.Tensor:
    """Causal paged attention of prompt portions on tcgen05 tensor cores (no window); the same
    semantics as ``paged_attention_generic``.  ``q`` is [N, >= heads*head_dim].  With ``kv_splits`` > 1 a tile of
    queries that sees more than ``tiles_per_split`` tiles of 64 keys has them divided among up to ``kv_splits``
    blocks, whose shares a second kernel adds (see ``prefill_kv_splits``); every row of ``q`` must then belong
    to a request.  ``skip_single`` leaves the rows of requests that bring one token as they are."""
    name = "prefill_attention_tcgen05"
    LAUNCHED["prefill_tcgen05"] += 1
    n, r = q.shape[0], q_start.numel() - 1
    _check_common(name, q, k_pool, v_pool, positions, positions, block_table, num_heads, num_kv_heads, head_dim)
    need(q.dtype == torch.bfloat16, name, "bfloat16 only")
    need(prefill_tcgen05_supports(head_dim, k_pool.shape[2], num_heads // num_kv_heads), name,
         "needs head_dim 64 or 128, page_size 8..128 (power of two) and at most 128 heads per KV head")
    need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.is_cuda, name, "q_start must be int32 [R+1]")
    need(block_table.shape[0] >= r, name, "block_table has fewer rows than requests")
    if out is None:
        out = torch.empty((n, num_heads * head_dim), dtype=q.dtype, device=q.device)
    need(out.shape == (n, num_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous(), name, "bad out tensor")
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    need(1 <= kv_splits <= 64 and tiles_per_split >= 1, name, "kv_splits must be 1..64, tiles_per_split positive")
    scratch = None
    if kv_splits > 1:
        floats = lib().yalis_prefill_attention_tcgen05_scratch_floats
        floats.restype = ctypes.c_longlong
        scratch = torch.empty(int(floats(i32(n), i32(num_heads), i32(head_dim), i32(kv_splits))), dtype=torch.float32,
                              device=q.device)
    check(lib().yalis_prefill_attention_tcgen05(
        ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(q_start),
        ptr(block_table), i32(block_table.shape[1]), i32(k_pool.shape[2]), i32(k_pool.shape[0]), i32(n), i32(r),
        i32(max_q_len), i32(num_heads), i32(num_kv_heads), i32(head_dim), f32(scale), i32(kv_splits), i32(tiles_per_split),
        i32(1 if skip_single else 0), ptr(scratch), ptr(_work_counters(q.device)), ptr(error_flag), stream()), name)
    return out


PREFILL_SPLIT_MIN_TILES = 16     # a share of a divided tile of queries is at least this many key tiles long
PREFILL_SPLIT_START_UP = 20.0    # what one more block costs (fill and drain, its share's outputs), in key tiles
PREFILL_SPLIT_UNSHARED = 1.4     # pace of a block whose keys no other block reads at the time (they come from HBM)


PREFILL_SPLIT_GAIN = 0.92        # dividing has to bring 8 %


def _policy_lib():
    host_lib = native.load("host")
    if not getattr(host_lib, "_ypol_typed", False):
        host_lib.ypol_step_length.restype = ctypes.c_double
        host_lib.ypol_step_length.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 4 + [ctypes.c_double]
        host_lib.ypol_kv_splits.restype = None
        host_lib.ypol_kv_splits.argtypes = ([ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5
                                            + [ctypes.c_double] * 3 + [ctypes.c_void_p])
        host_lib._ypol_typed = True
    return host_lib


def _prefill_step_length(items, slots: int, splits: int, limit: int) -> float:
    """Length of the tcgen05 prompt kernel, in key tiles of a block, for ``items`` = (key tiles, pace) of the
    tiles of queries of one KV head: the blocks in launch order (share after share) each go to the first of
    ``slots`` places to come free.  (The model itself is native, csrc/host/attention_policy.cpp: it runs for
    every step that is launched.)"""
    tiles = np.asarray([t for t, _ in items], dtype=np.int32)
    pace = np.asarray([p for _, p in items], dtype=np.float64)
    return float(_policy_lib().ypol_step_length(tiles.ctypes.data, pace.ctypes.data, len(items), slots, splits, limit,
                                                PREFILL_SPLIT_START_UP))


def prefill_kv_splits(host, heads_per_group: int, num_kv_heads: int, head_dim: int, skip_single: bool = False):
    """(kv_splits, tiles_per_split) for the tcgen05 prompt kernel in a step with the host facts ``host``.

    The kernel runs one block per (tile of 128 // heads_per_group queries, KV head), two to an SM, and a block's
    time grows with the keys its queries see.  Two things leave the GPU idle.  A few blocks with far more keys
    than the rest: one decoding request with 14,000 cached tokens beside a fresh prompt keeps its 8 blocks busy
    for 0.47 ms, everything else is done after 0.1 ms (with its keys in four shares the step takes 0.17 ms).  And
    a number of long blocks just above a multiple of the 296 that run at once, or well below it: a 2,048-token
    portion behind 12,000 tokens with 24 heads in 8 groups is 392 blocks, two rounds of which the second is a
    third full (0.59 ms; in halves 0.51 ms); a 512-token portion is 128 blocks (89 us; in halves 73 us).
    The choice is the best of 1, 2, 3, 4, 6 or 8 shares for the longest tile of queries (shorter ones get fewer)
    under a model of the launch (``_prefill_step_length``) whose three constants are fitted to 26 measured steps
    (portions of 512 to 2,048 tokens behind up to 14,000 cached ones, alone and beside decoding requests, 24 and
    32 heads in 8 groups: the choices cost 1.4 % over the best measured ones, the model's times are 10 % off).
    A tile of queries counts as reading its keys alone (a slower pace) when its request brings at most three
    tiles; requests of one token are left out with ``skip_single`` (they go to another kernel)."""
    if not host.ctx_before or host.q_start[-1] == host.q_start[0]:
        return 1, 1
    q_start = np.asarray(host.q_start, dtype=np.int32)
    q_lens = np.ascontiguousarray(q_start[1:] - q_start[:-1])
    before = np.asarray(host.ctx_before, dtype=np.int32)
    out = np.ones(2, dtype=np.int32)
    _policy_lib().ypol_kv_splits(q_lens.ctypes.data, before.ctypes.data, len(q_lens), 128 // heads_per_group,
                                 max(1, 2 * sm_count() // num_kv_heads), 1 if skip_single else 0, PREFILL_SPLIT_MIN_TILES,
                                 PREFILL_SPLIT_START_UP, PREFILL_SPLIT_UNSHARED, PREFILL_SPLIT_GAIN, out.ctypes.data)
    return int(out[0]), int(out[1])


MIXED_DECODE_MIN_KEYS = 4096     # cached tokens of a step's decoding requests from which they get a kernel of their own


def mixed_step_splits_off_decodes(host) -> bool:
    """Whether, in a step that holds prompt portions and decoding requests, the decoding requests go to the decode
    kernel (which streams their keys at HBM speed) and only the portions to the prompt kernel (where a request's
    single token would occupy a 128-row tile of its own per KV head and be fed two key tiles at a time): when
    the decoding requests hold enough cached tokens for that to outweigh one more launch."""
    q_lens = [b - a for a, b in zip(host.q_start[:-1], host.q_start[1:])]
    if not host.ctx_before:
        return False
    return sum(before for q, before in zip(q_lens, host.ctx_before) if q == 1) >= MIXED_DECODE_MIN_KEYS


def _splits_once(host, heads_per_group: int, num_kv_heads: int, head_dim: int, skip_single: bool) -> tuple:
    """``prefill_kv_splits`` once per step and shape (every layer asks, and so does the key of a recorded step)."""
    work = lambda: tuple(prefill_kv_splits(host, heads_per_group, num_kv_heads, head_dim, skip_single))
    once = getattr(host, "once", None)
    return once(("prefill_kv_splits", heads_per_group, num_kv_heads, head_dim, skip_single), work) if once else work()


def portion_step_kind(host, heads_per_group: int, num_kv_heads: int, head_dim: int) -> tuple:
    """What the attention of a step that holds prompt portions depends on besides the shapes of its tensors:
    whether its decoding requests go to the decode kernel, and how the keys of long tiles of queries are divided
    (a recorded step is keyed by it)."""
    return ((mixed_step_splits_off_decodes(host),) + _splits_once(host, heads_per_group, num_kv_heads, head_dim, True)
            + _splits_once(host, heads_per_group, num_kv_heads, head_dim, False))


def _prefill_split_choice(ctx, per: int, num_kv_heads: int, head_dim: int, skip_single: bool = False) -> dict:
    choice = _splits_once(ctx.host, per, num_kv_heads, head_dim, skip_single)
    return dict(kv_splits=choice[0], tiles_per_split=choice[1])


def paged_attention(qkv: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: str, num_heads: int,
                    num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                    window: Optional[int] = None) -> torch.Tensor:
    """Attention of the step's tokens over the cache of their requests: picks the kernel
    for the step's shape and dtype.  ``ctx`` is the step context.  bfloat16 with a head
    size the tensor-core kernel is built for goes there; everything else (float32, odd
    head sizes) to the exact generic kernel."""
    table = ctx.block_tables[group]
    per = num_heads // num_kv_heads
    if decode_tma_applicable(qkv.dtype, ctx, head_dim, k_pool.shape[2], per, window):
        deal_tiles, long_context = step_kind(ctx)
        if decode_lean_preferred(ctx.n_requests, num_kv_heads, head_dim, deal_tiles):
            return decode_attention_lean(qkv, k_pool, v_pool, ctx.positions, ctx.q_start, table, num_heads, num_kv_heads,
                                         head_dim, scale=scale, error_flag=ctx.error_flag,
                                         early_fetch=bool(getattr(ctx, "settled", False)))
        return decode_attention_tma(qkv, k_pool, v_pool, ctx.positions, ctx.q_start, table, num_heads, num_kv_heads,
                                    head_dim, scale=scale,
                                    n_splits=decode_tma_splits(ctx.n_requests, num_kv_heads, long_context),
                                    error_flag=ctx.error_flag, early_fetch=bool(getattr(ctx, "settled", False)))
    if (qkv.dtype == torch.bfloat16 and USE_PREFILL_TCGEN05 and window is None and ctx.host.max_q_len >= 16
            and prefill_tcgen05_supports(head_dim, k_pool.shape[2], per)):
        out = None
        split_off = ctx.extras.get("mixed_step_splits_off_decodes")
        if split_off is None:
            split_off = ctx.extras["mixed_step_splits_off_decodes"] = mixed_step_splits_off_decodes(ctx.host)
        split_off = split_off and USE_DECODE_LEAN and ctx.n_requests <= 4096 and decode_tma_supports(head_dim, k_pool.shape[2], per)
        if split_off:
            out = decode_attention_lean(qkv, k_pool, v_pool, ctx.positions, ctx.q_start, table, num_heads, num_kv_heads,
                                        head_dim, scale=scale, error_flag=ctx.error_flag,
                                        early_fetch=bool(getattr(ctx, "settled", False)), only_single=True)
        return prefill_attention_tcgen05(qkv, k_pool, v_pool, ctx.positions, ctx.q_start, table, ctx.host.max_q_len,
                                         num_heads, num_kv_heads, head_dim, scale=scale, error_flag=ctx.error_flag,
                                         out=out, skip_single=split_off,
                                         **_prefill_split_choice(ctx, per, num_kv_heads, head_dim, split_off))
    if qkv.dtype == torch.bfloat16 and mma_supports(head_dim):
        splits = decode_splits(ctx.n_requests, num_kv_heads) if ctx.host.max_q_len * per <= 16 else 1
        return paged_attention_mma(qkv, k_pool, v_pool, ctx.positions, ctx.q_start, ctx.req_of_token, table,
                                   ctx.host.max_q_len, num_heads, num_kv_heads, head_dim, scale=scale, window=window,
                                   n_splits=splits)
    return paged_attention_generic(qkv, k_pool, v_pool, ctx.positions, ctx.req_of_token, table, num_heads,
                                   num_kv_heads, head_dim, scale=scale, window=window)
