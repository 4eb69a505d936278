"""Wrappers of the paged attention kernels."""

from __future__ import annotations

import math
from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, lib, need, need_cuda, ptr, stream


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


def paged_attention(qkv: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, group: str, num_heads: int,
                    num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                    window: Optional[int] = None) -> torch.Tensor:
    """Attention of the step's tokens over the cache of their requests: picks the
    kernel for the step's shape and dtype.  ``ctx`` is the step context."""
    table = ctx.block_tables[group]
    return paged_attention_generic(qkv, k_pool, v_pool, ctx.positions, ctx.req_of_token, table, num_heads,
                                   num_kv_heads, head_dim, scale=scale, window=window)
