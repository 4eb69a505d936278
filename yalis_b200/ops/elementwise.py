"""Wrappers of the memory-bound kernels (csrc/elementwise.cu)."""

from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, dtype_code, f32, i32, i64, lib, need, need_cuda, ptr, stream


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None,
              bad_flag: Optional[torch.Tensor] = None, scale: Optional[float] = None,
              from_slot: Optional[torch.Tensor] = None, chosen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = float32(table[ids[t]]) (times ``scale`` if given).  ids int32 [N]; table [vocab, width].
    With ``from_slot`` (int32 [N]) and ``chosen`` (int32 vector), token t takes its id from
    ``chosen[from_slot[t]]`` where ``from_slot[t]`` is not negative."""
    name = "embedding"
    need_cuda(name, table, ids, out, bad_flag, from_slot, chosen)
    need((from_slot is None) == (chosen is None), name, "from_slot and chosen come together")
    if from_slot is not None:
        need(from_slot.dtype == torch.int32 and from_slot.shape == ids.shape and from_slot.is_contiguous()
             and chosen.dtype == torch.int32 and chosen.dim() == 1 and chosen.is_contiguous(), name,
             "from_slot must be int32 [N] and chosen a contiguous int32 vector")
    need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), name, "ids must be contiguous int32 [N]")
    need(table.dim() == 2 and table.is_contiguous(), name, "table must be contiguous [vocab, width]")
    n, (vocab, width) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (n, width), name, "out must be float32 [N, width]")
    check(lib().yalis_embedding(ptr(table), i32(dtype_code(table.dtype)), ptr(ids), ptr(from_slot), ptr(chosen),
                                ptr(out), i32(n), i32(width),
                                i32(vocab), f32(1.0 if scale is None else scale), ptr(bad_flag), stream()), name)
    return out


def softcap_(values: torch.Tensor, cap: float) -> torch.Tensor:
    """values <- cap * tanh(values / cap), in place (float32, contiguous)."""
    name = "softcap"
    need_cuda(name, values)
    need(values.dtype == torch.float32 and values.is_contiguous(), name, "values must be contiguous float32")
    need(cap > 0, name, "the cap must be positive")
    check(lib().yalis_softcap_f32(ptr(values), i64(values.numel()), f32(cap), stream()), name)
    return values


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x + delta) * weight, with x (float32 residual stream) updated in place.

    ``delta`` is None, [N, width], or split partial sums [S, N, width] (added in order).
    With ``rows`` (int32 indices) only those rows are normed and x is left untouched.
    """
    name = "add_rmsnorm"
    need_cuda(name, x, delta, weight, rows, out)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be contiguous float32 [N, width]")
    n, width = x.shape
    need(weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(), name,
         "weight must be float32 [width]")
    n_delta, d_stride, d_code = 0, 0, 0
    if delta is not None:
        need(delta.is_contiguous(), name, "delta must be contiguous")
        if delta.dim() == 2:
            need(delta.shape == (n, width), name, f"delta shape {tuple(delta.shape)} != {(n, width)}")
            n_delta, d_stride = 1, 0
        else:
            need(delta.dim() == 3 and delta.shape[1:] == (n, width), name, "split delta must be [S, N, width]")
            n_delta, d_stride = delta.shape[0], n * width
        d_code = dtype_code(delta.dtype)
    n_out = n
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
        n_out = rows.numel()
    if out is None:
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    need(out.shape == (n_out, width) and out.dtype == out_dtype and out.is_contiguous(), name, "bad out tensor")
    check(lib().yalis_add_rmsnorm(ptr(x), ptr(delta), i32(d_code), i32(n_delta), i64(d_stride), ptr(weight), ptr(out),
                                  i32(dtype_code(out_dtype)), ptr(rows), i32(n_out), i32(width), f32(eps),
                                  i32(0 if rows is not None else 1), stream()), name)
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    """x += delta (or the sum of split partials [S, ...]) in float32, in place."""
    name = "residual_add"
    need_cuda(name, x, delta)
    need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous(), name, "x float32, both contiguous")
    if delta.dim() == x.dim():
        need(delta.shape == x.shape, name, "shape mismatch")
        n_delta, stride = 1, 0
    else:
        need(delta.shape[1:] == x.shape, name, "split delta must be [S, *x.shape]")
        n_delta, stride = delta.shape[0], x.numel()
    check(lib().yalis_residual_add(ptr(x), ptr(delta), i32(dtype_code(delta.dtype)), i32(n_delta), i64(stride),
                                   i64(x.numel()), stream()), name)


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, req_of_token: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                  block_table: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  out_dtype: Optional[torch.dtype] = None, bad_flag: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate Q and K of the fused qkv rows, store K and V into their pages, return Q.

    ``qkv`` is [N, (nh + 2g) * hs] in the model dtype, or float32 partial sums
    [S, N, (nh + 2g) * hs] of a split product (summed in order).  Pools are
    [num_pages, g, page_size, hs]; block_table int32 [R, width].  Returns the rotated
    Q [N, nh * hs] in ``out_dtype`` (default: qkv's dtype).
    """
    name = "rope_kv_write"
    need_cuda(name, qkv, positions, req_of_token, inv_freq, k_pool, v_pool, block_table, bad_flag)
    width = (num_heads + 2 * num_kv_heads) * head_dim
    need(qkv.is_contiguous() and qkv.shape[-1] == width and qkv.dim() in (2, 3), name,
         "qkv must be contiguous [N, (heads + 2*kv_heads) * head_dim] or [S, N, ...]")
    parts = qkv.shape[0] if qkv.dim() == 3 else 1
    n = qkv.shape[-2]
    need(qkv.dim() == 2 or qkv.dtype == torch.float32, name, "split partial sums must be float32")
    out_dtype = out_dtype or qkv.dtype
    need(qkv.dim() == 3 or qkv.dtype == out_dtype, name, "an unsplit qkv must have the output dtype")
    need(head_dim % 2 == 0, name, f"head_dim {head_dim} must be even")
    for t in (positions, req_of_token):
        need(t.dtype == torch.int32 and t.shape == (n,) and t.is_contiguous(), name, "positions/req_of_token: int32 [N]")
    if inv_freq is not None:
        need(inv_freq.dtype == torch.float32 and inv_freq.shape == (head_dim // 2,) and inv_freq.is_contiguous(), name,
             "inv_freq must be float32 [head_dim / 2]")
    need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), name,
         "block_table must be contiguous int32 [R, width]")
    page_size, num_pages = 1, 0
    if k_pool is not None:
        need(v_pool is not None and k_pool.shape == v_pool.shape and k_pool.dtype == out_dtype == v_pool.dtype, name,
             "pools must match each other and the output dtype")
        need(k_pool.dim() == 4 and k_pool.shape[1] == num_kv_heads and k_pool.shape[3] == head_dim
             and k_pool.is_contiguous() and v_pool.is_contiguous(), name,
             "pools must be contiguous [pages, kv_heads, page_size, head_dim]")
        num_pages, page_size = k_pool.shape[0], k_pool.shape[2]
    q_out = torch.empty((n, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
    check(lib().yalis_rope_kv_write(ptr(qkv), i32(dtype_code(qkv.dtype)), i32(width), i32(parts), i64(n * width),
                                    ptr(q_out), i32(dtype_code(out_dtype)), ptr(positions), ptr(req_of_token),
                                    ptr(inv_freq), ptr(k_pool), ptr(v_pool), ptr(block_table),
                                    i32(block_table.shape[1]), i32(page_size), i32(num_pages), i32(num_heads),
                                    i32(num_kv_heads), i32(head_dim), i32(n), ptr(bad_flag), stream()), name)
    return q_out


def silu_mul(x: torch.Tensor, interleaved: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up for rows [gate | up] (or gate0, up0, gate1, ... when interleaved)."""
    name = "silu_mul"
    need_cuda(name, x, out)
    need(x.dim() == 2 and x.is_contiguous() and x.shape[1] % 2 == 0, name, "input must be contiguous [N, 2*inter]")
    n, inter = x.shape[0], x.shape[1] // 2
    if out is None:
        out = torch.empty((n, inter), dtype=x.dtype, device=x.device)
    need(out.shape == (n, inter) and out.dtype == x.dtype and out.is_contiguous(), name, "bad out tensor")
    check(lib().yalis_silu_mul(ptr(x), ptr(out), i32(dtype_code(x.dtype)), i32(n), i32(inter), i32(int(interleaved)),
                               stream()), name)
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    name = "gather_rows"
    need_cuda(name, x, rows)
    need(x.dtype == torch.float32 and x.dim() == 2 and x.is_contiguous(), name, "x must be float32 [N, width]")
    need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), name, "rows must be int32 [R]")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    check(lib().yalis_gather_rows_f32(ptr(x), ptr(rows), ptr(out), i32(rows.numel()), i32(x.shape[1]), stream()), name)
    return out
