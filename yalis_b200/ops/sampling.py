"""Wrappers of the token-selection kernels (csrc/sampling.cu)."""

from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, i32, i64, lib, need, need_cuda, ptr, stream


def _check_logits(name: str, logits: torch.Tensor) -> None:
    need_cuda(name, logits)
    need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, name,
         "logits must be float32 [rows, vocab] with unit inner stride")


def _check_scatter(name: str, rows: int, scatter_index, scatter) -> None:
    need((scatter_index is None) == (scatter is None), name, "scatter_index and scatter come together")
    if scatter is not None:
        need_cuda(name, scatter_index, scatter)
        need(scatter_index.dtype == torch.int32 and scatter_index.shape == (rows,) and scatter_index.is_contiguous()
             and scatter.dtype == torch.int32 and scatter.dim() == 1 and scatter.is_contiguous(), name,
             "scatter_index must be int32 [rows] and scatter a contiguous int32 vector")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, scatter_index: Optional[torch.Tensor] = None,
           scatter: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit of each row; ties go to the lowest index. int32 [rows].
    With ``scatter_index`` (int32 [rows]) the token of row i also goes to ``scatter[scatter_index[i]]`` where
    that index is not negative (the caller keeps the indices inside ``scatter``)."""
    name = "argmax"
    _check_logits(name, logits)
    _check_scatter(name, logits.shape[0], scatter_index, scatter)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    need(out.dtype == torch.int32 and out.shape == (rows,) and out.is_contiguous(), name, "bad out tensor")
    # wide rows are searched by 32 blocks each, then merged: needs a little scratch memory
    scratch = torch.empty((rows * 64,), dtype=torch.float32, device=logits.device) if vocab > 16384 else None
    check(lib().yalis_argmax(ptr(logits), i64(logits.stride(0)), i32(rows), i32(vocab), ptr(out), ptr(scratch),
                             ptr(scatter_index), ptr(scatter), stream()), name)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, draw_index: torch.Tensor, out: Optional[torch.Tensor] = None,
           scatter_index: Optional[torch.Tensor] = None, scatter: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row with per-row parameters (all device tensors of length rows).

    temperature float32, top_k int32 (0 = off), top_p float32, seed and draw_index
    int64 (read as unsigned).  A row with temperature 0 and top_p 0 is greedy.
    ``scatter_index`` / ``scatter`` as for ``argmax``.
    """
    name = "sample"
    _check_logits(name, logits)
    _check_scatter(name, logits.shape[0], scatter_index, scatter)
    rows, vocab = logits.shape
    need(vocab <= 1 << 19, name, f"rows of at most {1 << 19} logits are supported, got {vocab}")
    need_cuda(name, temperature, top_k, top_p, seed, draw_index, out)
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32), (seed, torch.int64),
                  (draw_index, torch.int64)):
        need(t.dtype == dt and t.shape == (rows,) and t.is_contiguous(), name, f"per-row parameter must be {dt} [rows]")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    need(out.dtype == torch.int32 and out.shape == (rows,) and out.is_contiguous(), name, "bad out tensor")
    scratch = torch.empty((rows * 68,), dtype=torch.float32, device=logits.device)   # partial draws and the cuts
    check(lib().yalis_sample(ptr(logits), i64(logits.stride(0)), i32(rows), i32(vocab), ptr(temperature), ptr(top_k),
                             ptr(top_p), ptr(seed), ptr(draw_index), ptr(out), ptr(scratch), ptr(scatter_index),
                             ptr(scatter), stream()), name)
    return out
