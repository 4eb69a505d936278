"""y = x W^T for the projections of the model.

Two precisions, chosen by the operands' dtype:

* float32 operands: the SIMT kernel of csrc/gemm_simt.cu.  True 32-bit FMAs in
  a fixed order, no tensor cores, no TF32.
* bfloat16 operands: float32 accumulation on the tensor cores.  Steps of up
  to 32 tokens (decode) go to the engine's own tcgen05 weight-streaming kernel,
  which takes up to 256 tokens but is the faster one only for few; larger
  steps go to cuBLAS through ``torch.matmul`` (the reference also leaves
  its projections to the library: ``nn.Linear``, yalis/external/model.py:449,
  462, 717, 720).
"""

from __future__ import annotations

from typing import Optional

import torch

import os

from ._lib import check, dtype_code, error_word, i32, i64, lib, need, need_cuda, ptr, stream

# YALIS_B200_NO_WSTREAM=1 sends every bfloat16 product to the library (for comparisons).
USE_WSTREAM = os.environ.get("YALIS_B200_NO_WSTREAM", "0") != "1"
# YALIS_B200_NO_FUSED_SILU=1 keeps the gated activation in its own kernel.
USE_FUSED_SILU = os.environ.get("YALIS_B200_NO_FUSED_SILU", "0") != "1"
FUSED_SILU_MAX_TOKENS = 16


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] . w [N, K]^T on the CUDA cores, float32 accumulation in k order."""
    name = "gemm_simt"
    need_cuda(name, x, w, out)
    need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], name,
         f"shapes {tuple(x.shape)} and {tuple(w.shape)} do not agree in K")
    need(x.stride(1) == 1 and w.stride(1) == 1, name, "operands must be K-contiguous")
    m, k = x.shape
    n = w.shape[0]
    out_dtype = out_dtype or x.dtype
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    need(out.shape == (m, n) and out.dtype == out_dtype and out.stride(1) == 1, name, "bad out tensor")
    check(lib().yalis_gemm_tn_simt(ptr(x), i32(dtype_code(x.dtype)), i64(x.stride(0)), ptr(w),
                                   i32(dtype_code(w.dtype)), i64(w.stride(0)), ptr(out), i32(dtype_code(out_dtype)),
                                   i64(out.stride(0)), i32(m), i32(n), i32(k), stream()), name)
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The projection used by the parts: picks the kernel by dtype and size (see module docstring)."""
    need_cuda("linear", x, w)
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32 or w.dtype == torch.float32:
        # the true 32-bit path, and a weight that its checkpoint stored in float32 (it stays so) under bfloat16 rows
        return gemm_simt(x, w, out_dtype)
    need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear", "operands must be bfloat16 or float32")
    if wstream_preferred(x, w):
        return gemm_wstream(x, w, out_dtype=out_dtype)
    if out_dtype == torch.bfloat16:
        return torch.matmul(x, w.t())
    need(out_dtype == torch.float32, "linear", f"unsupported output dtype {out_dtype}")
    return torch.mm(x, w.t(), out_dtype=torch.float32)


def linear_partial(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """A projection whose consumer can add partial sums: returns [M, N] in x's dtype, or
    float32 partial sums [S, M, N] when the weight-streaming kernel divides K among blocks."""
    if wstream_preferred(x, w) and wstream_splits(w.shape[0], w.shape[1]) > 1:
        return gemm_wstream(x, w, split=True)
    return linear(x, w)


# ---- the tcgen05 weight-streaming product (csrc/gemm_tcgen05.cu) -------------------------------

WSTREAM_MAX_TOKENS = 256        # what the kernel takes
# Up to this many tokens the engine's own kernel is the faster one in a decode step (measured on the Llama-3-8B
# shape: batch 32 4.20 ms against 4.36 ms with the library, batch 64 5.70 ms against 5.32 ms).
WSTREAM_PREFERRED_TOKENS = int(os.environ.get("YALIS_B200_WSTREAM_TOKENS", "32"))


def wstream_error_flag(device) -> torch.Tensor:
    """The device's error word: the kernel raises FLAG_WAIT_PRODUCT in it if one of its bounded waits ran out."""
    return error_word(device)


def wstream_splits(n: int, k: int) -> int:
    return int(lib().yalis_gemm_wstream_splits(i32(n), i32(k)))


def wstream_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """bfloat16, at most 256 tokens, K a multiple of 8 (16-byte rows for TMA), aligned bases."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and 0 < x.shape[0] <= WSTREAM_MAX_TOKENS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def wstream_preferred(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the projections of the parts send this product to the engine's own kernel."""
    return USE_WSTREAM and x.dtype == torch.bfloat16 and x.shape[0] <= WSTREAM_PREFERRED_TOKENS and wstream_supports(x, w)


def gemm_wstream(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 split: bool = False) -> torch.Tensor:
    """x [M <= 256, K] . w [N, K]^T on tcgen05 tensor cores with TMA-streamed weights.

    ``split=False``: returns [M, N] in ``out_dtype``.  ``split=True``: the K range may be
    divided among blocks (decided by the shape); returns float32 partial sums [S, M, N]
    that the consumer adds in order (S may be 1)."""
    name = "gemm_wstream"
    need_cuda(name, x, w)
    need(wstream_supports(x, w), name, "needs bfloat16, at most 256 tokens, K % 8 == 0, 16-byte aligned rows")
    need(x.shape[1] == w.shape[1], name, f"shapes {tuple(x.shape)} and {tuple(w.shape)} do not agree in K")
    m, k = x.shape
    n = w.shape[0]
    splits = wstream_splits(n, k) if split else 1
    if split:
        out = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
        code = dtype_code(torch.float32)
    else:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        code = dtype_code(out_dtype)
    check(lib().yalis_gemm_wstream(ptr(x), i64(x.stride(0)), ptr(w), i64(w.stride(0)), ptr(out), i32(code), i64(n),
                                   i32(m), i32(n), i32(k), i32(splits), ptr(wstream_error_flag(x.device)), stream()),
          name)
    return out


def gemm_wstream_silu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wgate^T) * (x . Wup^T) in one kernel: ``w_gate_up`` is [2 * inter, K] with the gate rows
    first.  Returns [M, inter] bfloat16 with the same bits as ``silu_mul(gemm_wstream(x, w_gate_up))``."""
    name = "gemm_wstream_silu"
    need_cuda(name, x, w_gate_up)
    need(wstream_supports(x, w_gate_up), name, "needs bfloat16, at most 256 tokens, K % 8 == 0, 16-byte aligned rows")
    need(x.shape[1] == w_gate_up.shape[1] and w_gate_up.shape[0] % 2 == 0, name,
         f"shapes {tuple(x.shape)} and {tuple(w_gate_up.shape)} do not fit a gate/up pair")
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    out = torch.empty((m, inter), dtype=torch.bfloat16, device=x.device)
    check(lib().yalis_gemm_wstream_silu(ptr(x), i64(x.stride(0)), ptr(w_gate_up), i64(w_gate_up.stride(0)), ptr(out),
                                        i64(inter), i32(m), i32(inter), i32(k), ptr(wstream_error_flag(x.device)),
                                        stream()), name)
    return out


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """The gated activation of a feed-forward: silu(gate) * up of the product with [Wgate; Wup];
    fused into the product where the weight-streaming kernel takes the shape."""
    from .elementwise import silu_mul
    # Measured on the Llama-3-8B shape: the fused epilogue wins up to 16 tokens (one chunk of tensor-memory
    # columns); from 17 on its blocks, heavier in registers and TMA requests, slow the products around it by more
    # than the activation kernel costs.
    if USE_FUSED_SILU and x.shape[0] <= FUSED_SILU_MAX_TOKENS and wstream_preferred(x, w_gate_up):
        return gemm_wstream_silu(x, w_gate_up)
    return silu_mul(linear(x, w_gate_up))
