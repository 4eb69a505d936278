"""y = x W^T for the projections of the model.

Two precisions, chosen by the operands' dtype:

* float32 operands: the SIMT kernel of csrc/gemm_simt.cu.  True 32-bit FMAs in
  a fixed order, no tensor cores, no TF32.
* bfloat16 operands: float32 accumulation on the tensor cores.  The engine's
  own tcgen05 kernels are used where they cover the shape; otherwise the
  product goes to cuBLAS through ``torch.matmul`` (the reference also leaves
  its projections to the library: ``nn.Linear``, yalis/external/model.py:449,
  462, 717, 720).
"""

from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, dtype_code, i32, i64, lib, need, need_cuda, ptr, stream


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
    """The projection used by the parts: picks the kernel by dtype (see module docstring)."""
    need_cuda("linear", x, w)
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        return gemm_simt(x, w, out_dtype)
    need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear", "operands must both be bfloat16 or float32")
    if out_dtype == torch.bfloat16:
        return torch.matmul(x, w.t())
    need(out_dtype == torch.float32, "linear", f"unsupported output dtype {out_dtype}")
    return torch.mm(x, w.t(), out_dtype=torch.float32)
