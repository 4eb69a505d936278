"""ctypes plumbing shared by the kernel wrappers.

Every wrapper checks its tensors on the host (device, dtype, contiguity,
shapes) before it hands raw pointers to the library, and raises
``KernelError`` when a launcher returns a non-zero status.  There is no
PyTorch or CPU fallback behind any wrapper: without the CUDA library the
import of a wrapper's first call fails with ``NativeBuildError``.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from yalis_b200 import native

F32, BF16 = 0, 1

_STATUS = {
    -1: "dtype not handled by this kernel",
    -2: "a size this kernel refuses",
    -3: "the launch failed (cudaGetLastError)",
    -4: "a pointer or stride is not aligned as the kernel needs",
    -5: "the problem exceeds the kernel's fixed scratch memory",
}


class KernelError(RuntimeError):
    pass


_configured = False


def lib() -> ctypes.CDLL:
    global _configured
    handle = native.load("cuda")
    if not _configured:
        _configured = True
        # Kernels are chained with programmatic dependent launch; YALIS_B200_NO_PDL=1 turns it off.
        handle.yalis_set_pdl(ctypes.c_int(0 if os.environ.get("YALIS_B200_NO_PDL", "0") == "1" else 1))
    return handle


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not supported (float32 and bfloat16 only)")


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle (asked thousands of times a step:
    the short way through torch's C module where it exists)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# ---- the device error word -----------------------------------------------------------------------
# One int32 per device that every kernel of the library may raise bits in (csrc/common.cuh) instead of trapping;
# the host reads it where it synchronises anyway.
FLAG_BAD_ID, FLAG_BAD_PAGE, FLAG_WAIT_ATTENTION, FLAG_WAIT_PRODUCT = 1, 2, 4, 8
_FLAG_TEXT = {
    FLAG_BAD_ID: "a token id outside the vocabulary",
    FLAG_BAD_PAGE: "a block-table entry outside the page pool (a visible token without a page)",
    FLAG_WAIT_ATTENTION: "a bounded wait inside an attention kernel ran out (its block gave up)",
    FLAG_WAIT_PRODUCT: "a bounded wait inside the weight-streaming product ran out (its block gave up)",
}
_error_words = {}


def error_word(device) -> torch.Tensor:
    """int32 [1] on ``device``: the error word every kernel launched through these wrappers reports to."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    word = _error_words.get(key)
    if word is None:
        word = _error_words[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return word


def describe_error_word(value: int) -> str:
    """What the bits of an error word mean, for messages."""
    found = [text for bit, text in _FLAG_TEXT.items() if value & bit]
    rest = value & ~sum(_FLAG_TEXT)
    if rest:
        found.append(f"unknown bits {rest:#x}")
    return "; ".join(found) if found else "no error"


LAUNCHES = [0]   # kernels of this library launched by this process (one per successful launcher call)


def check(status: int, name: str, detail: str = "") -> None:
    LAUNCHES[0] += 1
    if status != 0:
        why = _STATUS.get(status, f"status {status}")
        raise KernelError(f"{name}: {why}{(' (' + detail + ')') if detail else ''}")


def need(cond: bool, name: str, msg: str) -> None:
    if not cond:
        raise KernelError(f"{name}: {msg}")


def need_cuda(name: str, *tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(f"{name}: every tensor must be on the GPU (there is no CPU path)")


def i32(v: int) -> ctypes.c_int:
    return ctypes.c_int(int(v))


def i64(v: int) -> ctypes.c_longlong:
    return ctypes.c_longlong(int(v))


def f32(v: float) -> ctypes.c_float:
    return ctypes.c_float(float(v))
